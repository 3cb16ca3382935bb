"""Guzovik on the GPU: every new kernel alone against its reference at sizes other than any
model's, with inputs made so that a fault shows (a key just inside or just outside a window that
would carry all the weight, keys at page borders, NaN in pages that belong to nobody); the whole
model in float32 and bfloat16 against the plain implementation under every cut of the work; pages
used again; long decoding past the windows; greedy generation through ``LLM`` with recorded decode
steps; and ``bin/trace_run`` as a subprocess."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import kernel_refs as refs
import plain_guzovik as plain
import replay_cases as cases
from fegilix_cases import relative_error, run_steps
from guzovik_cases import CONFIGS, FakeCtx, assert_rows_close, random_config, write_model
from tiny_configs import random_prompt

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DTYPES = [torch.float32, torch.bfloat16]


def _rand(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()


def _tol(dtype):
    return {"atol": 2e-5, "rtol": 2e-5} if dtype == torch.float32 else {"atol": 2e-2, "rtol": 2e-2}


class Arena:
    def take(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device="cuda")


class Ctx(FakeCtx):
    def __init__(self, query_lens, context_lens):
        super().__init__(query_lens, context_lens, "cuda")
        self.arena = Arena()


# ------------------------------------------------------------ kernels one by one
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, hidden", [(1, 48), (37, 256), (5, 37), (300, 1024), (9, 4100)])
def test_norms_around_a_sub_layer_kernel(dtype, rows, hidden) -> None:
    from tinyserve_b200.kernels import ops

    x = _rand(rows, hidden, seed=1, scale=2.0)
    y = _rand(rows, hidden, seed=2, scale=3.0, dtype=dtype)
    wb, ls, w = (_rand(hidden, seed=s, scale=0.3, dtype=dtype) for s in (3, 4, 5))
    pick = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32, device="cuda")
    for delta, post, scale in [(y, wb, ls), (y, wb, None), (y, None, None), (None, None, None)]:
        got_x, want_x = x.clone(), x.clone()
        got, want = torch.empty(rows, hidden, dtype=dtype, device="cuda"), torch.empty(rows, hidden, dtype=dtype, device="cuda")
        ops.post_norm_add_rms_norm(got_x, delta, post, scale, 1e-5, True, w, True, 1e-6, got)
        refs.post_norm_add_rms_norm(want_x, delta, post, scale, 1e-5, True, w, True, 1e-6, want)
        torch.testing.assert_close(got_x, want_x, atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
        got3, want3 = torch.empty(3, hidden, dtype=dtype, device="cuda"), torch.empty(3, hidden, dtype=dtype, device="cuda")
        keep = x.clone()
        ops.post_norm_add_rms_norm(keep, delta, post, scale, 1e-5, True, w, False, 1e-6, got3, rows=pick)
        refs.post_norm_add_rms_norm(x.clone(), delta, post, scale, 1e-5, True, w, False, 1e-6, want3, rows=pick)
        assert torch.equal(keep, x), "chosen rows must leave the stream alone"
        torch.testing.assert_close(got3.float(), want3.float(), **_tol(dtype))


def _tables(lens: list[int], page: int, seed: int):
    """Block tables over shuffled pages (two spare pages stay NaN), as a device tensor and lists."""
    need = [-(-n // page) for n in lens]
    order = torch.randperm(sum(need) + 2, generator=torch.Generator().manual_seed(seed)).tolist()
    tables, at = [], 0
    for n in need:
        tables.append(order[at: at + n])
        at += n
    width = max(need)
    dev = torch.tensor([t + [0] * (width - len(t)) for t in tables], dtype=torch.int32, device="cuda")
    return tables, dev, sum(need) + 2


def _latent_case(dtype, heads, nope, rank, rot, rotary, page, lens, news, window, edge=None):
    """Two calls through the kernels and through the references: the earlier positions of every
    request, then its new tokens. ``edge = (gap, strength)``: the last query of request 0 and the key
    ``gap`` positions before it point the same way, strongly."""
    from tinyserve_b200.kernels import ops

    tables, table, pages = _tables(lens, page, 5)
    d = rank + rot
    stores = [torch.full((pages * page, d), float("nan"), dtype=dtype, device="cuda") for _ in range(2)]
    nw = (1 + _rand(rank, seed=1, scale=0.2)).to(dtype)
    res = None
    for phase, counts in enumerate(([n - m for n, m in zip(lens, news)], news)):
        starts = [0] * len(lens) if phase == 0 else [n - m for n, m in zip(lens, news)]
        live = [b for b, c in enumerate(counts) if c > 0]
        if not live:
            continue
        pos = torch.cat([torch.arange(starts[b], starts[b] + counts[b]) for b in live])
        t = len(pos)
        slots = torch.cat([torch.tensor([tables[b][p // page] * page + p % page for p in range(starts[b], starts[b] + counts[b])])
                           for b in live]).int().cuda()
        q_in = _rand(t, heads * (nope + rot), seed=10 + phase, dtype=dtype)
        folded = _rand(heads, t, rank, seed=20 + phase, dtype=dtype)
        ckr = _rand(t, d + 3, seed=30 + phase, dtype=dtype)[:, :d]        # rows of a wider matrix
        if edge is not None:
            gap, strength = edge
            target = lens[0] - 1 - gap
            rows = [i for i, p in enumerate(pos.tolist()) if i < counts[live[0]] and p == target and live[0] == 0]
            if rows:
                ckr[rows[0], :rank] = strength * (1 + torch.arange(rank, device="cuda") % 3).to(dtype)
            if phase == 1:
                # after the norm the marked latent is about (1, 2, 3, 1, ...) * weight / rms: the query follows it
                folded[:, counts[0] - 1] = (strength * (1 + torch.arange(rank, device="cuda") % 3)).to(dtype)
        angle = pos.double()[:, None] * (1e3 ** (-torch.arange(0, rotary, 2, dtype=torch.float64) / rotary))[None, :] if rotary else None
        cos = None if not rotary else angle.cos().float().cuda()
        sin = None if not rotary else angle.sin().float().cuda()
        ctx = Ctx([counts[b] for b in live], [starts[b] + counts[b] for b in live])
        tb = table[torch.tensor(live, device="cuda")].contiguous()
        res = []
        for impl, store in zip((ops, refs), stores):
            qo = torch.empty(t, heads, d, dtype=dtype, device="cuda")
            impl.latent_prepare(q_in, folded, ckr, nw, 1e-5, cos, sin, rotary, True, slots, store, heads, nope, rank, rot, qo)
            out = torch.empty(t, heads, rank, dtype=dtype, device="cuda")
            impl.latent_attention(qo, store, page, tb, ctx, rank, 0.2, window, out)
            res.append(out.float())
        res.append(counts)
    torch.testing.assert_close(stores[0].float(), stores[1].float(), equal_nan=True, **_tol(dtype))
    return res + [stores[1]]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, nope, rank, rot, rotary, page, window", [
    (3, 16, 20, 8, 4, 4, 5), (8, 64, 128, 16, 16, 16, 136), (1, 8, 12, 2, 2, 8, 0), (10, 24, 160, 32, 32, 16, 70),
    (4, 32, 300, 64, 48, 32, 33), (17, 16, 64, 0, 0, 16, 9)])
def test_latent_attention_kernels(dtype, heads, nope, rank, rot, rotary, page, window) -> None:
    """Prompt portions beside single decoded tokens, lengths around page borders."""
    lens, news = [page * 3 + 1, 70, page * 2, 33, 1, 200], [1, 17, 1, 33, 1, 2]
    got, want, *_ = _latent_case(dtype, heads, nope, rank, rot, rotary, page, lens, news, window)
    assert not got.isnan().any()
    torch.testing.assert_close(got, want, **_tol(dtype))


@pytest.mark.parametrize("lens, news, window", [([1500, 700, 64, 3000], [1, 1, 1, 1], 0), ([1500, 130], [1, 1], 1024),
                                                ([2100, 40, 900], [1, 40, 1], 300), ([5000], [1], 0), ([700, 300], [300, 130], 136)])
@pytest.mark.parametrize("heads, rank, rot", [(16, 512, 64), (8, 128, 16), (70, 64, 32)])
def test_latent_attention_on_the_tensor_cores_long_contexts(lens, news, window, heads, rank, rot) -> None:
    """bfloat16 at sizes the tensor-core form takes: single tokens with their keys cut into ranges and merged,
    prompt portions, more heads than a CTA's rows; against the reference and against the CUDA-core form."""
    from tinyserve_b200.kernels import ops

    got, want, *_ = _latent_case(torch.bfloat16, heads, 32, rank, rot, rot, 16, lens, news, window)
    assert not got.isnan().any()
    torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)
    ops.LATENT_TENSOR_CORES = False
    try:
        plain_cores, *_ = _latent_case(torch.bfloat16, heads, 32, rank, rot, rot, 16, lens, news, window)
    finally:
        ops.LATENT_TENSOR_CORES = True
    torch.testing.assert_close(got, plain_cores, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("new", [1, 2, 50])
@pytest.mark.parametrize("window", [16, 33, 100])
@pytest.mark.parametrize("rank, rot", [(32, 8), (64, 16)])
def test_latent_window_edges(dtype, new, window, rank, rot) -> None:
    """The key that matches the last query stands just inside the window (it carries the weight: the
    output is its latent) or just outside (it must not be seen), in a prompt portion and decoding."""
    heads, nope, page = 4, 16, 16
    for gap, inside in ((window - 1, True), (window, False)):
        got, want, counts, store = _latent_case(dtype, heads, nope, rank, rot, 8, page, [300, 40], [new, 1], window, edge=(gap, 6.0))
        torch.testing.assert_close(got, want, **_tol(dtype))
        row = counts[0] - 1
        tables, _, _ = _tables([300, 40], page, 5)
        p = 299 - gap
        latent = store[tables[0][p // page] * page + p % page, :rank].float()
        for h in range(heads):
            if inside:
                torch.testing.assert_close(got[row, h], latent, atol=3e-2, rtol=3e-2)
            else:
                assert (got[row, h] - latent).abs().max() > 0.3, "a key outside the window was seen"


def _window_case(dtype, heads, groups, d, dv, page, lens, news, window, edge=None):
    """The same for the attention with an added one in the denominator and a window."""
    from tinyserve_b200.kernels import ops

    tables, table, pages = _tables(lens, page, 7)
    caches = [(torch.full((pages, groups, page, d), float("nan"), dtype=dtype, device="cuda"),
               torch.full((pages, groups, page, dv), float("nan"), dtype=dtype, device="cuda")) for _ in range(2)]
    sinks = torch.zeros(heads, device="cuda")
    res = None
    for phase, counts in enumerate(([n - m for n, m in zip(lens, news)], news)):
        starts = [0] * len(lens) if phase == 0 else [n - m for n, m in zip(lens, news)]
        live = [b for b, c in enumerate(counts) if c > 0]
        if not live:
            continue
        pos = torch.cat([torch.arange(starts[b], starts[b] + counts[b]) for b in live])
        t = len(pos)
        slots = torch.cat([torch.tensor([tables[b][p // page] * page + p % page for p in range(starts[b], starts[b] + counts[b])])
                           for b in live]).int().cuda()
        q, k, v = (_rand(t, heads * d, seed=10 + phase, dtype=dtype), _rand(t, groups * d, seed=20 + phase, dtype=dtype),
                   _rand(t, groups * dv, seed=30 + phase, dtype=dtype))
        if edge is not None:
            gap, strength = edge
            target = lens[0] - 1 - gap
            rows = [i for i, p in enumerate(pos.tolist()) if i < counts[live[0]] and p == target and live[0] == 0]
            if rows:
                k[rows[0]] = strength
            if phase == 1:
                q[counts[0] - 1] = strength
        ctx = Ctx([counts[b] for b in live], [starts[b] + counts[b] for b in live])
        tb = table[torch.tensor(live, device="cuda")].contiguous()
        res = []
        for impl, (kc, vc) in zip((ops, refs), caches):
            qo = torch.empty(t, heads, d, dtype=dtype, device="cuda")
            impl.qkv_prepare(q, k, v, None, None, 0.0, None, None, 0, slots, kc, vc, page, heads, groups, d, dv, qo)
            out = torch.empty(t, heads * dv, dtype=dtype, device="cuda")
            impl.paged_attention(qo, kc, vc, page, tb, ctx, 0.3, window, out, sinks=sinks)
            res.append(out.float())
        res += [v, counts]
    return res


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, groups, d, dv, page, window", [
    (4, 2, 32, 16, 4, 7), (8, 1, 48, 48, 16, 96), (4, 2, 64, 64, 16, 40), (4, 4, 64, 64, 16, 33), (4, 1, 128, 128, 16, 100),
    (8, 2, 128, 128, 32, 1), (6, 3, 64, 64, 8, 200), (2, 2, 24, 40, 8, 19), (32, 1, 64, 64, 16, 100), (24, 1, 128, 128, 16, 60),
    (40, 2, 64, 64, 16, 0), (20, 1, 48, 48, 16, 96)])
def test_window_attention_with_an_added_one_kernels(dtype, heads, groups, d, dv, page, window) -> None:
    """CUDA-core kernels and, in bfloat16 at head sizes 64 / 128, the tensor-core prompt and decode kernels,
    with the fixed sink and a window together; prompt portions beside single tokens."""
    lens, news = [page * 3 + 1, 170, page * 2, 33, 1, 400], [1, 17, 1, 33, 1, 130]
    got, want, *_ = _window_case(dtype, heads, groups, d, dv, page, lens, news, window)
    assert not got.isnan().any()
    torch.testing.assert_close(got, want, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("new", [1, 2, 150])
@pytest.mark.parametrize("d, window", [(32, 16), (64, 33), (128, 96), (64, 128)])
def test_attention_window_edges(dtype, new, d, window) -> None:
    heads, groups, page = 4, 2, 16
    for gap, inside in ((window - 1, True), (window, False)):
        got, want, v, counts = _window_case(dtype, heads, groups, d, d, page, [500, 40], [new, 1], window, edge=(gap, 3.0))
        torch.testing.assert_close(got, want, **_tol(dtype))
        row = counts[0] - 1
        out = got[row].view(heads, d)
        if inside and gap < new:
            value = v[new - 1 - gap].float().view(groups, d)
            for h in range(heads):
                torch.testing.assert_close(out[h], value[h // (heads // groups)], atol=3e-2, rtol=3e-2)
        if not inside and gap < new:
            value = v[new - 1 - gap].float().view(groups, d)
            assert all((out[h] - value[h // (heads // groups)]).abs().max() > 0.3 for h in range(heads)), "a key outside the window was seen"


def test_the_added_one_takes_the_weight_on_the_device() -> None:
    from tinyserve_b200.kernels import ops

    for dtype, d in ((torch.float32, 32), (torch.bfloat16, 64), (torch.bfloat16, 48)):
        t, page = 40, 16
        q = torch.ones(t, 2, d, dtype=dtype, device="cuda")
        kc = torch.full((4, 1, page, d), -3.0, dtype=dtype, device="cuda")
        vc = torch.ones(4, 1, page, d, dtype=dtype, device="cuda")
        table = torch.tensor([[2, 0, 3]], dtype=torch.int32, device="cuda")
        out = torch.empty(t, 2 * d, dtype=dtype, device="cuda")
        ops.paged_attention(q, kc, vc, page, table, Ctx([t], [t]), 1.0, 0, out, sinks=torch.zeros(2, device="cuda"))
        assert out.float().abs().max() < 1e-6
        ops.paged_attention(q, -kc, vc, page, table, Ctx([t], [t]), 1.0, 0, out, sinks=torch.zeros(2, device="cuda"))
        torch.testing.assert_close(out.float(), torch.ones(t, 2 * d, device="cuda"), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_per_head_kernel(dtype) -> None:
    from tinyserve_b200.kernels import ops

    t, heads, w = 13, 5, 24
    x = _rand(t, heads, w, seed=1, dtype=dtype)
    proj = _rand(t, 40 + heads, seed=2, scale=2.0, dtype=dtype)
    got, want = torch.empty(t, heads * w, dtype=dtype, device="cuda"), torch.empty(t, heads * w, dtype=dtype, device="cuda")
    ops.head_norm_gate(x, None, False, proj[:, 40:], False, 0.0, got, gate_per_head=True)
    refs.head_norm_gate(x, None, False, proj[:, 40:], False, 0.0, want, gate_per_head=True)
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("rows, inter, k", [(3, 64, 128), (16, 512, 256), (40, 96, 64), (300, 1024, 256), (700, 2048, 512), (5, 20, 36)])
def test_clamped_feed_forward_products(rows, inter, k) -> None:
    """The clamped activation inside the few-row product, inside the tcgen05 product's epilogue, and as a
    kernel of its own behind a plain product; float32 too."""
    from tinyserve_b200.kernels import ops

    for dtype in DTYPES:
        x = _rand(rows, k, seed=1, dtype=dtype)
        w = _rand(2 * inter, k, seed=2, scale=2.0 / k ** 0.5, dtype=dtype)
        got, want = torch.empty(rows, inter, dtype=dtype, device="cuda"), torch.empty(rows, inter, dtype=dtype, device="cuda")
        ops.gemm_gated(x, w, got, Arena(), "clamped_swish", 1.5)
        refs.gemm_gated(x, w, want, None, "clamped_swish", 1.5)
        torch.testing.assert_close(got.float(), want.float(), atol=2e-5 if dtype == torch.float32 else 3e-2, rtol=2e-2)
        assert float(got.float().max()) <= 1.5 * 2.5 + 0.05        # g <= L, u + 1 <= L + 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, experts, top, hidden, ff, shared", [
    (1, 8, 3, 256, 64, True), (5, 5, 2, 48, 24, True), (300, 8, 3, 128, 64, False), (77, 3, 3, 64, 16, True),
    (513, 64, 6, 128, 96, False), (40, 2, 1, 36, 12, True), (9, 33, 32, 32, 8, False)])
def test_routed_expert_kernels(dtype, tokens, experts, top, hidden, ff, shared) -> None:
    from tinyserve_b200.kernels import ops

    logits = _rand(tokens, experts, seed=1, scale=2.0)
    logits[0, : min(3, experts)] = 1.25                      # a tie: the lower index wins
    counts = torch.zeros(experts, dtype=torch.int32, device="cuda")
    plan = ops.moe_route(logits, top, counts, Arena())
    want = refs.moe_route(logits, top, None)
    assert counts.abs().max() == 0, "the queue counters must be zero again"
    assert torch.equal(plan["ids"], want["ids"]) and torch.equal(plan["offsets"], want["offsets"])
    torch.testing.assert_close(plan["weights"], want["weights"])
    # the rows of an expert may stand in any order: every sorted row must belong to its expert, once
    token_of, row_of = plan["token_of"].long(), plan["row_of"].long()
    assert sorted(row_of.tolist()) == list(range(tokens * top))
    assert torch.equal(token_of[row_of], torch.arange(tokens * top, device="cuda") // top)
    expert_of_row = torch.bucketize(torch.arange(tokens * top, device="cuda"), plan["offsets"].long()[1:], right=True)
    assert torch.equal(expert_of_row[row_of], plan["ids"].long())
    tiles = int(plan["num_tiles"])
    assert tiles <= plan["max_tiles"] and tiles == sum(-(-int(c) // 64) for c in torch.bincount(plan["ids"].long(), minlength=experts))

    x = _rand(tokens, hidden, seed=2, dtype=dtype)
    w1 = _rand(experts, 2 * ff, hidden, seed=3, scale=hidden ** -0.5, dtype=dtype)
    w2 = _rand(experts, hidden, ff, seed=4, scale=ff ** -0.5, dtype=dtype)
    extra = _rand(tokens, hidden, seed=5, dtype=dtype) if shared else None
    outs = []
    for cores in ([True, False] if dtype == torch.bfloat16 else [False]):
        ops.MOE_TENSOR_CORES = cores
        try:
            act = torch.full((tokens * top, ff), float("nan"), dtype=dtype, device="cuda")
            y = torch.full((tokens * top, hidden), float("nan"), dtype=dtype, device="cuda")
            out = torch.empty(tokens, hidden, dtype=dtype, device="cuda")
            ops.moe_gemm(x, w1, act, plan, gated=True, gather=True)
            ops.moe_gemm(act, w2, y, plan, gated=False, gather=False)
            ops.moe_combine(y, plan, extra, out)
        finally:
            ops.MOE_TENSOR_CORES = True
        outs.append(out.float())
    act_r, y_r, out_r = (torch.empty(tokens * top, ff, dtype=dtype, device="cuda"), torch.empty(tokens * top, hidden, dtype=dtype, device="cuda"),
                         torch.empty(tokens, hidden, dtype=dtype, device="cuda"))
    refs.moe_gemm(x, w1, act_r, want, True, True)
    refs.moe_gemm(act_r, w2, y_r, want, False, False)
    refs.moe_combine(y_r, want, extra, out_r)
    for out in outs:
        assert not out.isnan().any()
        torch.testing.assert_close(out, out_r.float(), **_tol(dtype))


@pytest.mark.parametrize("tokens, experts, top, hidden, ff, skip", [
    (700, 4, 2, 256, 256, None), (2048, 16, 3, 1024, 768, 5), (1100, 3, 1, 512, 320, None), (600, 8, 8, 256, 1024, 0)])
def test_routed_experts_on_the_tcgen05_product(tokens, experts, top, hidden, ff, skip) -> None:
    """Steps of many rows: tiles of 128 sorted rows through the tcgen05 product, ragged experts, an expert
    that nobody picks, rows gathered first; against the reference and against the tiles of 64."""
    from tinyserve_b200.kernels import ops

    dtype = torch.bfloat16
    logits = _rand(tokens, experts, seed=1, scale=2.0)
    if skip is not None and top < experts:
        logits[:, skip] = -50.0
    counts = torch.zeros(experts, dtype=torch.int32, device="cuda")
    assert ops.moe_tile_rows(tokens, top, experts, dtype, (hidden, ff)) == 128
    x = _rand(tokens, hidden, seed=2, dtype=dtype)
    w1 = _rand(experts, 2 * ff, hidden, seed=3, scale=hidden ** -0.5, dtype=dtype)
    w2 = _rand(experts, hidden, ff, seed=4, scale=ff ** -0.5, dtype=dtype)
    outs = []
    for rows in (128, 64):
        plan = ops.moe_route(logits, top, counts, Arena(), rows)
        act = torch.full((tokens * top, ff), float("nan"), dtype=dtype, device="cuda")
        y = torch.full((tokens * top, hidden), float("nan"), dtype=dtype, device="cuda")
        out = torch.empty(tokens, hidden, dtype=dtype, device="cuda")
        ops.moe_gemm(x, w1, act, plan, gated=True, gather=True, arena=Arena())
        ops.moe_gemm(act, w2, y, plan, gated=False, gather=False, arena=Arena())
        ops.moe_combine(y, plan, None, out)
        ops.check_device_errors()
        outs.append(out.float())
    want = refs.moe_route(logits, top, None)
    act_r, y_r, out_r = (torch.empty(tokens * top, ff, dtype=dtype, device="cuda"), torch.empty(tokens * top, hidden, dtype=dtype, device="cuda"),
                         torch.empty(tokens, hidden, dtype=dtype, device="cuda"))
    refs.moe_gemm(x, w1, act_r, want, True, True)
    refs.moe_gemm(act_r, w2, y_r, want, False, False)
    refs.moe_combine(y_r, want, None, out_r)
    for out in outs:
        assert not out.isnan().any()
        torch.testing.assert_close(out, out_r.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, experts, top, hidden", [(1, 8, 3, 256), (8, 16, 3, 1024), (64, 5, 2, 36), (9, 33, 4, 40), (300, 8, 2, 128), (4, 700, 8, 64)])
def test_router_inside_the_routing_kernel(dtype, tokens, experts, top, hidden) -> None:
    """Small steps can form the router's logits in the CTA that routes; larger ones go through the product.
    Both pick what the reference picks (the inputs are made so that no two logits of a token lie close)."""
    from tinyserve_b200.kernels import ops

    for work in (1 << 22, 0):
        ops.MOE_ROUTE_FUSED_MAX_WORK = work
        try:
            _router_case(ops, dtype, tokens, experts, top, hidden)
        finally:
            ops.MOE_ROUTE_FUSED_MAX_WORK = 0


def _router_case(ops, dtype, tokens, experts, top, hidden) -> None:
    x = _rand(tokens, hidden, seed=1, dtype=dtype)
    w = _rand(experts, hidden, seed=2, dtype=dtype)
    w[:, 0] += (torch.arange(experts, device="cuda") * 0.7).to(dtype)        # spread the logits apart
    x[:, 0] = 3.0
    counts = torch.zeros(experts, dtype=torch.int32, device="cuda")
    plan = ops.moe_route_from(x, w, top, counts, Arena())
    want = refs.moe_route_from(x, w, top, None)
    assert torch.equal(plan["ids"], want["ids"]) and torch.equal(plan["offsets"], want["offsets"])
    torch.testing.assert_close(plan["weights"], want["weights"], atol=2e-3, rtol=2e-3)
    assert sorted(plan["row_of"].tolist()) == list(range(tokens * top)) and counts.abs().max() == 0


def test_a_token_alone_and_in_a_crowd_takes_the_same_experts_path() -> None:
    """float32: a row's sums do not depend on what shares its tile."""
    from tinyserve_b200.kernels import ops

    experts, top, hidden, ff = 4, 2, 64, 32
    x = _rand(200, hidden, seed=1)
    router, w1, w2 = _rand(experts, hidden, seed=2), _rand(experts, 2 * ff, hidden, seed=3, scale=0.1), _rand(experts, hidden, ff, seed=4, scale=0.1)
    counts = torch.zeros(experts, dtype=torch.int32, device="cuda")

    def run(rows):
        logits = torch.empty(rows.shape[0], experts, device="cuda")
        ops.gemm(rows, router, logits)
        plan = ops.moe_route(logits, top, counts, Arena())
        act, y = torch.empty(rows.shape[0] * top, ff, device="cuda"), torch.empty(rows.shape[0] * top, hidden, device="cuda")
        out = torch.empty(rows.shape[0], hidden, device="cuda")
        ops.moe_gemm(rows, w1, act, plan, gated=True, gather=True)
        ops.moe_gemm(act, w2, y, plan, gated=False, gather=False)
        ops.moe_combine(y, plan, None, out)
        return out

    crowd = run(x)
    assert torch.equal(run(x[17:18].contiguous())[0], crowd[17]) and torch.equal(run(x[150:153].contiguous())[1], crowd[151])


# ------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {k: write_model(tmp_path_factory.mktemp("guzovik" + k), k) for k in CONFIGS}


LENGTHS = {"A": [1, 2, 9, 37, 70, 131], "B": [3, 33, 64, 97, 150], "C": [5, 18, 40, 150], "D": [2, 47, 160, 330]}


@pytest.fixture(scope="module")
def oracle(folders):
    out = {}
    for which in CONFIGS:
        cfg, w = plain.read_config(folders[which]), plain.read_weights(folders[which], torch.float64)
        reqs = {f"r{i}": random_prompt(n, cfg["vocab"], 200 + 7 * i) for i, n in enumerate(LENGTHS[which])}
        out[which] = (reqs, {rid: plain.forward(cfg, w, toks).float() for rid, toks in reqs.items()})
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which, page", [("A", 4), ("A", 16), ("B", 8), ("B", 16), ("C", 16), ("C", 32), ("D", 16), ("D", 8)])
def test_model_under_every_cut(folders, oracle, dtype, which, page) -> None:
    from tinyserve_b200.model import DecoderModel

    reqs, want = oracle[which]
    model = DecoderModel.from_folder(folders[which], dtype, "cuda")
    plans = [cases.mixed(reqs, 3), cases.mixed(reqs, 4, max_live=2)]
    for rid, toks in reqs.items():
        plans += [cases.whole(rid, toks), cases.tail_decoded(rid, toks, 32), cases.portions(rid, toks, 1)]
    for n, steps in enumerate(plans):
        got, _ = run_steps(model, page, steps, cases.max_live_tokens(steps))
        assert all(sorted(got[rid]) == list(range(len(reqs[rid]))) for rid in got)
        rows = torch.cat([torch.stack([got[rid][p] for p in range(len(reqs[rid]))]) for rid in got])
        assert_rows_close(rows, torch.cat([want[rid] for rid in got]), dtype, f"{which}, schedule {n}")


@pytest.mark.parametrize("seed", list(range(1, 13)))
def test_configurations_drawn_at_random(seed, tmp_path) -> None:
    """Sizes, head counts, windows, layer order, shared tensors, feed-forward kinds and constants drawn at
    random; a prompt alone, decoded token by token, and mixed with others. float32 must equal the oracle.
    bfloat16 is a sanity check here: with wide random weights some of these models amplify rounding (several
    routed layers in a row, one expert of seven), the CUDA-core kernels on the same bfloat16 values land at the
    same distance from the oracle, so the rows must only stay in the oracle's neighbourhood, and the same
    prompt fed whole and decoded token by token must land at the same distance."""
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.model import DecoderModel
    from tinyserve_b200.weights import write_random_model

    cfg = random_config(seed)
    folder = write_random_model(tmp_path, config_from_dict(cfg), seed, torch.bfloat16, std_scale=6.0)
    w = plain.read_weights(folder, torch.float64)
    reqs = {f"r{i}": random_prompt(n, cfg["vocab"], 300 + seed + 7 * i) for i, n in enumerate([2, 35, 260, 121])}
    want = {rid: plain.forward(cfg, w, toks).float() for rid, toks in reqs.items()}
    page = [4, 8, 16, 32][seed % 4]
    plans = [cases.mixed(reqs, seed), cases.whole("r2", reqs["r2"]), cases.tail_decoded("r2", reqs["r2"], 40), cases.portions("r3", reqs["r3"], seed)]
    from guzovik_cases import row_errors

    for dtype in DTYPES:
        model = DecoderModel.from_folder(folder, dtype, "cuda")
        medians = []
        for n, steps in enumerate(plans):
            got, _ = run_steps(model, page, steps, cases.max_live_tokens(steps))
            rows = torch.cat([torch.stack([got[rid][p] for p in range(len(reqs[rid]))]) for rid in got])
            oracle_rows = torch.cat([want[rid] for rid in got])
            what = f"seed {seed}, schedule {n}: {json.dumps(cfg)[:300]}"
            if dtype == torch.float32:
                # a model that amplifies bfloat16 rounding to a tenth of the logits' spread amplifies 32-bit rounding too
                assert_rows_close(rows, oracle_rows, dtype, what, limit32=1e-4)
                continue
            assert not rows.isnan().any(), what
            medians.append(float(row_errors(rows, oracle_rows).median()))
            assert medians[-1] < 0.25, f"{what}: median relative error {medians[-1]:.3g}"
        if medians:
            assert abs(medians[1] - medians[2]) <= 0.25 * max(medians[1], 1e-3), f"seed {seed}: whole {medians[1]:.3g}, decoded {medians[2]:.3g}"


def test_model_with_its_experts_on_the_tcgen05_product(folders, oracle) -> None:
    """The thresholds lowered so that the small model's prompt portions take the tiles of 128 rows."""
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.model import DecoderModel

    reqs, want = oracle["D"]
    model = DecoderModel.from_folder(folders["D"], torch.bfloat16, "cuda")
    saved = ops.MOE_TCGEN05_MIN_ROWS, ops.MOE_TCGEN05_MIN_COLS
    ops.MOE_TCGEN05_MIN_ROWS, ops.MOE_TCGEN05_MIN_COLS = 256, 64
    try:
        assert ops.moe_tile_rows(330, 2, 4, torch.bfloat16, (128, 64)) == 128
        for steps in (cases.whole("r3", reqs["r3"]), cases.mixed(reqs, 3)):
            got, _ = run_steps(model, 16, steps, cases.max_live_tokens(steps))
            rows = torch.cat([torch.stack([got[rid][p] for p in range(len(reqs[rid]))]) for rid in got])
            assert_rows_close(rows, torch.cat([want[rid] for rid in got]), torch.bfloat16, "D")
    finally:
        ops.MOE_TCGEN05_MIN_ROWS, ops.MOE_TCGEN05_MIN_COLS = saved


def test_batch_mates_and_pages_do_not_matter(folders, oracle) -> None:
    """float32: a request's logits alone, beside others, and again on the pages that another request
    has just given back, agree to rounding."""
    from tinyserve_b200.engine.replay import Replayer
    from tinyserve_b200.model import DecoderModel

    reqs, _ = oracle["A"]
    model = DecoderModel.from_folder(folders["A"], torch.float32, "cuda")
    toks, other = reqs["r4"], reqs["r5"]
    rep = Replayer(model, 256, page_size=4, max_live=2)
    alone = rep.run_step([("x", toks, [len(toks) - 1])], ["x"]).clone()
    rep.run_step([("y", other[:50], [])], [])
    beside = rep.run_step([("y", other[50:51], []), ("x", toks, [len(toks) - 1])], ["x", "y"]).clone()
    again = rep.run_step([("z", toks[:7], []), ("w", other[:3], [])], [])
    again = rep.run_step([("w", other[3:4], []), ("z", toks[7:], [len(toks) - 8])], ["z", "w"]).clone()
    torch.testing.assert_close(beside, alone, atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(again, alone, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["B", "D"])
def test_long_decoding_past_the_windows(folders, dtype, which) -> None:
    from tinyserve_b200.model import DecoderModel

    cfg, w = plain.read_config(folders[which]), plain.read_weights(folders[which], torch.float64)
    toks = random_prompt(260, cfg["vocab"], 9)
    want = plain.forward(cfg, w, toks).float()
    model = DecoderModel.from_folder(folders[which], dtype, "cuda")
    got, _ = run_steps(model, 16, cases.tail_decoded("a", toks, 255), 320)
    rows = torch.stack([got["a"][p] for p in range(260)])
    assert_rows_close(rows[-20:], want[-20:], dtype, "the last decoded tokens")
    assert_rows_close(rows, want, dtype, "all tokens")


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("which", ["A", "D"])
def test_greedy_generation_through_llm(folders, graphs, which) -> None:
    from tinyserve_b200 import LLM

    cfg, w = plain.read_config(folders[which]), plain.read_weights(folders[which], torch.float64)
    prompts = [random_prompt(n, cfg["vocab"], 40 + n) for n in (3, 11, 26, 50)]
    want = [plain.greedy(cfg, w, p, 8) for p in prompts]
    llm = LLM.from_folder(folders[which], dtype="float32", page_size=8, num_pages=64, max_num_seqs=3, max_batch_tokens=32,
                          chunked_prefill=True, decode_graphs=graphs)
    assert llm.generate(prompts, max_new_tokens=8) == want
    assert (llm.engine.runner.num_graph_steps > 0) == graphs
    assert all(g.allocator.num_used == 0 for g in llm.cache.groups)


def test_command_line(folders) -> None:
    cfg, w = plain.read_config(folders["A"]), plain.read_weights(folders["A"], torch.float64)
    prompt = random_prompt(19, cfg["vocab"], 77)
    want = plain.greedy(cfg, w, prompt, 8)
    cmd = [sys.executable, str(ROOT / "bin" / "generate"), "--model-dir", str(folders["A"]), "--prompt-ids", ",".join(map(str, prompt)),
           "--max-new-tokens", "8", "--dtype", "float32", "--block-size", "8"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert f"new ids:    {want}" in out.stdout
    out = subprocess.run(cmd + ["--temperature", "0.8", "--top-p", "0.9", "--seed", "3", "--num-samples", "2"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "2 samples, 16 tokens" in out.stdout, out.stdout + out.stderr[-1000:]


def test_trace_run_subprocess(folders, oracle, tmp_path) -> None:
    reqs, want = oracle["C"]
    steps = cases.mixed(reqs, 6, max_live=3)
    lines = [json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": p} for r, t, p in entries], "end": end})
             for i, (entries, end) in enumerate(steps)]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders["C"]), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", str(cases.max_live_tokens(steps))],
                          input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [x for x in proc.stdout.split("\n") if x.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    fed: dict[str, int] = {}
    for i, (entries, _) in enumerate(steps):
        rows = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, 61))
        at = 0
        for rid, toks, places in entries:
            base = fed.get(rid, 0)
            for p in places:
                assert relative_error(rows[at], want[rid][base + p]) < 2e-5
                at += 1
            fed[rid] = base + len(toks)
