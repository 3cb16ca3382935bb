"""Fegilix on the GPU: every new kernel alone against its reference at sizes other than any
model's, with inputs made so that a fault shows (a far key that carries all the weight, keys at
page borders, NaN in pages and slots that belong to nobody); the whole model in float32 and
bfloat16 against the plain implementation under every cut of the work; slots and pages used
again; long decoding; greedy generation through ``LLM`` with recorded decode steps; and
``bin/trace_run`` as a subprocess."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import kernel_refs as refs
import plain_fegilix as plain
import replay_cases as cases
from fegilix_cases import CONFIGS, FakeStep, assert_close, relative_error, run_steps, write_model
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


# ------------------------------------------------------------ kernels one by one
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lanes, hidden", [(1, 48), (2, 256), (4, 100), (8, 64)])
def test_hyper_connection_kernels(dtype, lanes, hidden) -> None:
    from tinyserve_b200.kernels import ops

    t = 37
    x0, nw = _rand(t, hidden, seed=1), (1 + _rand(hidden, seed=2, scale=0.1)).to(dtype)
    w = [_rand(lanes, seed=3), _rand(lanes, seed=4), _rand(lanes, lanes, seed=5), _rand(lanes, seed=6)]
    y = _rand(t, hidden, seed=7, dtype=dtype)
    got_l, want_l = torch.full((lanes, t, hidden), float("nan"), device="cuda"), torch.zeros(lanes, t, hidden, device="cuda")
    got, want = torch.empty(t, hidden, dtype=dtype, device="cuda"), torch.empty(t, hidden, dtype=dtype, device="cuda")
    for fresh, delta, mix, out_w, in_w in [(x0, None, None, None, w[0]), (None, y, w[2], w[1], w[3]), (None, None, None, None, w[0])]:
        ops.hc_mix_norm(got_l, fresh, delta, mix, out_w, in_w, nw, 1e-5, got)
        refs.hc_mix_norm(want_l, fresh, delta, mix, out_w, in_w, nw, 1e-5, want)
        torch.testing.assert_close(got_l, want_l, atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
    rows = torch.tensor([36, 0, 5], dtype=torch.int32, device="cuda")
    for r in (rows, None):
        n = t if r is None else 3
        a, b = torch.empty(n, hidden, device="cuda"), torch.empty(n, hidden, device="cuda")
        ops.hc_collapse(got_l, None, y, w[2], w[1], r, a)
        refs.hc_collapse(want_l, None, y, w[2], w[1], r, b)
        torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-5)
    a, b = torch.empty(3, hidden, device="cuda"), torch.empty(3, hidden, device="cuda")
    ops.hc_collapse(got_l, x0, None, None, None, rows, a)
    refs.hc_collapse(want_l, x0, None, None, None, rows, b)
    torch.testing.assert_close(a, b)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_kernels(dtype) -> None:
    from tinyserve_b200.kernels import ops

    for act in ("gelu_tanh", "silu"):
        gu = _rand(19, 2 * 72, seed=1, scale=2.0, dtype=dtype)
        a, b = torch.empty(19, 72, dtype=dtype, device="cuda"), torch.empty(19, 72, dtype=dtype, device="cuda")
        ops.act_mul(gu, a, act)
        refs.act_mul(gu, b, act)
        torch.testing.assert_close(a.float(), b.float(), **_tol(dtype))
    lg = _rand(5, 301, seed=2, scale=30.0)
    want = lg.clone()
    ops.softcap(lg, 12.5)
    refs.softcap(want, 12.5)
    torch.testing.assert_close(lg, want, atol=1e-5, rtol=1e-5)
    for heads, width, per_head, normalise, f32_in in [(3, 48, True, True, True), (6, 64, False, True, True), (5, 40, None, False, False)]:
        x = _rand(11, heads, width, seed=3, dtype=torch.float32 if f32_in else dtype)
        weight = None if per_head is None else (1 + _rand(heads * width if per_head else width, seed=4, scale=0.1)).to(dtype)
        wide = _rand(11, 2 * heads * width, seed=5, dtype=dtype)
        gate = wide[:, heads * width:]                    # a column slice of a wider product
        a, b = torch.empty(11, heads * width, dtype=dtype, device="cuda"), torch.empty(11, heads * width, dtype=dtype, device="cuda")
        ops.head_norm_gate(x, weight, bool(per_head), gate, normalise, 1e-5, a)
        refs.head_norm_gate(x, weight, bool(per_head), gate, normalise, 1e-5, b)
        torch.testing.assert_close(a.float(), b.float(), **_tol(dtype))


@pytest.mark.parametrize("m, inter, k", [(3, 96, 64), (8, 3072, 1024), (16, 1024, 512), (40, 200, 72), (300, 3072, 1024), (2048, 3072, 1024)])
def test_gated_product_with_gelu(m, inter, k) -> None:
    """The three routes of the gate/up product with the tanh form of GELU (skinny, tcgen05 epilogue,
    product + activation kernel), chosen by the shape, against the reference."""
    from tinyserve_b200.kernels import ops

    x, w = _rand(m, k, seed=1, dtype=torch.bfloat16), _rand(2 * inter, k, seed=2, scale=k ** -0.5, dtype=torch.bfloat16)
    got, want = torch.empty(m, inter, dtype=torch.bfloat16, device="cuda"), torch.empty(m, inter, dtype=torch.bfloat16, device="cuda")
    ops.gemm_gated(x, w, got, Arena(), "gelu_tanh")
    ops.check_device_errors()
    refs.gemm_gated(x, w, want, None, "gelu_tanh")
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    x32, w32 = x.float(), w.float()
    got32, want32 = torch.empty(m, inter, device="cuda"), torch.empty(m, inter, device="cuda")
    ops.gemm_gated(x32, w32, got32, Arena(), "gelu_tanh")
    refs.gemm_gated(x32, w32, want32, None, "gelu_tanh")
    torch.testing.assert_close(got32, want32, atol=2e-5, rtol=2e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps, channels", [(1, 40), (2, 96), (4, 384), (8, 33)])
def test_causal_conv_carries_its_state(dtype, taps, channels) -> None:
    from tinyserve_b200.kernels import ops

    lens1, lens2, slots = [5, 1, 2, 9], [1, 3, 1, 2], [4, 0, 2, 1]
    width = 7 + (taps - 1) * channels                    # the conv state is a column range of a wider slot
    got = torch.zeros(6, width, device="cuda")
    want = got.clone()
    w_taps = _rand(channels, taps, seed=1, scale=0.5, dtype=dtype)
    for i, lens in enumerate((lens1, lens2)):
        step = FakeStep(lens, slots, "cuda")
        x = _rand(sum(lens), channels, seed=10 + i, dtype=dtype)
        a, b = torch.empty(sum(lens), channels, device="cuda"), torch.empty(sum(lens), channels, device="cuda")
        ops.causal_conv_silu(x, w_taps, got[:, 7:], step, a)
        refs.causal_conv_silu(x, w_taps, want[:, 7:], step, b)
        torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-6)
    assert got[3].abs().max() == 0 and got[5].abs().max() == 0 and got[:, :7].abs().max() == 0


@pytest.mark.parametrize("heads, groups, d, dv", [(4, 2, 16, 32), (2, 2, 40, 24), (3, 1, 64, 80), (1, 1, 128, 128), (2, 1, 200, 16)])
def test_delta_scan_kernel(heads, groups, d, dv) -> None:
    from tinyserve_b200.kernels import ops

    qk, lens_a, lens_b, slots = groups * d, [7, 1, 19], [1, 4, 1], [2, 5, 0]
    size = heads * d * dv
    got, want = torch.zeros(7, size + 5, device="cuda"), torch.zeros(7, size + 5, device="cuda")
    bias, a_log = _rand(heads * d, seed=1), _rand(heads, seed=2, scale=0.3)
    for i, lens in enumerate((lens_a, lens_b)):
        t, step = sum(lens), FakeStep(lens, slots, "cuda")
        x, a, beta = _rand(t, 2 * qk + heads * dv, seed=20 + i), _rand(t, heads * d, seed=30 + i), _rand(t, heads, seed=40 + i)
        o1, o2 = torch.empty(t, heads, dv, device="cuda"), torch.empty(t, heads, dv, device="cuda")
        ops.delta_scan(x, 0, qk, 2 * qk, a, bias, a_log, beta, d ** -0.5, got[:, :size], step, heads, groups, d, dv, o1)
        refs.delta_scan(x, 0, qk, 2 * qk, a, bias, a_log, beta, d ** -0.5, want[:, :size], step, heads, groups, d, dv, o2)
        torch.testing.assert_close(o1, o2, atol=2e-5, rtol=2e-4)
        torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-4)
    assert got[1].abs().max() == 0 and got[:, size:].abs().max() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, d, dv", [(2, 48, 48), (3, 16, 40), (1, 128, 64), (2, 72, 100), (1, 256, 32)])
def test_mlstm_scan_kernel(dtype, heads, d, dv) -> None:
    from tinyserve_b200.kernels import ops

    lens_a, lens_b, slots = [6, 1, 23], [1, 2, 1], [1, 3, 0]
    size = ops.mlstm_state_size(heads, d, dv)
    assert size == refs.mlstm_state_size(heads, d, dv)
    got, want = torch.zeros(5, size, device="cuda"), torch.zeros(5, size, device="cuda")
    gb = _rand(2 * heads, seed=1)
    for i, lens in enumerate((lens_a, lens_b)):
        t, step = sum(lens), FakeStep(lens, slots, "cuda")
        wide = _rand(t, 9 + 2 * heads * d + heads * dv, seed=20 + i, dtype=dtype)      # q, k, v at column offsets
        gates = _rand(t, 2 * heads, seed=30 + i, scale=4.0)
        o1, o2 = torch.empty(t, heads, dv, device="cuda"), torch.empty(t, heads, dv, device="cuda")
        ops.mlstm_scan(wide, 9, 9 + heads * d, 9 + 2 * heads * d, gates, gb, 5.0, d ** -0.5, got, step, heads, d, dv, o1)
        refs.mlstm_scan(wide, 9, 9 + heads * d, 9 + 2 * heads * d, gates, gb, 5.0, d ** -0.5, want, step, heads, d, dv, o2)
        torch.testing.assert_close(o1, o2, atol=2e-5, rtol=2e-4)
        torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-4)
    assert got[2].abs().max() == 0 and got[4].abs().max() == 0


def _attention_case(dtype, heads, groups, d, dv, page, lens, news, rot, sink_shift=0.0, far=None):
    """Requests with ``lens`` tokens of which the last ``news`` are this step's; the earlier ones are
    already in the cache (written by a first call). Returns kernel and reference outputs of the step."""
    from tinyserve_b200.kernels import ops

    total_pages = sum(-(-n // page) for n in lens) + 3
    perm = torch.randperm(total_pages, generator=torch.Generator().manual_seed(5)).tolist()
    tables, at = [], 0
    for n in lens:
        k = -(-n // page)
        tables.append(perm[at: at + k])
        at += k
    width = max(len(x) for x in tables)
    table = torch.tensor([x + [0] * (width - len(x)) for x in tables], dtype=torch.int32, device="cuda")
    caches = []
    for _ in range(2):
        caches.append((torch.full((total_pages, groups, page, d), float("nan"), dtype=dtype, device="cuda"),
                       torch.full((total_pages, groups, page, dv), float("nan"), dtype=dtype, device="cuda")))
    qw, kw = (1 + _rand(d, seed=1, scale=0.2)).to(dtype), (1 + _rand(d, seed=2, scale=0.2)).to(dtype)
    sinks = _rand(heads, seed=3) + sink_shift
    outs = []
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
        if far is not None:
            # one key of request 0 and this step's last query of request 0 point the same way, strongly:
            # that key must carry nearly all the weight of every head
            req_pos, strength = far
            row = [i for i, p in enumerate(pos.tolist()) if i < counts[live[0]] and p == req_pos]
            if phase == 0 and row:
                k[row[0]] = strength
            if phase == 1:
                q[counts[live[0]] - 1] = strength
        angle = pos.double()[:, None] * (1e4 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot))[None, :] if rot else None
        cos = None if rot == 0 else angle.cos().float().cuda()
        sin = None if rot == 0 else angle.sin().float().cuda()

        class Ctx:
            num_seqs = len(live)
            query_lens = [counts[b] for b in live]
            context_lens = [starts[b] + counts[b] for b in live]
            cu_query_lens = torch.tensor([0] + np.cumsum([counts[b] for b in live]).tolist(), dtype=torch.int32, device="cuda")
            context_lens_dev = torch.tensor([starts[b] + counts[b] for b in live], dtype=torch.int32, device="cuda")
            decode_seqs = torch.tensor([i for i, b in enumerate(live) if counts[b] == 1] or [0], dtype=torch.int32, device="cuda")
            prefill_seqs = torch.tensor([i for i, b in enumerate(live) if counts[b] > 1] or [0], dtype=torch.int32, device="cuda")
            num_decode = sum(1 for b in live if counts[b] == 1)
            num_prefill = sum(1 for b in live if counts[b] > 1)
            max_query_len = max(counts[b] for b in live)
            max_context_len = max(starts[b] + counts[b] for b in live)
            arena = Arena()

        tb = table[torch.tensor(live, device="cuda")].contiguous()
        res = []
        for impl, (kc, vc) in zip((ops, refs), caches):
            qo = torch.empty(t, heads, d, dtype=dtype, device="cuda")
            impl.qkv_prepare(q, k, v, qw, kw, 1e-5, cos, sin, rot, slots, kc, vc, page, heads, groups, d, dv, qo)
            out = torch.empty(t, heads * dv, dtype=dtype, device="cuda")
            impl.paged_attention(qo, kc, vc, page, tb, Ctx, 0.3, 0, out, sinks=sinks)
            res.append(out.float())
        outs = res + [v, counts, live]
    return outs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, groups, d, dv, page, rot", [(4, 2, 32, 16, 4, 16), (6, 6, 128, 128, 16, 64), (3, 1, 24, 40, 8, 0),
                                                              (2, 2, 64, 64, 16, 64), (8, 2, 48, 80, 32, 12), (8, 2, 64, 64, 16, 32),
                                                              (8, 4, 128, 128, 16, 128), (12, 2, 128, 128, 32, 64), (4, 1, 64, 64, 8, 0),
                                                              (2, 1, 256, 256, 16, 64), (2, 2, 192, 96, 16, 192)])
def test_sink_attention_kernels(dtype, heads, groups, d, dv, page, rot) -> None:
    """Prompt portions beside single decoded tokens, lengths around page borders."""
    lens, news = [page * 3 + 1, 70, page * 2, 33, 1], [1, 17, 1, 33, 1]
    got, want, *_ = _attention_case(dtype, heads, groups, d, dv, page, lens, news, rot)
    assert not got.isnan().any()
    torch.testing.assert_close(got, want, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far_pos, new", [(3, 1), (15, 1), (16, 1), (250, 40), (0, 300)])
def test_a_far_key_carries_the_weight(dtype, far_pos, new) -> None:
    """Among hundreds of keys one, far back (also the first of a page and the last of the one
    before), matches the last query: every head's output is that key's value."""
    heads, groups, d, dv, page = 4, 2, 32, 48, 16
    got, want, v, counts, live = _attention_case(dtype, heads, groups, d, dv, page, [600, 20], [new, 1], 0, far=(far_pos, 4.0))
    torch.testing.assert_close(got, want, **_tol(dtype))
    if new < 600 - far_pos:      # the far key was written by the first call
        return
    row = counts[0] - 1
    value = v[[i for i in range(counts[0]) if 600 - new + i == far_pos][0]].float().view(groups, dv)
    out = got[row].view(heads, dv)
    for h in range(heads):
        torch.testing.assert_close(out[h], value[h // (heads // groups)], atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("lens, news", [([1500, 700, 64, 3000], [1, 1, 1, 1]), ([1500, 130], [300, 130]), ([2100, 40, 900], [1, 40, 1])])
@pytest.mark.parametrize("heads, groups, d", [(8, 2, 128), (4, 4, 64), (16, 2, 64)])
def test_sink_attention_on_the_tensor_cores_long_contexts(lens, news, heads, groups, d) -> None:
    """bfloat16 with equal key and value sizes of 64 / 128: the tcgen05 prompt kernel and the TMA decode kernel
    (key ranges merged inside a cluster or by the last arriver) with sink logits, grouped heads and long contexts;
    the last query of request 0 matches one key far back."""
    got, want, *_ = _attention_case(torch.bfloat16, heads, groups, d, d, 16, lens, news, d // 2, far=(37, 3.0))
    assert not got.isnan().any()
    torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)


def test_a_large_sink_takes_the_weight() -> None:
    base, *_ = _attention_case(torch.float32, 4, 2, 32, 16, 8, [40, 9], [5, 1], 16)
    sunk, *_ = _attention_case(torch.float32, 4, 2, 32, 16, 8, [40, 9], [5, 1], 16, sink_shift=25.0)
    assert sunk.abs().max() < 1e-4 * base.abs().max()


# ------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {k: write_model(tmp_path_factory.mktemp("fegilix" + k), k) for k in CONFIGS}


LENGTHS = {"A": [1, 2, 9, 37, 70, 131], "B": [3, 33, 64, 97], "C": [5, 18, 40, 150], "D": [2, 47, 160, 330]}


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
    for steps in plans:
        got, _ = run_steps(model, page, steps, cases.max_live_tokens(steps))
        for rid in got:
            assert sorted(got[rid]) == list(range(len(reqs[rid])))
            rows = torch.stack([got[rid][p] for p in range(len(reqs[rid]))])
            assert_close(rows, want[rid], dtype, f"{which}/{rid}")


def test_batch_mates_slots_and_pages_do_not_matter(folders, oracle) -> None:
    """float32: a request's logits alone, beside others, and again on the slot and pages that
    another request has just given back, agree to rounding."""
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
def test_long_decoding(folders, dtype) -> None:
    from tinyserve_b200.model import DecoderModel

    cfg, w = plain.read_config(folders["B"]), plain.read_weights(folders["B"], torch.float64)
    toks = random_prompt(260, cfg["vocab"], 9)
    want = plain.forward(cfg, w, toks).float()
    model = DecoderModel.from_folder(folders["B"], dtype, "cuda")
    got, _ = run_steps(model, 16, cases.tail_decoded("a", toks, 255), 320)
    rows = torch.stack([got["a"][p] for p in range(260)])
    assert_close(rows[-20:], want[-20:], dtype, "the last decoded tokens")
    assert_close(rows, want, dtype, "all tokens")


@pytest.mark.parametrize("graphs", [True, False])
def test_greedy_generation_through_llm(folders, graphs) -> None:
    from tinyserve_b200 import LLM

    cfg, w = plain.read_config(folders["A"]), plain.read_weights(folders["A"], torch.float64)
    prompts = [random_prompt(n, cfg["vocab"], 40 + n) for n in (3, 11, 26, 50)]
    want = [plain.greedy(cfg, w, p, 8) for p in prompts]
    llm = LLM.from_folder(folders["A"], dtype="float32", page_size=8, num_pages=64, max_num_seqs=3, max_batch_tokens=32,
                          chunked_prefill=True, decode_graphs=graphs)
    assert llm.generate(prompts, max_new_tokens=8) == want
    assert (llm.engine.runner.num_graph_steps > 0) == graphs
    assert all(g.allocator.num_used == 0 for g in llm.cache.groups) and llm.cache.state_pool.num_free == 3


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
