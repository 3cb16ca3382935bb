"""Guzovik on the host: its configuration and tensor names; the kernels' references against the
plain implementation, one mechanism at a time; and the whole engine (cache manager, step function,
scheduler, sampler) with the references in the kernels' place against the plain model, under
every cut of the work."""

from __future__ import annotations

import json
import math

import pytest
import torch

import kernel_refs as refs
import plain_guzovik as plain
import replay_cases as cases
from fegilix_cases import assert_close, run_steps
from guzovik_cases import CONFIGS, CONFIG_A, CONFIG_B, FakeCtx, write_model
from kernel_refs import use_references
from tiny_configs import random_prompt

from tinyserve_b200.config import UnsupportedConfigError, config_from_dict
from tinyserve_b200.model import DecoderModel, build_parts
from tinyserve_b200.parts import KVNeed, SplitKVNeed
from tinyserve_b200.parts.base import LatentNeed
from tinyserve_b200.weights.loader import checkpoint_names, merge_specs


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {k: write_model(tmp_path_factory.mktemp("guzovik" + k), k) for k in CONFIGS}


def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


# ------------------------------------------------------------------ configuration
def test_config_round_trip_and_names(folders) -> None:
    for which, (cfg, _) in CONFIGS.items():
        c = config_from_dict(cfg)
        assert config_from_dict(c.to_dict()) == c and c.to_dict() == cfg
        assert json.loads((folders[which] / "config.json").read_text())["architecture"] == "Guzovik"
    names = checkpoint_names(merge_specs(build_parts(config_from_dict(CONFIG_A).to_spec()).tensor_specs()))
    assert names["l0.mix.q"] == (128, 48) and names["l0.mix.k"] == (64, 48) and names["l0.mix.v"] == (32, 48)
    assert names["l0.mix.g"] == (4, 48) and names["l0.mix.o"] == (48, 64) and names["l0.ls1"] == (48,)
    assert names["l0.mlp.gate"] == (40, 48) and names["l0.norm2b"] == (48,)
    assert names["l1.mix.q"] == (72, 48) and names["l1.mix.dkv"] == (28, 48) and names["l1.mix.dkv.norm"] == (20,)
    assert names["l1.mix.uk"] == (48, 20) and names["l1.mix.uv"] == (72, 20) and names["l1.mix.o"] == (48, 72)
    assert names["l1.mlp.router"] == (5, 48) and names["l1.mlp.e4.down"] == (48, 24) and names["l1.mlp.shared.up"] == (16, 48)
    assert not any(n.startswith(("l2.", "l3.")) for n in names), "a layer on another's tensors has none of its own"
    assert names["final.norm"] == (48,) and names["head"] == (83, 48) and "l0.mix.sink" not in names
    b = checkpoint_names(merge_specs(build_parts(config_from_dict(CONFIG_B).to_spec()).tensor_specs()))
    assert "l0.mlp.shared.gate" not in b and b["l0.mlp.e7.gate"] == (32, 64)


def test_cache_needs_and_order(folders) -> None:
    model = DecoderModel.from_folder(folders["A"], torch.float32, "cpu")
    assert model.cache_needs() == [SplitKVNeed(2, 32, 16, 7), LatentNeed(28, 5), SplitKVNeed(2, 32, 16, 7), LatentNeed(28, 5)]
    assert [c.layer for c in model.spec.order] == [0, 1, 0, 1] and all(c.reads_cache_of is None for c in model.spec.order)
    assert model.parts.recordable("decode") and model.parts.recordable("prefill")
    b = DecoderModel.from_folder(folders["B"], torch.float32, "cpu").cache_needs()
    assert b == [LatentNeed(96, None), KVNeed(2, 64, 40), KVNeed(4, 64, 33)]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "unknown mixer type"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 1), "another type"),
    (lambda c: c["layers"][3].__setitem__("weights_of", 3), "weights_of"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "sparse"), "'dense' and 'moe'"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), "top=6"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_config_refusals(change, message) -> None:
    cfg = json.loads(json.dumps(CONFIG_A))
    change(cfg)
    with pytest.raises(UnsupportedConfigError, match=message):
        config_from_dict(cfg)


# --------------------------------------------- references against the plain mechanisms
def test_reference_norms_around_a_sub_layer() -> None:
    t, h = 6, 20
    x, y = _rand(t, h, seed=1).float(), _rand(t, h, seed=2, scale=3.0).float()
    wb, ls, w = _rand(h, seed=3, scale=0.2).float(), _rand(h, seed=4).float(), _rand(h, seed=5, scale=0.2).float()
    want_x = x + plain.offset_norm(y, wb, 1e-5) * ls
    want = plain.offset_norm(want_x, w, 1e-5)
    resid, out = x.clone(), torch.zeros(t, h)
    refs.post_norm_add_rms_norm(resid, y, wb, ls, 1e-5, True, w, True, 1e-5, out)
    torch.testing.assert_close(resid, want_x)
    torch.testing.assert_close(out, want)
    rows = torch.tensor([4, 1], dtype=torch.int32)
    resid, some = x.clone(), torch.zeros(2, h)
    refs.post_norm_add_rms_norm(resid, y, wb, ls, 1e-5, True, w, True, 1e-5, some, rows=rows)
    torch.testing.assert_close(some, want[rows.long()])
    torch.testing.assert_close(resid, x)           # chosen rows leave the stream alone
    refs.post_norm_add_rms_norm(resid, None, None, None, 0.0, False, w, True, 1e-5, out)
    torch.testing.assert_close(out, plain.offset_norm(x, w, 1e-5))


def _paged(rows: torch.Tensor, page: int, table: list[int]) -> tuple[torch.Tensor, torch.Tensor]:
    """``rows [T, ...]`` laid into pages in the table's order, NaN elsewhere; returns the storage
    ``[pages, page, ...]`` and the tokens' slots."""
    t = rows.shape[0]
    store = torch.full((max(table) + 2, page, *rows.shape[1:]), float("nan"), dtype=rows.dtype)
    pos = torch.arange(t)
    slots = torch.tensor(table)[pos // page] * page + pos % page
    store.view(-1, *rows.shape[1:])[slots] = rows
    return store, slots.int()


@pytest.mark.parametrize("window", [None, 1, 6, 9])
def test_reference_window_attention_with_an_added_one(window) -> None:
    t, width, page = 23, 24, 4
    m = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.4, "mask": {"size": window} if window else None}
    w = {"q": _rand(32, width, seed=1), "k": _rand(16, width, seed=2), "v": _rand(24, width, seed=3),
         "g": _rand(4, width, seed=4), "o": torch.eye(48, dtype=torch.float64)}
    h = _rand(t, width, seed=5)
    want = plain.window_attention(h, torch.arange(t), w, "", m)
    table = [5, 2, 7, 0, 3, 6]
    q, k, v = (h @ w["q"].T).float(), (h @ w["k"].T).float(), (h @ w["v"].T).float()
    kc = _paged(k.view(t, 2, 8), page, table)[0].transpose(1, 2).contiguous()
    vc = _paged(v.view(t, 2, 12), page, table)[0].transpose(1, 2).contiguous()
    out = torch.zeros(t, 48)
    refs.paged_attention(q.view(t, 4, 8), kc, vc, page, torch.tensor([table], dtype=torch.int32), FakeCtx([t], [t]),
                         0.4, window or 0, out, sinks=torch.zeros(4))
    gated = torch.zeros(t, 48)
    refs.head_norm_gate(out.view(t, 4, 12), None, False, (h @ w["g"].T).float(), False, 0.0, gated, gate_per_head=True)
    torch.testing.assert_close(gated.double(), want, atol=1e-5, rtol=1e-5)


def test_the_added_one_takes_the_weight_when_every_score_is_low() -> None:
    t = 5
    q, k, v = torch.ones(t, 1, 4), -50.0 * torch.ones(8, 1, 4, 4), torch.ones(8, 1, 4, 3)
    out = torch.zeros(t, 3)
    refs.paged_attention(q, k, v, 4, torch.tensor([[1, 3]], dtype=torch.int32), FakeCtx([t], [t]), 1.0, 0, out, sinks=torch.zeros(1))
    assert out.abs().max() < 1e-30
    refs.paged_attention(q, -k, v, 4, torch.tensor([[1, 3]], dtype=torch.int32), FakeCtx([t], [t]), 1.0, 0, out, sinks=torch.zeros(1))
    torch.testing.assert_close(out, torch.ones(t, 3))


@pytest.mark.parametrize("window, dims", [(None, 6), (4, 6), (11, 2)])
def test_reference_latent_attention_folded_against_plain(window, dims) -> None:
    """The folded form (queries through the keys' up-projection, values' up-projection after the sum,
    one cached row per token) equals keys and values made per head."""
    t, width, page, heads, d, dr, dv, rank = 19, 20, 4, 3, 8, 6, 10, 12
    m = {"heads": heads, "dim": d, "rot_dim": dr, "vdim": dv, "kv_rank": rank, "scale": 0.3,
         "mask": {"size": window} if window else None, "rot": {"dims": dims, "base": 30.0}}
    w = {"q": _rand(heads * (d + dr), width, seed=1), "dkv": _rand(rank + dr, width, seed=2), "dkv.norm": 1 + _rand(rank, seed=3, scale=0.1),
         "uk": _rand(heads * d, rank, seed=4), "uv": _rand(heads * dv, rank, seed=5), "o": torch.eye(heads * dv, dtype=torch.float64)}
    h = _rand(t, width, seed=6)
    want = plain.latent_attention(h, torch.arange(t), w, "", m, 1e-5)
    q, ckr = (h @ w["q"].T).float(), (h @ w["dkv"].T).float()
    folded = torch.zeros(heads, t, rank)
    refs.bmm(q.view(t, heads, d + dr)[:, :, :d].transpose(0, 1), w["uk"].float().view(heads, d, rank), folded)
    f = torch.tensor([30.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    angle = torch.arange(t).double()[:, None] * f
    table = [4, 1, 6, 0, 3]
    store, slots = _paged(torch.zeros(t, rank + dr), page, table)
    qo = torch.zeros(t, heads, rank + dr)
    refs.latent_prepare(q, folded, ckr, w["dkv.norm"].float(), 1e-5, angle.cos().float(), angle.sin().float(), dims, True,
                        slots, store.view(-1, rank + dr), heads, d, rank, dr, qo)
    mixed = torch.zeros(t, heads, rank)
    refs.latent_attention(qo, store.view(-1, rank + dr), page, torch.tensor([table], dtype=torch.int32), FakeCtx([t], [t]),
                          rank, 0.3, window or 0, mixed)
    up = torch.zeros(heads, t, dv)
    refs.bmm(mixed.transpose(0, 1), w["uv"].float().view(heads, dv, rank).transpose(1, 2), up)
    torch.testing.assert_close(up.transpose(0, 1).reshape(t, heads * dv).double(), want, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("experts, top, shared", [(5, 2, True), (8, 1, False), (3, 3, True), (70, 4, False)])
def test_reference_routed_experts(experts, top, shared) -> None:
    t, width, ff = 37, 16, 12
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": 8} if shared else None}
    w = {"router": _rand(experts, width, seed=1)}
    for e in range(experts):
        w.update({f"e{e}.gate": _rand(ff, width, seed=10 + e), f"e{e}.up": _rand(ff, width, seed=200 + e),
                  f"e{e}.down": _rand(width, ff, seed=400 + e)})
    if shared:
        w.update({"shared.gate": _rand(8, width, seed=2), "shared.up": _rand(8, width, seed=3), "shared.down": _rand(width, 8, seed=4)})
    h = _rand(t, width, seed=5, scale=0.5)
    want = plain.expert_mixture(h, w, "", mlp)
    plan = refs.moe_route((h @ w["router"].T).float(), top, torch.zeros(experts, dtype=torch.int32))
    assert plan["offsets"][-1] == t * top and sorted(plan["row_of"].tolist()) == list(range(t * top))
    gate_up = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)]).float()
    down = torch.stack([w[f"e{e}.down"] for e in range(experts)]).float()
    act, y, out = torch.zeros(t * top, ff), torch.zeros(t * top, width), torch.zeros(t, width)
    refs.moe_gemm(h.float(), gate_up, act, plan, True, True)
    refs.moe_gemm(act, down, y, plan, False, False)
    extra = plain.silu_glu(h, w, "shared.").float() if shared else None
    refs.moe_combine(y, plan, extra, out)
    torch.testing.assert_close(out.double(), want, atol=2e-4, rtol=2e-4)


def test_router_ties_go_to_the_lower_index() -> None:
    z = torch.tensor([[1.0, 3.0, 3.0, 0.0, 3.0], [2.0, 2.0, 2.0, 2.0, 2.0]])
    plan = refs.moe_route(z, 2, torch.zeros(5, dtype=torch.int32))
    assert plan["ids"].view(2, 2).tolist() == [[1, 2], [0, 1]]
    torch.testing.assert_close(plan["weights"].view(2, 2), torch.full((2, 2), 0.5))


def test_reference_clamped_feed_forward() -> None:
    w = {"gate": _rand(6, 5, seed=1, scale=2.0), "up": _rand(6, 5, seed=2, scale=2.0), "down": torch.eye(6, dtype=torch.float64)}
    h = _rand(9, 5, seed=3)
    out = torch.zeros(9, 6)
    refs.gemm_gated(h.float(), torch.cat([w["gate"], w["up"]]).float(), out, None, "clamped_swish", 1.25)
    torch.testing.assert_close(out.double(), plain.clamped_glu(h, w, "", 1.25), atol=1e-5, rtol=1e-5)
    g, u = 5.0, -7.0        # both beyond the limit: min(g, L) sigmoid(1.702 L) (max(u, -L) + 1)
    one = torch.zeros(1, 1)
    refs.act_mul(torch.tensor([[g, u]]), one, "clamped_swish", 1.25)
    assert abs(float(one) - 1.25 / (1 + math.exp(-1.702 * 1.25)) * (-1.25 + 1)) < 1e-6


# ----------------------------------------------- the engine on the host, every cut
LENGTHS = {"A": [1, 2, 9, 37, 70], "B": [3, 45, 90], "C": [5, 18, 40], "D": [2, 21]}


@pytest.fixture(scope="module")
def oracle(folders):
    out = {}
    for which in CONFIGS:
        cfg, w = plain.read_config(folders[which]), plain.read_weights(folders[which], torch.float64)
        reqs = {f"r{i}": random_prompt(n, cfg["vocab"], 100 + 7 * i) for i, n in enumerate(LENGTHS[which])}
        out[which] = (reqs, {rid: plain.forward(cfg, w, toks).float() for rid, toks in reqs.items()})
    return out


@pytest.mark.parametrize("which, page", [("A", 4), ("A", 16), ("B", 8), ("C", 4), ("D", 16)])
def test_engine_on_host_under_every_cut(folders, oracle, which, page) -> None:
    reqs, want = oracle[which]
    model = DecoderModel.from_folder(folders[which], torch.float32, "cpu")
    plans = [cases.mixed(reqs, 3), cases.mixed(reqs, 5, max_live=2)]
    for rid, toks in reqs.items():
        plans += [cases.whole(rid, toks), cases.tail_decoded(rid, toks, 12), cases.portions(rid, toks, 1)]
    with use_references():
        for steps in plans:
            got, _ = run_steps(model, page, steps, cases.max_live_tokens(steps))
            for rid in got:
                rows = torch.stack([got[rid][p] for p in range(len(reqs[rid]))])
                assert_close(rows, want[rid], torch.float32, f"{which}/{rid}")


def test_greedy_generation_through_the_engine_on_host(folders) -> None:
    from tinyserve_b200.cache import CacheManager
    from tinyserve_b200.engine import Engine

    cfg, w = plain.read_config(folders["A"]), plain.read_weights(folders["A"], torch.float64)
    prompts = [random_prompt(n, cfg["vocab"], 40 + n) for n in (3, 11, 26)]
    want = [plain.greedy(cfg, w, p, 6) for p in prompts]
    model = DecoderModel.from_folder(folders["A"], torch.float32, "cpu")
    for kw in (dict(num_pages=64), dict(num_pages=64, max_batch_tokens=8, chunked_prefill=True), dict(num_pages=5)):
        pages = kw.pop("num_pages")
        cache = CacheManager(model.cache_needs(), page_size=8, num_pages=pages, max_requests=3, dtype=torch.float32, device="cpu")
        with use_references():
            e = Engine(model, cache, max_num_seqs=3, **kw)
            assert e.generate(prompts, 6) == want
        assert all(g.allocator.num_used == 0 for g in cache.groups)
    assert len({tuple(x) for x in want}) > 1
