"""Fegilix on the host: its configuration and tensor names; the kernels' references against the
plain implementation, one mechanism at a time; and the whole engine (cache manager, step function,
scheduler, sampler) with the references in the kernels' place against the plain model, under
every cut of the work."""

from __future__ import annotations

import json

import pytest
import torch

import kernel_refs as refs
import plain_fegilix as plain
import replay_cases as cases
from fegilix_cases import CONFIGS, CONFIG_A, FakeStep, assert_close, run_steps, write_model
from kernel_refs import use_references
from tiny_configs import random_prompt

from tinyserve_b200.config import UnsupportedConfigError, config_from_dict
from tinyserve_b200.model import DecoderModel, build_parts
from tinyserve_b200.parts import KVNeed, SplitKVNeed, StateNeed
from tinyserve_b200.weights import WeightLoadError
from tinyserve_b200.weights.loader import checkpoint_names, merge_specs


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {k: write_model(tmp_path_factory.mktemp("fegilix" + k), k) for k in CONFIGS}


# ------------------------------------------------------------------ configuration
def test_config_round_trip_and_names(folders) -> None:
    for which, (cfg, _) in CONFIGS.items():
        c = config_from_dict(cfg)
        assert config_from_dict(c.to_dict()) == c and c.to_dict() == cfg
        assert json.loads((folders[which] / "config.json").read_text())["architecture"] == "Fegilix"
    names = checkpoint_names(merge_specs(build_parts(config_from_dict(CONFIG_A).to_spec()).tensor_specs()))
    assert names["l0.mix.q.conv"] == (32, 3) and names["l0.mix.a2"] == (64, 8) and names["l0.mix.g2"] == (128, 12)
    assert names["l1.mix.sink"] == (4,) and names["l1.mix.k.norm"] == (32,) and names["l1.hc2.mix"] == (3, 3)
    assert names["l2.mix.i.b"] == (3,) and names["l2.mix.norm"] == (144,) and names["l0.mix.norm"] == (32,)
    assert "l3.mix.k" not in names and "l3.mix.k.norm" not in names and "l3.mix.q.norm" in names
    assert "l0.norm2" not in names and "l0.hc2.in" not in names and names["head"] == (89, 64)


def test_cache_needs_and_order(folders) -> None:
    model = DecoderModel.from_folder(folders["A"], torch.float32, "cpu")
    needs = model.cache_needs()
    assert isinstance(needs[0], StateNeed) and needs[0].shape == (4 * 16 * 32 + 2 * (2 * 2 * 16 + 4 * 32),)
    assert needs[1] == SplitKVNeed(2, 32, 16) and isinstance(needs[2], StateNeed) and needs[3] is None
    assert model.spec.order[3].reads_cache_of == 1
    assert model.parts.recordable("decode") and model.parts.recordable("prefill")
    b = DecoderModel.from_folder(folders["B"], torch.float32, "cpu").cache_needs()
    assert b[0] == KVNeed(1, 32, None) and b[3] == SplitKVNeed(3, 16, 48)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "unknown mixer type"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 0), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "routed"), "only 'dense'"),
    (lambda c: c["layers"][2]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.__setitem__("streams", 0), "streams"),
])
def test_config_refusals(change, message) -> None:
    cfg = json.loads(json.dumps(CONFIG_A))
    change(cfg)
    with pytest.raises(UnsupportedConfigError, match=message):
        config_from_dict(cfg)


def test_ranks_come_from_the_checkpoint(folders, tmp_path) -> None:
    """A configuration without the low-rank sizes loads (the shapes give them); a wrong width still fails."""
    cfg = json.loads((folders["A"] / "config.json").read_text())
    for key in ("step_rank", "gate_rank"):
        cfg["layers"][0]["mixer"].pop(key)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    (tmp_path / "model.safetensors").write_bytes((folders["A"] / "model.safetensors").read_bytes())
    model = DecoderModel.from_folder(tmp_path, torch.float32, "cpu")
    assert model.tensors["l0.mix.a1"].shape == (8, 64) and model.tensors["l0.mix.g2"].shape == (128, 12)
    cfg["width"] = 32
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(WeightLoadError, match="wrong shape"):
        DecoderModel.from_folder(tmp_path, torch.float32, "cpu")


def test_random_weights_need_the_ranks(tmp_path) -> None:
    from tinyserve_b200.weights import write_random_model

    cfg = json.loads(json.dumps(CONFIG_A))
    cfg["layers"][0]["mixer"].pop("step_rank")
    with pytest.raises(ValueError, match="only a checkpoint gives"):
        write_random_model(tmp_path, config_from_dict(cfg), 0)


# --------------------------------------------- references against the plain mechanisms
def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def test_reference_hyper_connections() -> None:
    s, t, h = 3, 5, 16
    x0, y1, y2 = _rand(t, h, seed=1), _rand(t, h, seed=2), _rand(t, h, seed=3)
    w = {k: _rand(*shape, seed=i + 10) for i, (k, shape) in enumerate(
        {"in1": (s,), "out1": (s,), "mix1": (s, s), "in2": (s,), "out2": (s,), "mix2": (s, s)}.items())}
    nw = 1 + _rand(h, seed=5) * 0.1
    # plain: explicit lanes
    lanes = [x0.clone() for _ in range(s)]
    u1 = sum(w["in1"][i] * lanes[i] for i in range(s))
    lanes = [sum(w["mix1"][i, j] * lanes[i] for i in range(s)) + w["out1"][j] * y1 for j in range(s)]
    u2 = sum(w["in2"][i] * lanes[i] for i in range(s))
    lanes = [sum(w["mix2"][i, j] * lanes[i] for i in range(s)) + w["out2"][j] * y2 for j in range(s)]
    buf, out = torch.zeros(s, t, h), torch.zeros(t, h)
    refs.hc_mix_norm(buf, x0, None, None, None, w["in1"], nw, 1e-5, out)
    torch.testing.assert_close(out, plain.rms_norm(u1, nw, 1e-5))
    refs.hc_mix_norm(buf, None, y1, w["mix1"], w["out1"], w["in2"], nw, 1e-5, out)
    torch.testing.assert_close(out, plain.rms_norm(u2, nw, 1e-5))
    rows = torch.tensor([4, 0], dtype=torch.int32)
    total = torch.zeros(2, h)
    refs.hc_collapse(buf, None, y2, w["mix2"], w["out2"], rows, total)
    torch.testing.assert_close(total, sum(lanes)[rows.long()])


def test_reference_sink_attention_and_preparation() -> None:
    t, heads, groups, d, dv, page = 21, 4, 2, 32, 16, 4
    q, k, v = _rand(t, heads * d, seed=1), _rand(t, groups * d, seed=2), _rand(t, groups * dv, seed=3)
    qw, kw, sink = 1 + _rand(d, seed=4) * 0.2, 1 + _rand(d, seed=5) * 0.2, _rand(heads, seed=6)
    freqs = plain.rotary_frequencies(16, 1e4, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32})
    pos = torch.arange(t)
    pq = plain.rotate(plain.rms_norm(q.view(t, heads, d), qw, 1e-5), pos, freqs, 16)
    pk = plain.rotate(plain.rms_norm(k.view(t, groups, d), kw, 1e-5), pos, freqs, 16)
    want = plain.sink_attention(pq, pk, v.view(t, groups, dv), 0.2, sink)

    from tinyserve_b200.parts.rope import RotaryEncoding
    enc = RotaryEncoding(d, 16, 1e4, "half", {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32})
    torch.testing.assert_close(enc._inv_freq_host, freqs.double())
    angle = pos.double()[:, None] * enc._inv_freq_host
    cos, sin = angle.cos().float(), angle.sin().float()
    pages = 8
    kc, vc = torch.full((pages, groups, page, d), float("nan")), torch.full((pages, groups, page, dv), float("nan"))
    table = torch.tensor([[5, 2, 7, 0, 3, 6]], dtype=torch.int32)
    slots = (table[0].long()[pos // page] * page + pos % page).int()
    qo = torch.zeros(t, heads, d)
    refs.qkv_prepare(q, k, v, qw, kw, 1e-5, cos, sin, 16, slots, kc, vc, page, heads, groups, d, dv, qo)
    torch.testing.assert_close(qo, pq)

    class Ctx:
        num_seqs = 1
        cu_query_lens = torch.tensor([0, t], dtype=torch.int32)
        context_lens_dev = torch.tensor([t], dtype=torch.int32)

    out = torch.zeros(t, heads * dv)
    refs.paged_attention(qo, kc, vc, page, table, Ctx, 0.2, 0, out, sinks=sink)
    torch.testing.assert_close(out.view(t, heads, dv), want)
    # a large sink takes the weight away from every value
    big = torch.zeros(t, heads * dv)
    refs.paged_attention(qo, kc, vc, page, table, Ctx, 0.2, 0, big, sinks=sink + 30.0)
    assert big.abs().max() < 1e-6 * out.abs().max() + 1e-9


@pytest.mark.parametrize("cuts", [[13], [1, 1, 1, 10], [5, 2, 6]])
def test_reference_recurrences_carry_their_state(cuts) -> None:
    """Conv + delta rule and mLSTM references, fed in portions through a state slot, equal the
    plain scans over the whole sequence."""
    t, heads, groups, d, dv, taps = 13, 4, 2, 16, 24, 3
    c = 2 * groups * d + heads * dv
    x, w_taps = _rand(t, c, seed=1), _rand(c, taps, seed=2, scale=0.5)
    a, bias, a_log, beta = _rand(t, heads * d, seed=3), _rand(heads * d, seed=4), _rand(heads, seed=5, scale=0.3), _rand(t, heads, seed=6)
    y = plain.causal_conv_silu(x, w_taps)
    rep = heads // groups
    q = (plain.unit(y[:, : groups * d].view(t, groups, d)) * d ** -0.5).repeat_interleave(rep, 1)
    k = plain.unit(y[:, groups * d: 2 * groups * d].view(t, groups, d)).repeat_interleave(rep, 1)
    decay = torch.exp(-torch.exp(a_log)[None, :, None] * torch.nn.functional.softplus(a + bias).view(t, heads, d))
    want = plain.delta_rule_scan(q, k, y[:, 2 * groups * d:].view(t, heads, dv), torch.sigmoid(beta), decay)
    state = torch.zeros(3, heads * d * dv + (taps - 1) * c)
    got, at = torch.zeros(t, heads, dv), 0
    for n in cuts:
        step = FakeStep([n], [1])
        conved = torch.zeros(n, c)
        refs.causal_conv_silu(x[at: at + n], w_taps, state[:, heads * d * dv:], step, conved)
        out = torch.zeros(n, heads, dv)
        refs.delta_scan(conved, 0, groups * d, 2 * groups * d, a[at: at + n], bias, a_log, beta[at: at + n], d ** -0.5,
                        state[:, : heads * d * dv], step, heads, groups, d, dv, out)
        got[at: at + n] = out
        at += n
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    assert state[0].abs().max() == 0 and state[2].abs().max() == 0

    qkv, gates, gb = _rand(t, 2 * heads * d + heads * dv, seed=7), _rand(t, 2 * heads, seed=8, scale=3.0), _rand(2 * heads, seed=9)
    cap = 4.0
    li = cap * torch.tanh((gates[:, :heads] + gb[:heads]) / cap)
    lf = torch.nn.functional.logsigmoid(cap * torch.tanh((gates[:, heads:] + gb[heads:]) / cap))
    want = plain.mlstm_scan(qkv[:, : heads * d].view(t, heads, d) * d ** -0.5, qkv[:, heads * d: 2 * heads * d].view(t, heads, d),
                            qkv[:, 2 * heads * d:].view(t, heads, dv), li, lf)
    state = torch.zeros(2, refs.mlstm_state_size(heads, d, dv))
    got, at = torch.zeros(t, heads, dv), 0
    for n in cuts:
        out = torch.zeros(n, heads, dv)
        refs.mlstm_scan(qkv[at: at + n], 0, heads * d, 2 * heads * d, gates[at: at + n], gb, cap, d ** -0.5, state,
                        FakeStep([n], [0]), heads, d, dv, out)
        got[at: at + n] = out
        at += n
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


def test_reference_gates() -> None:
    from fegilix_cases import gelu_tanh

    gu, out = _rand(3, 8, seed=1, scale=2.0), torch.zeros(3, 4)
    refs.act_mul(gu, out, "gelu_tanh")
    assert abs(float(out[1, 2]) - gelu_tanh(float(gu[1, 2])) * float(gu[1, 6])) < 1e-6
    x, w, g = _rand(2, 3, 8, seed=2), _rand(8, seed=3), _rand(2, 24, seed=4)
    out = torch.zeros(2, 24)
    refs.head_norm_gate(x, w, False, g, True, 1e-5, out)
    torch.testing.assert_close(out.view(2, 3, 8), plain.rms_norm(x, w, 1e-5) * torch.sigmoid(g).view(2, 3, 8))
    lg = _rand(2, 9, seed=5, scale=40.0)
    want = 20.0 * torch.tanh(lg / 20.0)
    refs.softcap(lg, 20.0)
    torch.testing.assert_close(lg, want)
    assert lg.abs().max() <= 20.0


# ----------------------------------------------- the engine on the host, every cut
LENGTHS = {"A": [1, 2, 9, 37, 70], "B": [3, 33, 64], "C": [5, 18, 40], "D": [2, 21, 50]}


@pytest.fixture(scope="module")
def oracle(folders):
    out = {}
    for which in CONFIGS:
        cfg, w = plain.read_config(folders[which]), plain.read_weights(folders[which], torch.float64)
        reqs = {f"r{i}": random_prompt(n, cfg["vocab"], 100 + 7 * i) for i, n in enumerate(LENGTHS[which])}
        out[which] = (reqs, {rid: plain.forward(cfg, w, toks).float() for rid, toks in reqs.items()})
    return out


@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
@pytest.mark.parametrize("page", [4, 16])
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
        assert all(g.allocator.num_used == 0 for g in cache.groups) and cache.state_pool.num_free == 3
    assert len({tuple(x) for x in want}) > 1
