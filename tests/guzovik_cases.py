"""Small Guzovik configurations that differ from one another in every size and option, shared by the
host-only and the GPU tests of that architecture."""

from __future__ import annotations

from pathlib import Path

import torch

# Grouped heads with keys and values of different sizes, windows that end inside a page, a latent layer
# whose rotation covers only part of its rotated elements, a dense and a routed feed-forward (5 experts,
# 2 used, a shared one), a layer that runs on another's tensors, a layer without a feed-forward.
CONFIG_A = {
    "architecture": "Guzovik", "vocab": 83, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 40, "limit": 1.5},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2, "mask": {"size": 7}}},
        {"type": "latent_attention",
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 24}, "shared": {"ff": 16}},
         "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 20, "scale": 0.25, "mask": {"size": 5},
                   "rot": {"dims": 4, "base": 100.0}}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2, "mask": {"size": 7}}, "weights_of": 0},
        {"type": "latent_attention",
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 24}, "shared": {"ff": 16}},
         "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 20, "scale": 0.25, "mask": {"size": 5},
                   "rot": {"dims": 4, "base": 100.0}}, "weights_of": 1},
    ],
}
CONFIG_A["layers"][2]["mlp"] = CONFIG_A["layers"][0]["mlp"]        # an entry equals the one whose tensors it uses

# Equal key and value sizes of 64 (bfloat16 attention on the tensor cores, with sink and window), a latent
# layer without a window, one expert used of eight and no shared one, every expert used, no embedding scale.
CONFIG_B = {
    "architecture": "Guzovik", "vocab": 131, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "layers": [
        {"type": "latent_attention", "mlp": {"kind": "moe", "router": {"experts": 8, "top": 1}, "expert": {"ff": 32}},
         "mixer": {"heads": 2, "dim": 32, "rot_dim": 32, "vdim": 32, "kv_rank": 64, "scale": 0.125,
                   "rot": {"dims": 32, "base": 10000.0}}},
        {"type": "attention", "mlp": {"kind": "moe", "router": {"experts": 3, "top": 3}, "expert": {"ff": 16}, "shared": {"ff": 32}},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 40}}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 96, "limit": 4.0},
         "mixer": {"heads": 4, "kv_heads": 4, "dim": 64, "vdim": 64, "scale": 0.11, "mask": {"size": 33}}},
    ],
}

# One head everywhere, a width that is no multiple of 32, odd inner sizes, an attention layer without a
# window, a window of one (a token sees itself only).
CONFIG_C = {
    "architecture": "Guzovik", "vocab": 61, "width": 36, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 20, "limit": 0.75},
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25}},
        {"type": "latent_attention", "mlp": {"kind": "moe", "router": {"experts": 2, "top": 1}, "expert": {"ff": 12}, "shared": {"ff": 20}},
         "mixer": {"heads": 1, "dim": 8, "rot_dim": 2, "vdim": 40, "kv_rank": 12, "scale": 0.3, "mask": {"size": 19},
                   "rot": {"dims": 2, "base": 50.0}}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 24, "vdim": 8, "scale": 0.2, "mask": {"size": 1}}},
    ],
}

# Sizes at which the experts' products run on the tensor cores, one shared key/value head of 128, a long
# window, a latent as large as the kernels' middle form takes, the routed layers on the same tensors.
MOE_D = {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 64}, "shared": {"ff": 128}}
CONFIG_D = {
    "architecture": "Guzovik", "vocab": 211, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
    "layers": [
        {"type": "attention", "mlp": dict(MOE_D),
         "mixer": {"heads": 4, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.09, "mask": {"size": 100}}},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 256, "limit": 2.0},
         "mixer": {"heads": 4, "dim": 32, "rot_dim": 16, "vdim": 32, "kv_rank": 160, "scale": 0.14, "mask": {"size": 70},
                   "rot": {"dims": 16, "base": 1000.0}}},
        {"type": "attention", "mlp": dict(MOE_D),
         "mixer": {"heads": 4, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.09, "mask": {"size": 100}}, "weights_of": 0},
    ],
}

CONFIGS = {"A": (CONFIG_A, 21), "B": (CONFIG_B, 22), "C": (CONFIG_C, 23), "D": (CONFIG_D, 24)}


def write_model(folder: Path, which: str, std_scale: float = 6.0) -> Path:
    """The configuration with random weights, through the framework's random-weights mode."""
    import tinyserve_b200.architectures  # noqa: F401
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model

    cfg, seed = CONFIGS[which]
    return write_random_model(folder, config_from_dict(cfg), seed, torch.bfloat16, std_scale=std_scale)


class FakeCtx:
    """The fields of a step that the attention references and kernels read."""

    def __init__(self, query_lens: list[int], context_lens: list[int], device="cpu") -> None:
        cu = [0]
        for n in query_lens:
            cu.append(cu[-1] + n)
        self.num_seqs = len(query_lens)
        self.query_lens, self.context_lens = list(query_lens), list(context_lens)
        self.cu_query_lens = torch.tensor(cu, dtype=torch.int32, device=device)
        self.context_lens_dev = torch.tensor(context_lens, dtype=torch.int32, device=device)
        dec = [i for i, n in enumerate(query_lens) if n == 1]
        pre = [i for i, n in enumerate(query_lens) if n != 1]
        self.decode_seqs = torch.tensor(dec + [0] * (len(query_lens) - len(dec)), dtype=torch.int32, device=device)
        self.prefill_seqs = torch.tensor(pre + [0] * (len(query_lens) - len(pre)), dtype=torch.int32, device=device)
        self.num_decode, self.num_prefill = len(dec), len(pre)
        self.max_query_len, self.max_context_len = max(query_lens), max(context_lens)
        self.num_tokens = cu[-1]


def row_errors(rows: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference over that of the centred oracle."""
    w = want.double() - want.double().mean(-1, keepdim=True)
    return (rows.double() - want.double()).pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt()


def assert_rows_close(rows: torch.Tensor, want: torch.Tensor, dtype: torch.dtype, what: str = "", limit32: float = 2e-5) -> None:
    """float32: every row equals the oracle up to summation order. bfloat16: rounding moves a typical row by
    about one percent of the logits' spread, but a token whose best router logits lie closer together than
    that rounding takes another expert than the oracle, and its row (and, diluted, later rows that attend
    to it) differs by much more; so the rows are judged by their median and their upper quartile, and the
    float32 run of the same schedule carries the exactness."""
    assert not rows.isnan().any(), f"{what}: NaN in the logits"
    err = row_errors(rows, want)
    if dtype == torch.float32:
        assert float(err.max()) < limit32, f"{what}: relative error {float(err.max()):.3g}"
        return
    s = err.sort().values
    median, upper = float(s[len(s) // 2]), float(s[(3 * len(s)) // 4])
    assert median < (0.03 if len(s) >= 20 else 0.08), f"{what}: median relative error {median:.3g} over {len(s)} rows"
    if len(s) >= 20:
        assert upper < 0.06, f"{what}: upper quartile of the relative error {upper:.3g} over {len(s)} rows"


def random_config(seed: int) -> dict:
    """A configuration drawn at random: sizes, head counts, windows, the order of the layers, which layers
    run on another's tensors, the kinds of feed-forward and every constant."""
    import random

    rng = random.Random(seed)
    width = rng.choice([32, 40, 64, 96, 128, 160, 256])

    def window():
        return rng.choice([None, 1, 5, 17, 64, 100, 200])

    def mixer(kind: str) -> dict:
        w = window()
        if kind == "attention":
            heads = rng.choice([1, 2, 3, 4, 6, 8, 12])
            groups = rng.choice([g for g in (1, 2, 3, 4, 6) if heads % g == 0])
            dim = rng.choice([16, 24, 32, 48, 64, 80, 128])
            m = {"heads": heads, "kv_heads": groups, "dim": dim, "vdim": rng.choice([dim, dim, 16, 40, 64]),
                 "scale": rng.uniform(0.5, 1.5) * dim ** -0.5}
        else:
            rot_dim = rng.choice([8, 16, 32, 64])
            dim = rng.choice([16, 32, 64])
            m = {"heads": rng.choice([1, 2, 4, 5, 8]), "dim": dim, "rot_dim": rot_dim, "vdim": rng.choice([16, 32, 48, 64]),
                 "kv_rank": rng.choice([16, 24, 48, 64, 96, 128, 192, 256]), "scale": rng.uniform(0.5, 1.5) * (dim + rot_dim) ** -0.5,
                 "rot": {"dims": rng.choice([rot_dim, rot_dim // 2]), "base": rng.choice([100.0, 1e4, 1e6])}}
        if w is not None:
            m["mask"] = {"size": w}
        return m

    def mlp():
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return {"kind": "dense", "ff": rng.choice([24, 64, 128, 200]), "limit": rng.choice([0.5, 2.0, 7.0])}
        experts = rng.randint(2, 12)
        out = {"kind": "moe", "router": {"experts": experts, "top": rng.randint(1, min(4, experts))},
               "expert": {"ff": rng.choice([16, 32, 64, 72])}}
        if rng.random() < 0.6:
            out["shared"] = {"ff": rng.choice([16, 64, 96])}
        return out

    layers: list[dict] = []
    for i in range(rng.randint(2, 7)):
        own = [j for j, layer in enumerate(layers) if "weights_of" not in layer]
        if own and rng.random() < 0.35:
            j = rng.choice(own)
            layers.append({**{k: v for k, v in layers[j].items()}, "weights_of": j})
            continue
        kind = rng.choice(["attention", "latent_attention"])
        layers.append({"type": kind, "mixer": mixer(kind), "mlp": mlp()})
    return {"architecture": "Guzovik", "vocab": rng.randint(50, 600), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])},
            "embedding": {"scale": rng.choice([1.0, 4.0, width ** 0.5])}, "layers": layers}
