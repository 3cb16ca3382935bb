"""A plain, slow implementation of the Guzovik decoder, one function per mechanism, written from
the design's equations and sharing no code with the product path. Everything runs with full
matrices on the CPU in one floating type (float64 for an oracle); nothing is cached between calls.

Notation: ``h`` is a sub-layer's input ``[T, width]``; weights are ``[out, in]``; ``w`` maps
tensor names to tensors already converted to the working type; ``pos`` are the tokens' positions.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path
from typing import Any, Mapping

import torch


# ------------------------------------------------------------------------ files
def read_config(folder: str | Path) -> dict[str, Any]:
    return json.loads((Path(folder) / "config.json").read_text())


def read_weights(folder: str | Path, dtype: torch.dtype = torch.float64) -> dict[str, torch.Tensor]:
    """``model.safetensors`` parsed by hand: 8-byte length, JSON header, raw data."""
    raw = (Path(folder) / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8: 8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + a: 8 + n + b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t if info["dtype"] == "I32" else t.to(dtype)
    return out


# -------------------------------------------------------------------- mechanisms
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The weight is stored around zero: the gain is ``1 + weight``."""
    return unit_rms(x, eps) * (1.0 + weight)


def plain_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight


def visible(pos: torch.Tensor, window: int | None) -> torch.Tensor:
    """``[T, T]`` bool: query i sees key j when ``0 <= pos_i - pos_j`` (``< window`` if one is set)."""
    gap = pos[:, None] - pos[None, :]
    ok = gap >= 0
    return ok if window is None else ok & (gap < window)


def softmax_rows(scores: torch.Tensor, ok: torch.Tensor, extra_one: bool) -> torch.Tensor:
    """Softmax over the visible keys; ``extra_one`` puts one more term, exp(0), into the denominator
    (a key of score 0 that carries no value)."""
    s = scores.masked_fill(~ok, -math.inf)
    top = s.max(-1, keepdim=True).values
    if extra_one:
        top = top.clamp_min(0.0)
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if extra_one:
        den = den + torch.exp(-top)
    return e / den


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Neighbouring elements ``(2i, 2i+1)`` of the first ``dims`` of the last axis turn by
    ``pos * base^(-2i/dims)``; the rest pass. ``x`` is ``[T, ..., n]``."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=x.dtype)
    a = pos.to(x.dtype)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = a.cos().reshape(shape), a.sin().reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def window_attention(h: torch.Tensor, pos: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any]) -> torch.Tensor:
    """Grouped heads without rotation, a window, one added to the softmax's denominator, and a
    sigmoid gate per head on the heads' outputs."""
    t = h.shape[0]
    heads, groups, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(t, heads, d)
    k = (h @ w[p + "k"].T).view(t, groups, d)
    v = (h @ w[p + "v"].T).view(t, groups, dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)                     # [T, heads]
    ok = visible(pos, m["mask"]["size"] if m.get("mask") else None)
    outs = []
    for a in range(heads):
        b = a // (heads // groups)
        pr = softmax_rows((q[:, a] @ k[:, b].T) * m["scale"], ok, extra_one=True)
        outs.append((pr @ v[:, b]) * gate[:, a: a + 1])
    return torch.cat(outs, -1) @ w[p + "o"].T


def latent_attention(h: torch.Tensor, pos: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping[str, Any],
                     eps: float) -> torch.Tensor:
    """Keys and values made from one normed latent vector per token; a small rotated key part
    shared by the heads; ordinary softmax over a window."""
    t = h.shape[0]
    heads, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    q = (h @ w[p + "q"].T).view(t, heads, d + dr)
    down = h @ w[p + "dkv"].T
    c = plain_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_turn = rotate_pairs(down[:, rank:], pos, rot["dims"], rot["base"])          # [T, dr]
    q_still, q_turn = q[..., :d], rotate_pairs(q[..., d:].contiguous(), pos, rot["dims"], rot["base"])
    k_still = (c @ w[p + "uk"].T).view(t, heads, d)
    v = (c @ w[p + "uv"].T).view(t, heads, dv)
    ok = visible(pos, m["mask"]["size"] if m.get("mask") else None)
    outs = []
    for a in range(heads):
        s = (q_still[:, a] @ k_still[:, a].T + q_turn[:, a] @ k_turn.T) * m["scale"]
        outs.append(softmax_rows(s, ok, extra_one=False) @ v[:, a])
    return torch.cat(outs, -1) @ w[p + "o"].T


def clamped_glu(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = (h @ w[p + "gate"].T).clamp(max=limit)
    u = (h @ w[p + "up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def silu_glu(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    z = h @ w[p + "gate"].T
    return (z * torch.sigmoid(z) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h: torch.Tensor, router: torch.Tensor, top: int) -> tuple[torch.Tensor, torch.Tensor]:
    """The ``top`` largest router logits of each token and the softmax over those alone."""
    z = h @ router.T
    best, ids = z.topk(top, dim=-1)
    return ids, torch.softmax(best, -1)


def expert_mixture(h: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mlp: Mapping[str, Any]) -> torch.Tensor:
    ids, weights = route(h, w[p + "router"], mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), weights[t]):
            out[t] += a * silu_glu(h[t: t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + silu_glu(h, w, p + "shared.")
    return out


# ------------------------------------------------------------------------ model
def tensors_of(cfg: Mapping[str, Any], i: int) -> int:
    """The layer whose tensors layer ``i`` uses."""
    return int(cfg["layers"][i].get("weights_of", i))


def forward(cfg: Mapping[str, Any], w: Mapping[str, torch.Tensor], tokens: list[int], keep_layers: bool = False):
    """Logits ``[T, vocab]`` of one sequence from position 0 (and, on request, the stream after
    every layer)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    pos = torch.arange(len(tokens))
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{tensors_of(cfg, i)}."
        h = offset_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = window_attention(h, pos, w, p + "mix.", layer["mixer"])
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, pos, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + offset_norm(y, w[p + "norm1b"], eps) * w[p + "ls1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            h = offset_norm(x, w[p + "norm2"], eps)
            y = clamped_glu(h, w, p + "mlp.", mlp["limit"]) if mlp["kind"] == "dense" else expert_mixture(h, w, p + "mlp.", mlp)
            x = x + offset_norm(y, w[p + "norm2b"], eps) * w[p + "ls2"]
        after.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if keep_layers else logits


def greedy(cfg: Mapping[str, Any], w: Mapping[str, torch.Tensor], prompt: list[int], new_tokens: int) -> list[int]:
    """The ``new_tokens`` most likely next tokens, one after the other (the whole sequence is run again each time)."""
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(forward(cfg, w, seq)[-1].argmax()))
    return seq[len(prompt):]
