"""A plain, slow implementation of the Fegilix decoder, one function per mechanism, written
from the design's equations and sharing no code with the product path. Everything runs token
by token or with full matrices on the CPU in one floating type (float64 for an oracle,
float32 otherwise); nothing is cached between calls.

Notation: ``h`` is a sub-layer's input ``[T, width]``; weights are ``[out, in]``; ``w`` maps
tensor names to tensors already converted to the working type.
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
    """Parse ``model.safetensors`` by hand: 8-byte length, JSON header, raw data."""
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
def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_mlp(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


def rotary_frequencies(dims: int, base: float, scaling: Mapping[str, float] | None, dtype=torch.float64) -> torch.Tensor:
    """f_i = base^(-2i/dims); with scaling, long wavelengths are divided by ``factor``, short ones
    kept, and those in between blended linearly in original/wavelength."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f.tolist():
            wavelength = 2.0 * math.pi / fi
            if wavelength < orig / high:
                out.append(fi)
            elif wavelength > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wavelength - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f.to(dtype)


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, dims: int) -> torch.Tensor:
    """x ``[T, heads, dim]``: element i < dims/2 pairs with element i + dims/2; the rest pass."""
    half = dims // 2
    angle = positions.to(freqs.dtype)[:, None] * freqs[None, :]
    c, s = angle.cos().to(x.dtype)[:, None, :], angle.sin().to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, sink: torch.Tensor | None,
                   first_pos: int = 0) -> torch.Tensor:
    """q ``[Tq, H, D]`` at positions first_pos.., k ``[Tk, G, D]``, v ``[Tk, G, Dv]`` at positions 0..;
    causal; the softmax's denominator also holds exp(sink_h), which carries no value."""
    tq, heads, _ = q.shape
    tk, groups, _ = k.shape
    rep = heads // groups
    out = torch.zeros(tq, heads, v.shape[-1], dtype=q.dtype)
    for hd in range(heads):
        g = hd // rep
        s = (q[:, hd] @ k[:, g].T) * scale
        qpos = torch.arange(first_pos, first_pos + tq)[:, None]
        s = s.masked_fill(torch.arange(tk)[None, :] > qpos, float("-inf"))
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[hd].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[hd] - m)
        out[:, hd] = (e / den) @ v[:, g]
    return out


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x ``[T, C]``, taps ``[C, K]`` with the last column on the current token; zeros before the start."""
    t, c = x.shape
    k = taps.shape[1]
    padded = torch.cat([torch.zeros(k - 1, c, dtype=x.dtype), x])
    y = torch.zeros_like(x)
    for j in range(k):
        y = y + padded[j: j + t] * taps[:, j][None, :]
    return y * torch.sigmoid(y)


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)


def delta_rule_scan(q, k, v, beta, decay):
    """Per head, token by token: S <- decay * S (per key channel); u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q. q, k, decay ``[T, H, D]``; v ``[T, H, Dv]``; beta ``[T, H]``."""
    t, heads, d = q.shape
    dv = v.shape[-1]
    s = torch.zeros(heads, d, dv, dtype=q.dtype)
    outs = []
    for i in range(t):
        s = decay[i][:, :, None] * s
        u = beta[i][:, None] * (v[i] - torch.einsum("hdv,hd->hv", s, k[i]))
        s = s + k[i][:, :, None] * u[:, None, :]
        outs.append(torch.einsum("hdv,hd->hv", s, q[i]))
    return torch.stack(outs)


def mlstm_scan(q, k, v, log_i, log_f):
    """Matrix memory with the stabiliser m (a running maximum) initialised to 0. q, k ``[T, H, D]`` (q already
    scaled), v ``[T, H, Dv]``, log gates ``[T, H]``."""
    t, heads, d = q.shape
    dv = v.shape[-1]
    s = torch.zeros(heads, d, dv, dtype=q.dtype)
    n = torch.zeros(heads, d, dtype=q.dtype)
    m = torch.zeros(heads, dtype=q.dtype)
    outs = []
    for j in range(t):
        m_new = torch.maximum(log_f[j] + m, log_i[j])
        keep = torch.exp(log_f[j] + m - m_new)
        take = torch.exp(log_i[j] - m_new)
        s = keep[:, None, None] * s + take[:, None, None] * (k[j][:, :, None] * v[j][:, None, :])
        n = keep[:, None] * n + take[:, None] * k[j]
        m = m_new
        num = torch.einsum("hdv,hd->hv", s, q[j])
        den = torch.maximum((n * q[j]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        outs.append(num / den[:, None])
    return torch.stack(outs)


# ------------------------------------------------------------------------ mixers
def mix_attention(h, w, p, mc, eps, positions, kv_store, layer_index):
    t = h.shape[0]
    heads, groups, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    rot = mc.get("rot")
    freqs = None if not rot else rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))

    def prepare(x, norm_w):
        x = rms_norm(x, norm_w, eps)
        return x if freqs is None else rotate(x, positions, freqs, rot["dims"])

    q = prepare((h @ w[p + "q"].T).view(t, heads, d), w[p + "q.norm"])
    src = mc.get("kv_from")
    if src is None:
        k = prepare((h @ w[p + "k"].T).view(t, groups, d), w[p + "k.norm"])
        v = (h @ w[p + "v"].T).view(t, groups, dv)
        kv_store[layer_index] = (k, v)
    else:
        k, v = kv_store[src]
    o = sink_attention(q, k, v, mc["scale"], w.get(p + "sink"))
    o = o.reshape(t, heads * dv) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def mix_mlstm(h, w, p, mc, eps):
    t = h.shape[0]
    heads, d, dv, cap = mc["heads"], mc["dim"], mc["vdim"], float(mc["gate_cap"])
    q = (h @ w[p + "q"].T).view(t, heads, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(t, heads, d)
    v = (h @ w[p + "v"].T).view(t, heads, dv)
    log_i = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    o = rms_norm(mlstm_scan(q, k, v, log_i, log_f), None, eps).reshape(t, heads * dv)
    o = o * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def mix_channel_delta(h, w, p, mc, eps):
    t = h.shape[0]
    heads, groups, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    rep = heads // groups
    q = causal_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).view(t, groups, d)
    k = causal_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).view(t, groups, d)
    v = causal_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).view(t, heads, dv)
    q = (unit(q) * d ** -0.5).repeat_interleave(rep, dim=1)
    k = unit(k).repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    step = torch.nn.functional.softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(t, heads, d)
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)
    o = rms_norm(delta_rule_scan(q, k, v, beta, decay), w[p + "norm"], eps)
    o = o.reshape(t, heads * dv) * torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T)
    return o @ w[p + "o"].T


# ------------------------------------------------------------------------- model
def forward(cfg: Mapping[str, Any], w: Mapping[str, torch.Tensor], ids: list[int], layers_out: list | None = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of the whole sequence. ``layers_out`` receives the sum of the
    streams after every layer."""
    eps = float(cfg["norm"]["eps"])
    t = len(ids)
    positions = torch.arange(t)
    x0 = w["embed"][torch.tensor(ids)]
    ns = cfg.get("streams")
    streams = [x0.clone() for _ in range(ns or 1)]
    kv_store: dict[int, Any] = {}

    def sublayer(prefix: str, which: int, fn) -> None:
        nonlocal streams
        norm_w = w[f"{prefix}norm{which}"]
        if ns is None:
            streams = [streams[0] + fn(rms_norm(streams[0], norm_w, eps))]
            return
        w_in, w_out, w_mix = (w[f"{prefix}hc{which}.{n}"] for n in ("in", "out", "mix"))
        u = sum(w_in[s] * streams[s] for s in range(ns))
        y = fn(rms_norm(u, norm_w, eps))
        streams = [sum(w_mix[s, j] * streams[s] for s in range(ns)) + w_out[j] * y for j in range(ns)]

    for li, layer in enumerate(cfg["layers"]):
        pre, mc, kind = f"l{li}.", layer["mixer"], layer["type"]
        p = pre + "mix."
        if kind == "attention":
            sublayer(pre, 1, lambda h: mix_attention(h, w, p, mc, eps, positions, kv_store, li))
        elif kind == "mlstm":
            sublayer(pre, 1, lambda h: mix_mlstm(h, w, p, mc, eps))
        elif kind == "channel_delta":
            sublayer(pre, 1, lambda h: mix_channel_delta(h, w, p, mc, eps))
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            sublayer(pre, 2, lambda h: gated_mlp(h, w[pre + "mlp.gate"], w[pre + "mlp.up"], w[pre + "mlp.down"]))
        if layers_out is not None:
            layers_out.append(sum(streams))
    x = rms_norm(sum(streams), w["final.norm"], eps)
    logits = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits


def greedy(cfg, w, prompt: list[int], new_tokens: int) -> list[int]:
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(forward(cfg, w, seq)[-1].argmax()))
    return seq[len(prompt):]
