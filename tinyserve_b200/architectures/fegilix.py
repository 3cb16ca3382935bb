"""Fegilix: a decoder whose layers are listed one by one in ``config.json``, each with one of three
mixers (sink attention with an output gate, an mLSTM matrix memory, a gated delta rule with
per-channel decay), an optional gated feed-forward, and hyper-connections between them.

``config.json`` keys read here: ``architecture`` = "Fegilix"; ``vocab``, ``width``; ``norm.eps``;
``streams`` (lanes of the hyper-connections; absent = a plain residual stream);
``logit_softcap`` (absent = none); ``layers``: a list of ``{"type", "mixer": {...}, "mlp": {...} | null}``.
Mixer keys by type: ``attention``: ``heads, kv_heads, dim, vdim, scale``, optional ``rot``
(``dims, base``, optional ``scaling`` with ``factor, low, high, original``) and ``kv_from`` (the layer
whose cached keys and values this layer reads instead of making its own); ``mlstm``: ``heads, dim,
vdim, gate_cap``; ``channel_delta``: ``heads, kv_heads, dim, vdim, conv`` (and, only in configurations
written by this framework, the ranks ``step_rank`` and ``gate_rank``, which a checkpoint's shapes
give otherwise). ``mlp``: ``kind`` = "dense" and ``ff``. Optional ``max_positions`` bounds a request's length for the
engine's bookkeeping. Every size and constant comes from these keys.

What the design fixes, passed to the parts as arguments by ``to_spec``: pre-norm layers with
plain-weight RMSNorm; q/k RMSNorm per head before a rotate-half rotation; causal attention; the
tanh form of GELU in the feed-forward; tensor names ``embed``, ``l<i>.norm1|norm2``,
``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from ..config.base import LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec, UnsupportedConfigError
from ..config.registry import register_architecture

ARCHITECTURE = "Fegilix"
MIXER_TYPES = ("attention", "mlstm", "channel_delta")
DEFAULT_MAX_POSITIONS = 1 << 17


def _need(d: Mapping[str, Any], key: str, where: str) -> Any:
    if key not in d or d[key] is None:
        raise UnsupportedConfigError(f"{where} has no {key!r}")
    return d[key]


@dataclass(frozen=True)
class FegilixConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[Mapping[str, Any], ...]
    streams: int | None = None
    logit_softcap: float | None = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    architecture = ARCHITECTURE

    def __post_init__(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or not self.norm_eps > 0:
            raise UnsupportedConfigError("vocab, width and norm.eps must be positive")
        if self.streams is not None and self.streams < 1:
            raise UnsupportedConfigError(f"streams={self.streams} must be at least 1")
        if not self.layers:
            raise UnsupportedConfigError("layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXER_TYPES:
                raise UnsupportedConfigError(f"{where}: unknown mixer type {kind!r}; known: {MIXER_TYPES}")
            m = _need(layer, "mixer", where)
            for key in {"attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
                        "mlstm": ("heads", "dim", "vdim", "gate_cap"),
                        "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv")}[kind]:
                _need(m, key, f"{where}.mixer")
            src = m.get("kv_from")
            if src is not None:
                if kind != "attention" or not 0 <= int(src) < i or self.layers[int(src)]["type"] != "attention" \
                        or self.layers[int(src)]["mixer"].get("kv_from") is not None:
                    raise UnsupportedConfigError(f"{where}: kv_from={src} must name an earlier attention layer with keys and values of its own")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise UnsupportedConfigError(f"{where}: mlp.kind={mlp.get('kind')!r}: only 'dense' is implemented")
                _need(mlp, "ff", f"{where}.mlp")

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FegilixConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != ARCHITECTURE:
            raise UnsupportedConfigError(f"expected {ARCHITECTURE}, got {name!r}")
        norm = _need(d, "norm", "config.json")
        streams = d.get("streams")
        cap = d.get("logit_softcap")
        return cls(
            vocab_size=int(_need(d, "vocab", "config.json")),
            hidden_size=int(_need(d, "width", "config.json")),
            norm_eps=float(_need(norm, "eps", "norm")),
            layers=tuple(copy.deepcopy(dict(layer)) for layer in _need(d, "layers", "config.json")),
            streams=None if streams is None else int(streams),
            logit_softcap=None if cap is None else float(cap),
            max_positions=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
        )

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.norm_eps}, "layers": [copy.deepcopy(dict(layer)) for layer in self.layers]}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d

    # ------------------------------------------------------------------ the spec
    def _mixer(self, kind: str, m: Mapping[str, Any]) -> tuple[PartSpec, PartSpec | None]:
        h, eps = self.hidden_size, self.norm_eps
        if kind == "attention":
            rot = m.get("rot")
            position = None
            if rot:
                position = PartSpec("rope", {"head_dim": int(m["dim"]), "rotary_dim": int(_need(rot, "dims", "rot")),
                                             "theta": float(_need(rot, "base", "rot")), "pairing": "half",
                                             "scaling": dict(rot["scaling"]) if rot.get("scaling") else None})
            return PartSpec("gated_sink_attention", {
                "prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]), "qk_norm": True,
                "qk_norm_eps": eps, "sink": True, "own_kv": m.get("kv_from") is None}), position
        if kind == "mlstm":
            return PartSpec("mlstm", {"prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]),
                                      "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]),
                                      "gate_cap": float(m["gate_cap"]), "norm_eps": eps}), None
        return PartSpec("channel_delta", {
            "prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
            "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "conv_taps": int(m["conv"]), "norm_eps": eps,
            "step_rank": int(m.get("step_rank", -1)), "gate_rank": int(m.get("gate_rank", -1))}), None

    def to_spec(self) -> ModelSpec:
        h, eps = self.hidden_size, self.norm_eps
        lanes = self.streams or 1

        def norm(name: str, connection: str) -> PartSpec:
            return PartSpec("hyper_rms_norm", {"name": name, "size": h, "eps": eps, "streams": lanes,
                                               "connection": connection if self.streams is not None else None})

        layers, order = [], []
        for i, layer in enumerate(self.layers):
            mixer, position = self._mixer(layer["type"], layer["mixer"])
            parts = {"mixer_norm": norm("norm1", "hc1."), "mixer": mixer}
            if layer.get("mlp") is not None:
                parts["feed_forward_norm"] = norm("norm2", "hc2.")
                parts["feed_forward"] = PartSpec("gated_mlp", {
                    "prefix": "mlp.", "hidden_size": h, "intermediate_size": int(layer["mlp"]["ff"]),
                    "activation": "gelu_tanh", "names": {"gate": "gate", "up": "up", "down": "down"}})
            layers.append(LayerSpec(prefix=f"l{i}.", block="hyper_prenorm", parts=parts, position=position))
            src = layer["mixer"].get("kv_from")
            order.append(LayerCall(i, None if src is None else int(src)))
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab_size, hidden_size=h, layers=tuple(layers), order=tuple(order),
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": self.vocab_size, "hidden_size": h}),
            final_norm=PartSpec("hyper_final_norm", {"name": "final.norm", "size": h, "eps": eps}),
            head=PartSpec("lm_head", {"name": "head", "tied": False, "vocab_size": self.vocab_size, "hidden_size": h,
                                      "softcap": self.logit_softcap}),
            max_position_embeddings=self.max_positions,
        )


register_architecture(ARCHITECTURE, FegilixConfig)
