"""Guzovik: a decoder whose layers are listed one by one in ``config.json``. Each layer has one of
two mixers (windowed grouped-query attention without rotation, with one added to the softmax's
denominator and a sigmoid gate per head; or latent attention, whose keys and values come from one
cached low-rank vector per token plus a small rotated key part shared by the heads) and optionally
a feed-forward (a clamped gated one, or a routed mixture of SwiGLU experts with a shared expert).
Every sub-layer stands between two norms, and its normed output is scaled per column before the
residual sum. A layer may run on another layer's tensors with a cache of its own.

``config.json`` keys read here: ``architecture`` = "Guzovik"; ``vocab``, ``width``; ``norm.eps``;
``embedding.scale``; ``layers``: a list of ``{"type", "mixer": {...}, "mlp": {...} | null}`` and
optionally ``"weights_of": j`` (the layer has no tensors: it uses layer j's). Mixer keys by type:
``attention``: ``heads, kv_heads, dim, vdim, scale`` and optional ``mask.size``;
``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, scale``, ``rot`` (``dims, base``) and
optional ``mask.size``. ``mlp``: ``kind`` = "dense" with ``ff, limit``, or "moe" with
``router.experts, router.top, expert.ff`` and optional ``shared.ff``. Optional ``max_positions``
bounds a request's length for the engine's bookkeeping. Every size and constant comes from these keys.

What the design fixes, passed to the parts as arguments by ``to_spec``: RMS norms whose weights are
stored around zero (gain ``1 + w``) before and after every sub-layer, a layer scale on the normed
output; a sink of score 0 and a gate per head in the windowed attention; neighbouring elements as
rotation pairs and a plain-weight norm of the latent; 1.702 in the clamped feed-forward; SiLU
experts weighted by the softmax over the chosen router logits; tensor names ``embed``,
``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.ls1|ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from ..config.base import LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec, UnsupportedConfigError
from ..config.registry import register_architecture

ARCHITECTURE = "Guzovik"
MIXER_TYPES = ("attention", "latent_attention")
DEFAULT_MAX_POSITIONS = 1 << 17
_MIXER_KEYS = {"attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
               "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot")}


def _need(d: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise UnsupportedConfigError(f"{where} has no {key!r}")
    return d[key]


def _window(m: Mapping[str, Any], where: str) -> int | None:
    mask = m.get("mask")
    if mask is None:
        return None
    size = int(_need(mask, "size", f"{where}.mask"))
    if size <= 0:
        raise UnsupportedConfigError(f"{where}.mask.size={size} must be positive")
    return size


@dataclass(frozen=True)
class GuzovikConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[Mapping[str, Any], ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    architecture = ARCHITECTURE

    def __post_init__(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or not self.norm_eps > 0:
            raise UnsupportedConfigError("vocab, width and norm.eps must be positive")
        if not self.layers:
            raise UnsupportedConfigError("layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXER_TYPES:
                raise UnsupportedConfigError(f"{where}: unknown mixer type {kind!r}; known: {MIXER_TYPES}")
            m = _need(layer, "mixer", where)
            for key in _MIXER_KEYS[kind]:
                _need(m, key, f"{where}.mixer")
            _window(m, f"{where}.mixer")
            if kind == "attention" and int(m["heads"]) % int(m["kv_heads"]):
                raise UnsupportedConfigError(f"{where}: heads={m['heads']} is not a multiple of kv_heads={m['kv_heads']}")
            if kind == "latent_attention":
                dims = int(_need(m["rot"], "dims", f"{where}.mixer.rot"))
                _need(m["rot"], "base", f"{where}.mixer.rot")
                if dims % 2 or not 0 < dims <= int(m["rot_dim"]):
                    raise UnsupportedConfigError(f"{where}: rot.dims={dims} must be even and at most rot_dim={m['rot_dim']}")
            mlp = layer.get("mlp")
            if mlp is not None:
                mk = _need(mlp, "kind", f"{where}.mlp")
                if mk == "dense":
                    _need(mlp, "ff", f"{where}.mlp")
                    _need(mlp, "limit", f"{where}.mlp")
                elif mk == "moe":
                    router = _need(mlp, "router", f"{where}.mlp")
                    experts, top = int(_need(router, "experts", "router")), int(_need(router, "top", "router"))
                    if not 0 < top <= experts:
                        raise UnsupportedConfigError(f"{where}: top={top} of {experts} experts")
                    _need(_need(mlp, "expert", f"{where}.mlp"), "ff", f"{where}.mlp.expert")
                    if mlp.get("shared") is not None:
                        _need(mlp["shared"], "ff", f"{where}.mlp.shared")
                else:
                    raise UnsupportedConfigError(f"{where}: mlp.kind={mk!r}: 'dense' and 'moe' are implemented")
            src = layer.get("weights_of")
            if src is not None:
                src = int(src)
                if not 0 <= src < i or self.layers[src].get("weights_of") is not None:
                    raise UnsupportedConfigError(f"{where}: weights_of={src} must name an earlier layer with tensors of its own")
                if self.layers[src]["type"] != kind:
                    raise UnsupportedConfigError(f"{where}: weights_of={src} names a layer of another type")

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "GuzovikConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != ARCHITECTURE:
            raise UnsupportedConfigError(f"expected {ARCHITECTURE}, got {name!r}")
        emb = d.get("embedding") or {}
        return cls(
            vocab_size=int(_need(d, "vocab", "config.json")),
            hidden_size=int(_need(d, "width", "config.json")),
            norm_eps=float(_need(_need(d, "norm", "config.json"), "eps", "norm")),
            embedding_scale=float(emb.get("scale", 1.0)),
            layers=tuple(copy.deepcopy(dict(layer)) for layer in _need(d, "layers", "config.json")),
            max_positions=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
        )

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                             "layers": [copy.deepcopy(dict(layer)) for layer in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d

    # ------------------------------------------------------------------ the spec
    def _mixer(self, kind: str, m: Mapping[str, Any]) -> tuple[PartSpec, PartSpec | None]:
        h = self.hidden_size
        window = _window(m, "mixer")
        if kind == "attention":
            return PartSpec("gated_sink_attention", {
                "prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]), "qk_norm": False,
                "sink": "zero", "gate": "head", "window": window}), None
        rot = m["rot"]
        position = PartSpec("rope", {"head_dim": int(m["rot_dim"]), "rotary_dim": int(rot["dims"]),
                                     "theta": float(rot["base"]), "pairing": "interleaved"})
        return PartSpec("latent_attention", {
            "prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]), "nope_dim": int(m["dim"]),
            "rope_dim": int(m["rot_dim"]), "value_dim": int(m["vdim"]), "rank": int(m["kv_rank"]),
            "scale": float(m["scale"]), "norm_eps": self.norm_eps, "window": window}), position

    def _feed_forward(self, mlp: Mapping[str, Any]) -> PartSpec:
        h = self.hidden_size
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"prefix": "mlp.", "hidden_size": h, "intermediate_size": int(mlp["ff"]),
                                          "activation": "clamped_swish", "limit": float(mlp["limit"]),
                                          "names": {"gate": "gate", "up": "up", "down": "down"}})
        shared = mlp.get("shared")
        return PartSpec("routed_experts", {"prefix": "mlp.", "hidden_size": h, "num_experts": int(mlp["router"]["experts"]),
                                           "top": int(mlp["router"]["top"]), "expert_size": int(mlp["expert"]["ff"]),
                                           "shared_size": None if shared is None else int(shared["ff"])})

    def to_spec(self) -> ModelSpec:
        h, eps = self.hidden_size, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"name": name, "size": h, "eps": eps, "unit_offset": True})

        def post(name: str, scale: str) -> PartSpec:
            return PartSpec("post_rms_norm", {"name": name, "size": h, "eps": eps, "unit_offset": True, "scale_name": scale})

        # layers with tensors of their own become LayerSpecs; the order names one per config entry, so
        # a layer that uses another's tensors is a second call of that LayerSpec with a cache of its own
        layers: list[LayerSpec] = []
        spec_of: dict[int, int] = {}
        order: list[LayerCall] = []
        for i, layer in enumerate(self.layers):
            src = layer.get("weights_of")
            if src is None:
                mixer, position = self._mixer(layer["type"], layer["mixer"])
                parts = {"mixer_norm": norm("norm1"), "mixer": mixer, "mixer_post_norm": post("norm1b", "ls1")}
                if layer.get("mlp") is not None:
                    parts["feed_forward_norm"] = norm("norm2")
                    parts["feed_forward"] = self._feed_forward(layer["mlp"])
                    parts["feed_forward_post_norm"] = post("norm2b", "ls2")
                spec_of[i] = len(layers)
                layers.append(LayerSpec(prefix=f"l{i}.", block="sandwich", parts=parts, position=position))
                order.append(LayerCall(spec_of[i]))
            else:
                order.append(LayerCall(spec_of[int(src)]))
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab_size, hidden_size=h, layers=tuple(layers), order=tuple(order),
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": self.vocab_size, "hidden_size": h,
                                                   "scale": self.embedding_scale}),
            final_norm=PartSpec("rms_norm", {"name": "final.norm", "size": h, "eps": eps, "unit_offset": True}),
            head=PartSpec("lm_head", {"name": "head", "tied": False, "vocab_size": self.vocab_size, "hidden_size": h}),
            max_position_embeddings=self.max_positions,
        )


register_architecture(ARCHITECTURE, GuzovikConfig)
