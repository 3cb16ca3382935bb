"""Hyper-connections: the residual stream in ``S`` parallel lanes, and the parts that read and
rebuild them.

Before sub-layer ``q`` the lanes are read, ``u = sum_s in_q[s] x_s``; the sub-layer runs on
``norm(u)``; its output ``y`` then rebuilds every lane from the old ones at once,
``x_t <- sum_s mix_q[s, t] x_s + out_q[t] y`` (``mix`` is indexed ``[from, to]``). All lanes
start as the embedding output; after the last layer the stream is the sum of the lanes. With
``S = 1`` and ``in = out = mix = 1`` this is the plain residual sum.

As with the single stream, a sub-layer's output stays *pending*: ``HyperRMSNorm`` is the norm in
front of a sub-layer and owns that sub-layer's three connection tensors. Its kernel applies the
pending rebuild (with the weights of the sub-layer before, which the block left on the stream),
reads the lanes with its own ``in`` and normalises, in one pass over the lanes.
``HyperFinalNorm`` collapses the lanes for the wanted rows and applies the model's last norm.
``HyperBlock`` is the pre-norm arrangement around these, with an optional feed-forward.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..kernels import ops
from .base import (EVERY_STEP, Block, Norm, Part, ResidualStream, StepContext, TensorSpec, register_block,
                   register_norm)


class HyperRMSNorm(Norm):
    recordable = EVERY_STEP

    def __init__(self, name: str, size: int, eps: float, streams: int = 1, connection: str | None = None) -> None:
        """``connection``: prefix of the sub-layer's ``in [S]``, ``out [S]`` and ``mix [S, S]``
        tensors; ``None`` means fixed weights of one (then ``streams`` must be 1)."""
        if streams < 1 or (connection is None and streams != 1):
            raise ValueError(f"streams={streams}: fixed connections exist for one stream only")
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.streams, self.connection = int(streams), connection
        self.weight = self.w_in = self.w_out = self.w_mix = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        specs = [TensorSpec(prefix + self.name, (self.size,), init="one_plus_normal")]
        if self.connection is not None:
            c, s = prefix + self.connection, self.streams
            specs += [TensorSpec(c + "in", (s,), init="one_plus_normal", std=0.1),
                      TensorSpec(c + "out", (s,), init="one_plus_normal", std=0.1),
                      TensorSpec(c + "mix", (s, s), init="normal", std=0.3)]
        return specs

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[prefix + self.name]
        if self.connection is not None:
            c = prefix + self.connection
            self.w_in, self.w_out, self.w_mix = (tensors[c + n].float().contiguous() for n in ("in", "out", "mix"))
        else:
            one = torch.ones(1, dtype=torch.float32, device=self.weight.device)
            self.w_in, self.w_out, self.w_mix = one, one, one.view(1, 1)

    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        t, h = stream.resid.shape
        fresh = None
        if stream.lanes is None:
            if stream.delta is not None:
                raise RuntimeError("a sub-layer output is pending on a stream that has no lanes yet")
            stream.lanes = ctx.arena.take_step((self.streams, t, h), torch.float32)
            fresh = stream.resid
        elif stream.lanes.shape[0] != self.streams:
            raise RuntimeError(f"the stream has {stream.lanes.shape[0]} lanes, this connection {self.streams}")
        mix, out_w = stream.connection if stream.delta is not None else (None, None)
        out = ctx.arena.take((t, h), ctx.dtype)
        ops.hc_mix_norm(stream.lanes, fresh, stream.delta, mix, out_w, self.w_in, self.weight, self.eps, out)
        stream.delta = None
        stream.connection = None
        return out

    def leave(self, stream: ResidualStream, y: torch.Tensor) -> None:
        """The sub-layer behind this norm has produced ``y``: it stays pending with this
        connection's weights."""
        stream.delta = y
        stream.connection = (self.w_mix, self.w_out)
        stream.sumsq = None

    def forward_rows(self, stream, rows, num_rows, ctx):
        raise NotImplementedError("a connection norm stands in front of a sub-layer; the model's last norm is 'hyper_final_norm'")


class HyperFinalNorm(Norm):
    """The model's last norm over the sum of the lanes, for chosen rows."""

    recordable = EVERY_STEP

    def __init__(self, name: str, size: int, eps: float) -> None:
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix + self.name, (self.size,), init="one_plus_normal")]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[prefix + self.name]

    def summed(self, stream: ResidualStream, rows: torch.Tensor | None, num_rows: int, ctx: StepContext) -> torch.Tensor:
        """The sum of the lanes (pending output included) at ``rows``, 32-bit ``[num_rows, hidden]``."""
        total = ctx.arena.take_step((num_rows, self.size), torch.float32)
        if stream.lanes is None:
            lanes, fresh = stream.resid.view(1, *stream.resid.shape), stream.resid
        else:
            lanes, fresh = stream.lanes, None
        mix, out_w = stream.connection if stream.delta is not None else (None, None)
        ops.hc_collapse(lanes, fresh, stream.delta, mix, out_w, rows, total)
        return total

    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        t = stream.resid.shape[0]
        out = ctx.arena.take_step((t, self.size), ctx.dtype)
        ops.add_rms_norm(self.summed(stream, None, t, ctx), None, self.weight, self.eps, out)
        return out

    def forward_rows(self, stream: ResidualStream, rows: torch.Tensor, num_rows: int, ctx: StepContext) -> torch.Tensor:
        out = ctx.arena.take_step((num_rows, self.size), ctx.dtype)
        ops.add_rms_norm(self.summed(stream, rows, num_rows, ctx), None, self.weight, self.eps, out)
        return out


class HyperBlock(Block):
    """``mixer`` and (optionally) ``feed_forward``, each behind a ``HyperRMSNorm``."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    optional_roles = frozenset({"feed_forward_norm", "feed_forward"})

    def __init__(self, parts: Mapping[str, Part]) -> None:
        super().__init__(parts)
        if ("feed_forward" in parts) != ("feed_forward_norm" in parts):
            raise ValueError("a feed-forward and its norm come together")
        for role in ("mixer_norm", "feed_forward_norm"):
            if role in parts and not isinstance(parts[role], HyperRMSNorm):
                raise TypeError(f"role {role!r} of a hyper-connection block takes a 'hyper_rms_norm'")

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, Any], writes_cache: bool,
                position: Any) -> None:
        p = self.parts
        ctx.arena.next_frame()
        ctx.upcoming_weights = []
        norm = p["mixer_norm"]
        norm.leave(stream, p["mixer"].forward(norm.forward(stream, ctx), ctx, caches.get("mixer"), writes_cache, position))
        if "feed_forward" in p:
            norm = p["feed_forward_norm"]
            norm.leave(stream, p["feed_forward"].forward(norm.forward(stream, ctx), ctx))


register_norm("hyper_rms_norm", HyperRMSNorm)
register_norm("hyper_final_norm", HyperFinalNorm)
register_block("hyper_prenorm", HyperBlock)
