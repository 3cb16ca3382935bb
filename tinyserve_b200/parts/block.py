"""Pre-norm residual block: ``x += mixer(norm(x)); x += feed_forward(norm(x))``
(upstream src/tinyserve/model.py:154-179). The two sums are not made here: each sub-layer's
output is left pending on the stream and the next norm adds it in 32-bit.
"""

from __future__ import annotations

from typing import Any, Mapping

from .base import Block, Part, ResidualStream, StepContext, register_block


class PreNormBlock(Block):
    # the order is the order of the layer's tensors in ``tensor_specs``
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, parts: Mapping[str, Part]) -> None:
        super().__init__(parts)
        self.mixer, self.feed_forward = parts["mixer"], parts["feed_forward"]
        self.mixer_norm, self.feed_forward_norm = parts["mixer_norm"], parts["feed_forward_norm"]

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, Any], writes_cache: bool,
                position: Any) -> None:
        # Scratch of this layer goes to the other half of the arena than the previous
        # layer's, whose pending output the first norm below still has to read.
        ctx.arena.next_frame()
        mixer, ff = self.mixer, self.feed_forward
        cache = caches.get("mixer")
        ctx.upcoming_weights = ff.streamed_weights()
        hn = self.mixer_norm.lazy(stream, ctx) if mixer.takes_lazy_input else self.mixer_norm.forward(stream, ctx)
        if mixer.adds_to_stream:
            mixed = mixer.forward(hn, ctx, cache, writes_cache, position, stream=stream)
        else:
            mixed = mixer.forward(hn, ctx, cache, writes_cache, position)
        self._leave(stream, mixed)
        hn = self.feed_forward_norm.lazy(stream, ctx) if ff.takes_lazy_input else self.feed_forward_norm.forward(stream, ctx)
        self._leave(stream, ff.forward(hn, ctx, stream=stream) if ff.adds_to_stream else ff.forward(hn, ctx))

    @staticmethod
    def _leave(stream: ResidualStream, out: Any) -> None:
        """A sub-layer's output stays pending on the stream, unless the part has added it itself."""
        if out is not None:
            stream.delta = out
            stream.sumsq = None


class SandwichBlock(Block):
    """A norm before and after each sub-layer: ``x += post(mixer(norm(x)))`` and, when the layer has
    a feed-forward, ``x += post(feed_forward(norm(x)))``. The post norms (``PostRMSNorm``, which may
    carry a layer scale) stay pending with the output and are applied by the next norm's kernel."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    optional_roles = frozenset({"feed_forward_norm", "feed_forward", "feed_forward_post_norm"})

    def __init__(self, parts: Mapping[str, Part]) -> None:
        super().__init__(parts)
        ff = [r for r in ("feed_forward_norm", "feed_forward", "feed_forward_post_norm") if r in parts]
        if ff and len(ff) != 3:
            raise ValueError("a feed-forward comes with its norm and its post norm")
        for role in ("mixer_post_norm", "feed_forward_post_norm"):
            if role in parts and not hasattr(parts[role], "leave"):
                raise TypeError(f"role {role!r} takes a norm that can stay pending (a 'post_rms_norm')")

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, Any], writes_cache: bool,
                position: Any) -> None:
        p = self.parts
        ctx.arena.next_frame()
        ctx.upcoming_weights = []
        hn = p["mixer_norm"].forward(stream, ctx)
        p["mixer_post_norm"].leave(stream, p["mixer"].forward(hn, ctx, caches.get("mixer"), writes_cache, position))
        if "feed_forward" in p:
            hn = p["feed_forward_norm"].forward(stream, ctx)
            p["feed_forward_post_norm"].leave(stream, p["feed_forward"].forward(hn, ctx))


register_block("prenorm", PreNormBlock)
register_block("sandwich", SandwichBlock)
