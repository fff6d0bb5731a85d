"""The parallel residual arrangement: one norm, and mixer and feed-forward side by side on its output,

    h = norm(x);   x += s_m * mixer(h) + s_f * feed_forward(h);   x += side(x, tokens)

``s_m`` and ``s_f`` are optional per-channel scales (layer scale), the feed-forward and the side input
(something the layer adds from the step's token ids, reading the new stream) are optional.  The stream
and every sum into it are fp32.
"""
from __future__ import annotations

from ..kernels import mixing
from .base import Arrangement, register_arrangement


@register_arrangement("parallel_residual")
class ParallelResidual(Arrangement):
    ROLES = {"norm": ("norm", True), "mixer": ("mixer", True), "feed_forward": ("feed_forward", False),
             "mixer_scale": ("scale", False), "ffn_scale": ("scale", False), "side": ("side", False)}

    def __init__(self, layer):
        super().__init__(layer)
        if self.ffn_scale is not None and self.feed_forward is None:
            raise ValueError("arrangement 'parallel_residual': a feed-forward scale without a feed-forward")

    def forward(self, ctx, x, pending, cache):
        h = self.norm.forward(ctx, x, delta=pending)
        y = self.mixer.forward(ctx, h, cache)
        f = self.feed_forward.forward(ctx, h) if self.feed_forward is not None else None
        # (the side input's first product reads the new stream in the products' dtype: the sum writes that copy too)
        rounded = mixing.scaled_add_(x, y, None if self.mixer_scale is None else self.mixer_scale.weight,
                                     f, None if self.ffn_scale is None else self.ffn_scale.weight,
                                     copy_dtype=ctx.precision.act_dtype if self.side is not None else None)
        if self.side is not None:
            self.side.forward(ctx, x, rounded)
        return x, None
