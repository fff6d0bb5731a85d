"""Two mixers side by side on one input: half the sum of their outputs, each brought to unit root
mean square over the model width and multiplied by a weight of its own first,

    y = 0.5 (w_left * unit(left(h)) + w_right * unit(right(h)))

The two may be of any registered kinds; between them they keep at most one set of pages and one
fixed-size state (an attention beside a recurrence), which the cache manager serves through the layer's
one ``LayerCache``.
"""
from __future__ import annotations

from ..kernels import mixing
from ..weights.loader import TensorDecl
from .base import FixedState, Mixer, PagedKV, Precision, build_mixer, register_mixer


@register_mixer("mixer_pair")
class MixerPair(Mixer):
    """params: hidden_size, eps, left, right (``PartSpec`` of a mixer each).  tensors: left_out, right_out
    [H]: the weights of the two output norms."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.eps = float(self.params["eps"])
        self.left = build_mixer(self.params["left"])
        self.right = build_mixer(self.params["right"])
        self.graph_safe = bool(self.left.graph_safe and self.right.graph_safe)
        specs = self.state_spec()
        specs = specs if isinstance(specs, tuple) else (() if specs is None else (specs,))
        for kind in (PagedKV, FixedState):
            if sum(isinstance(s, kind) for s in specs) > 1:
                raise ValueError("the two halves of a mixer pair may keep one set of pages and one fixed state "
                                 f"between them, not two {kind.__name__}")
        self.w_left = self.w_right = None

    def _halves(self):
        return (self.left, self.right)

    def declare(self):
        out = {self.names["left_out"]: TensorDecl((self.hidden,), "norm"),
               self.names["right_out"]: TensorDecl((self.hidden,), "norm")}
        for half in self._halves():
            out.update(half.declare())
        return out

    def bind(self, get, precision: Precision, device):
        for half in self._halves():
            half.bind(get, precision, device)
        self.w_left = precision.vector(get(self.names["left_out"]), device)
        self.w_right = precision.vector(get(self.names["right_out"]), device)

    def weight_bytes(self):
        return sum(half.weight_bytes() for half in self._halves()) + 8 * self.hidden

    def active_weight_bytes(self, n_tokens):
        return sum(half.active_weight_bytes(n_tokens) for half in self._halves()) + 8 * self.hidden

    def flops_per_token(self):
        return sum(half.flops_per_token() for half in self._halves())

    def context_flops(self, n_tokens):
        return sum(half.context_flops(n_tokens) for half in self._halves())

    def state_spec(self):
        specs = []
        for half in self._halves():
            spec = half.state_spec()
            if spec is not None:
                specs.extend(spec if isinstance(spec, tuple) else (spec,))
        if not specs:
            return None
        return specs[0] if len(specs) == 1 else tuple(specs)

    def prepare(self, max_positions, device):
        for half in self._halves():
            half.prepare(max_positions, device)

    def forward(self, ctx, h, cache):
        a = self.left.forward(ctx, h, cache)
        b = self.right.forward(ctx, h, cache)
        return mixing.pair_norm_mean(a, self.w_left, b, self.w_right, self.eps)
