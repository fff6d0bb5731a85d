"""RMSNorm with a plain (not 1+w) weight, computed in fp32.

``(x * rsqrt(mean(x^2) + eps)) * w`` -- native/include/flyweight_v2_qwen_kernels.hpp:424-447,
called with one_centered=0 (native/src/v2_runtime.cpp:27741).  The residual sum that
precedes a norm in a block is folded into the same kernel.
"""
from __future__ import annotations

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import DeferredNorm, Norm, Precision, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: size, eps, and optionally ``gain``: one constant that multiplies the normed rows beside the
    weight (a model that adds ``m * norm(y)`` into its stream names m here; it is folded into the weight
    once, in fp32, when the weight is bound).  tensors: weight [size]."""
    graph_safe = True


    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.params["size"])
        self.eps = float(self.params["eps"])
        self.gain = float(self.params.get("gain", 1.0))
        self.weight = None

    def declare(self):
        return {self.names["weight"]: TensorDecl((self.size,), "norm")}

    def bind(self, get, precision: Precision, device):
        self.weight = precision.vector(get(self.names["weight"]), device)
        if self.gain != 1.0:
            self.weight = (self.weight * self.gain).contiguous()

    def weight_bytes(self):
        return self.size * 4

    def forward(self, ctx, x, delta=None, rows=None):
        return ops.rmsnorm(x, self.weight, self.eps, ctx.precision.act_dtype, delta=delta, rows=rows)

    def defer(self, ctx, x, rows=None):
        return DeferredNorm(x, self.weight, self.eps, rows)

    def plan_params(self):
        """(weight, eps): what the native step plan needs to run this norm in front of a product."""
        return self.weight, self.eps


@register_norm("rms_gain")
class RMSGain(Norm):
    """RMS norm with a single gain for all channels: ``g * x / sqrt(mean(x^2) + eps)``.
    params: size, eps.  tensors: weight [] (one number).

    In front of a product (``forward``, ``defer``) it is the ordinary RMS norm with the gain in every
    channel.  Behind a sublayer (``add_normed``) it adds the normed rows into the residual stream."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.params["size"])
        self.eps = float(self.params["eps"])
        self.gain = self.weight = None

    def declare(self):
        return {self.names["weight"]: TensorDecl((), "norm", also=((1,),))}

    def bind(self, get, precision: Precision, device):
        self.gain = precision.vector(get(self.names["weight"]).reshape(1), device)
        self.weight = self.gain.expand(self.size).contiguous()

    def weight_bytes(self):
        return 4

    def forward(self, ctx, x, delta=None, rows=None):
        return ops.rmsnorm(x, self.weight, self.eps, ctx.precision.act_dtype, delta=delta, rows=rows)

    def defer(self, ctx, x, rows=None):
        return DeferredNorm(x, self.weight, self.eps, rows)

    def plan_params(self):
        return self.weight, self.eps

    def add_normed(self, ctx, x, y, copy_dtype=None):
        """``x += g * y / sqrt(mean(y^2) + eps)`` in fp32, in place; with ``copy_dtype`` the new rows
        are also returned in that dtype."""
        from ..kernels import latent as latent_kernels
        return latent_kernels.unit_rms_gain_add_(x, y, self.gain, self.eps, copy_dtype)
