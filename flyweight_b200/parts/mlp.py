"""Dense feed-forward without a gate: down( act(up h) ), no bias.  ``act`` is a parameter: the square of
relu, silu, or the tanh form of gelu.  The activation is computed in fp32 on the product's fp32 output."""
from __future__ import annotations

import torch

from ..kernels import mixing, ops
from ..weights.loader import TensorDecl
from .base import FeedForward, Precision, register_feed_forward


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    """params: hidden_size, ffn_dim, activation ("relu_squared" | "silu" | "gelu_tanh").
    tensors: up [F][H], down [H][F]."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.ffn_dim = int(self.params["ffn_dim"])
        self.activation = str(self.params.get("activation", "relu_squared"))
        if self.activation not in mixing.UNARY_ACTIVATIONS or self.activation == "sigmoid":
            raise ValueError(f"unknown feed-forward activation {self.activation!r}; known: relu_squared, silu, gelu_tanh")
        self.w_up = self.w_down = None

    def declare(self):
        n, H, F = self.names, self.hidden, self.ffn_dim
        return {n["up"]: TensorDecl((F, H)), n["down"]: TensorDecl((H, F))}

    def bind(self, get, precision: Precision, device):
        self.w_up = precision.matrix(get(self.names["up"]), device)
        self.w_down = precision.matrix(get(self.names["down"]), device)

    def weight_bytes(self):
        return (self.w_up.numel() * self.w_up.element_size() + self.w_down.numel() * self.w_down.element_size())

    def flops_per_token(self):
        return 2.0 * (self.w_up.numel() + self.w_down.numel())

    def forward(self, ctx, h):
        act = ctx.precision.act_dtype
        if not isinstance(h, torch.Tensor):
            h = h.materialize(act)
        # (the hidden row leaves its product in the products' dtype; the activation itself is computed in fp32)
        a = mixing.unary_act(ops.linear(h, self.w_up, act), self.activation, act)
        return ops.linear(a, self.w_down, torch.float32)
