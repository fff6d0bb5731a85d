"""A per-layer input from the token ids: every layer owns a slice of a second, narrow embedding table and
adds, behind its sublayers,

    e = table[token];   g = gelu_tanh(W_gate x) * e;   y = W_proj g;   x <- x + w * y / rms(y)

with x the residual stream as the sublayers left it.  The gate, the norm and the sum are fp32.
"""
from __future__ import annotations

import torch

from ..kernels import mixing, ops
from ..weights.loader import TensorDecl
from .base import Precision, SideInput, register_side_input


@register_side_input("token_side_input")
class TokenSideInput(SideInput):
    """params: hidden_size, vocab_size, dim (entries of a token's slice), index and count (which slice of
    how many the table's rows hold), eps.  tensors: table [vocab][count dim], gate [dim][H], proj
    [H][dim], norm [H]."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.vocab = int(p["vocab_size"])
        self.dim = int(p["dim"])
        self.index = int(p["index"])
        self.count = int(p["count"])
        self.eps = float(p["eps"])
        if self.dim <= 0 or not 0 <= self.index < self.count:
            raise ValueError("token side input: dim must be positive and index one of the table's slices")
        self.table = self.w_gate = self.w_proj = self.norm = None

    def declare(self):
        n, H = self.names, self.hidden
        return {n["table"]: TensorDecl((self.vocab, self.count * self.dim), "embedding"),
                n["gate"]: TensorDecl((self.dim, H)), n["proj"]: TensorDecl((H, self.dim)),
                n["norm"]: TensorDecl((H,), "norm")}

    def bind(self, get, precision: Precision, device):
        n = self.names
        # this layer's columns of the table only: the layers' slices together are the table once
        lo = self.index * self.dim
        self.table = precision.matrix(get(n["table"])[:, lo:lo + self.dim].contiguous(), device)
        self.w_gate = precision.matrix(get(n["gate"]), device)
        self.w_proj = precision.matrix(get(n["proj"]), device)
        self.norm = precision.vector(get(n["norm"]), device)

    def weight_bytes(self):
        return (self.w_gate.numel() * self.w_gate.element_size() + self.w_proj.numel() * self.w_proj.element_size()
                + 4 * self.hidden)

    def flops_per_token(self):
        return 2.0 * (self.w_gate.numel() + self.w_proj.numel())

    def forward(self, ctx, x, x_act=None):
        act = ctx.precision.act_dtype
        g = ops.linear(x_act if x_act is not None else ops.cast(x, act), self.w_gate, torch.float32)
        a = mixing.side_gate(g, self.table, 0, ctx.batch.token_ids, act)
        y = ops.linear(a, self.w_proj, torch.float32)
        ops.rmsnorm_add_(x, y, self.norm, self.eps)
