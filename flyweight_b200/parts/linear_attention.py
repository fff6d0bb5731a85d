"""Linear attention with a fixed decay per head (lightning attention): a recurrence whose state is one
[dim][vdim] matrix per head and request.

Per token, with h the mixer's input:  q = act(W_q h), k = act(W_k h) (heads x dim), v = act(W_v h) (heads x
vdim), act = silu; per head

    S <- decay_h S + k v^T;     o = S^T q

and the output is ``W_o( w * o / rms(o) * sigmoid(W_g h) )`` with the root mean square over all heads of a
token together.  S lives in the request's state slot (fp32, zero at admission), so a sequence may be cut
into steps anywhere.  One fused projection q|k|v|gate leaves its product in fp32; the activations, the
recurrence, the norm and the gate are computed in 32-bit in both precisions.
"""
from __future__ import annotations

import torch

from ..kernels import mixing, ops
from ..weights.loader import TensorDecl
from .base import FixedState, Mixer, Precision, register_mixer


@register_mixer("decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    """params: hidden_size, num_heads, dim, vdim, decay (one number per head), eps (of the output's norm).
    tensors: q, k [heads dim][H]; v, g [heads vdim][H]; norm [heads vdim]; o [H][heads vdim]."""
    graph_safe = True
    RUNS_FROM = 16      # the longest portion of a step from which the tensor-core form takes the step

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.eps = float(p["eps"])
        self.decay_values = [float(x) for x in p["decay"]]
        if min(self.n_heads, self.dim, self.vdim) <= 0:
            raise ValueError("linear attention: heads, dim and vdim must be positive")
        if len(self.decay_values) != self.n_heads:
            raise ValueError(f"linear attention: {len(self.decay_values)} decays for {self.n_heads} heads")
        self.w_in = self.w_o = self.norm = self.decay = None

    @property
    def _qk(self) -> int:
        return self.n_heads * self.dim

    @property
    def _v(self) -> int:
        return self.n_heads * self.vdim

    def declare(self):
        n, H = self.names, self.hidden
        return {n["q"]: TensorDecl((self._qk, H)), n["k"]: TensorDecl((self._qk, H)),
                n["v"]: TensorDecl((self._v, H)), n["g"]: TensorDecl((self._v, H)),
                n["norm"]: TensorDecl((self._v,), "norm"), n["o"]: TensorDecl((H, self._v))}

    def bind(self, get, precision: Precision, device):
        n = self.names
        mats = [get(n[name]) for name in ("q", "k", "v", "g")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.to(torch.float32) for m in mats]
        # one projection: the rows of the four matrices, one after the other
        self.w_in = precision.matrix(torch.cat(mats, dim=0), device)
        self.w_o = precision.matrix(get(n["o"]), device)
        self.norm = precision.vector(get(n["norm"]), device)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)

    def weight_bytes(self):
        return self.w_in.numel() * self.w_in.element_size() + self.w_o.numel() * self.w_o.element_size()

    def flops_per_token(self):
        # the products, and per head two passes over the [dim][vdim] state (decay and write, read-out)
        return 2.0 * (self.w_in.numel() + self.w_o.numel()) + 4.0 * self.n_heads * self.dim * self.vdim

    def state_spec(self):
        # (slots start on 16-byte borders)
        return FixedState((-(-self.n_heads * self.dim * self.vdim // 4) * 4,))

    def forward(self, ctx, h, cache):
        p = ops.linear(h, self.w_in, torch.float32)
        # portions of prompts in bfloat16 walk 64 tokens at a time on tensor cores (q, k, v rounded to bfloat16,
        # the state and the sums in fp32); single tokens, short portions and 32-bit runs go token by token
        runs = (ctx.precision.act_dtype == torch.bfloat16 and self.dim <= 256
                and getattr(ctx.batch, "max_segment", 1) >= self.RUNS_FROM)
        o = (mixing.decay_runs if runs else mixing.decay_scan)(
            p, 0, self._qk, 2 * self._qk, self.decay, cache.state, ctx.batch, self.n_heads, self.dim, self.vdim,
            act_silu=True)
        gate_at = 2 * self._qk + self._v
        z = mixing.gated_rmsnorm(o, p[:, gate_at:gate_at + self._v], self.norm, self.eps, ctx.precision.act_dtype)
        return ops.linear(z, self.w_o, torch.float32)
