"""Mixture-of-experts feed-forward with a grouped, bias-corrected softmax router and identity experts.

Router scores s = softmax(W_router h) over all router outputs, in fp32.  The choice is made on s +
correction: the outputs form ``groups`` equal runs of neighbours, only the ``keep_groups`` runs with
the largest choice value stay in the race, and the ``top`` largest survivors are chosen; the weights
are the plain s of the chosen, not renormalised.  The first ``experts`` outputs are small gated
feed-forwards, down(act(gate h) * (up h)); the ``identity`` outputs behind them hand h itself on.  The
result is the weighted sum over the chosen.
"""
from __future__ import annotations

import torch

from ..kernels import experts as expert_kernels
from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, Precision, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """params: hidden_size, ffn_dim (of one expert), experts, identity (0), top, groups (1), keep_groups
    (1), activation ("silu").  tensors: router [experts + identity][H], correction [experts + identity],
    and per expert j ``gate{j}``, ``up{j}`` [F][H], ``down{j}`` [H][F]."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.ffn_dim = int(p["ffn_dim"])
        self.n_experts = int(p["experts"])
        self.n_identity = int(p.get("identity", 0) or 0)
        self.top = int(p["top"])
        self.groups = int(p.get("groups", 1) or 1)
        self.keep_groups = int(p.get("keep_groups", self.groups) or self.groups)
        self.activation = str(p.get("activation", "silu"))
        outputs = self.n_experts + self.n_identity
        if self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"unknown gate activation {self.activation!r}")
        if self.n_experts < 0 or self.n_identity < 0 or outputs <= 0:
            raise ValueError("a router needs at least one output")
        if outputs % self.groups or not 0 < self.keep_groups <= self.groups:
            raise ValueError(f"{outputs} router outputs do not form {self.groups} equal groups of which "
                             f"{self.keep_groups} are kept")
        if not 0 < self.top <= self.keep_groups * (outputs // self.groups):
            raise ValueError(f"top {self.top} does not fit the {self.keep_groups} kept groups")
        self.router = self.correction = self.w_gate_up = self.w_down = None

    @property
    def n_outputs(self) -> int:
        return self.n_experts + self.n_identity

    def declare(self):
        n, H, F = self.names, self.hidden, self.ffn_dim
        out = {n["router"]: TensorDecl((self.n_outputs, H)), n["correction"]: TensorDecl((self.n_outputs,), "bias")}
        for j in range(self.n_experts):
            out[n[f"gate{j}"]] = TensorDecl((F, H))
            out[n[f"up{j}"]] = TensorDecl((F, H))
            out[n[f"down{j}"]] = TensorDecl((H, F))
        return out

    def bind(self, get, precision: Precision, device):
        n = self.names
        # the router runs in fp32 whatever the precision (a bfloat16 matrix widens exactly)
        self.router = precision.vector(get(n["router"]), device)
        self.correction = precision.vector(get(n["correction"]), device)
        mats = [get(n[f"{role}{j}"]) for j in range(self.n_experts) for role in ("gate", "up", "down")]
        dtype = torch.float32 if (precision.name == "float32" or len({m.dtype for m in mats}) > 1) \
            else (mats[0].dtype if mats else precision.act_dtype)
        H, F, E = self.hidden, self.ffn_dim, self.n_experts
        if E:
            # [E][gate rows | up rows][H] and [E][H][F]: one stacked tensor per product
            gate_up = torch.stack([torch.cat([get(n[f"gate{j}"]).to(dtype), get(n[f"up{j}"]).to(dtype)], dim=0)
                                   for j in range(E)])
            down = torch.stack([get(n[f"down{j}"]).to(dtype) for j in range(E)])
        else:
            gate_up, down = torch.empty((0, 2 * F, H), dtype=dtype), torch.empty((0, H, F), dtype=dtype)
        self.w_gate_up = gate_up.to(device).contiguous()
        self.w_down = down.to(device).contiguous()

    def weight_bytes(self):
        # what a step reads at most: the router, and the experts its tokens choose (all of them, from
        # enough tokens on)
        return (self.router.numel() * 4 + self.w_gate_up.numel() * self.w_gate_up.element_size()
                + self.w_down.numel() * self.w_down.element_size())

    def active_weight_bytes(self, n_tokens):
        chosen = min(self.n_experts, n_tokens * self.top)
        per_expert = 3 * self.ffn_dim * self.hidden * self.w_gate_up.element_size()
        return self.router.numel() * 4 + chosen * per_expert

    def flops_per_token(self):
        return 2.0 * self.router.numel() + 2.0 * self.top * 3 * self.ffn_dim * self.hidden

    def forward(self, ctx, h, add_normed_into=None):
        ids, weights = expert_kernels.route(h, self.router, self.correction, self.groups, self.keep_groups, self.top)
        if h.dtype != self.w_gate_up.dtype:
            h = ops.cast(h, self.w_gate_up.dtype)
        return expert_kernels.experts_forward(h, ids, weights, self.w_gate_up, self.w_down, self.activation,
                                              add_normed_into)

    def forward_add_normed(self, ctx, h, x, norm_weight, eps):
        """``x += norm_weight * unit(ff(h))`` with the weighted sum, the output norm and the residual sum in
        one kernel (an arrangement with a norm on the sublayer's output asks for it)."""
        self.forward(ctx, h, add_normed_into=(x, norm_weight, eps))


@register_feed_forward("table_experts")
class TableExperts(FeedForward):
    """Experts chosen by the token's id instead of a router: row ``id`` of an integer table names the
    token's ``top`` experts (the entries of a row differ), each counts 1 / top, and the result is the sum;
    an optional shared expert of its own width runs for every token and is added.  Every expert is a gated
    feed-forward ``down(act(gate h, up h))`` without biases.

    params: hidden_size, vocab_size, ffn_dim (of one expert), experts, top, activation ("silu", "gelu_tanh" or
    "swish_clamped"), limit (of "swish_clamped"), and optionally shared_ffn_dim (> 0: there is a shared expert)
    with shared_limit.  tensors: table [vocab][top] (integers), per expert j ``gate{j}``, ``up{j}`` [F][H],
    ``down{j}`` [H][F], and ``shared_gate``, ``shared_up`` [Fs][H], ``shared_down`` [H][Fs]."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.vocab = int(p["vocab_size"])
        self.ffn_dim = int(p["ffn_dim"])
        self.n_experts = int(p["experts"])
        self.top = int(p["top"])
        self.activation = str(p.get("activation", "silu"))
        self.limit = float(p.get("limit", 0.0) or 0.0)
        self.shared_ffn = int(p.get("shared_ffn_dim", 0) or 0)
        self.shared_limit = float(p.get("shared_limit", self.limit) or 0.0)
        if self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"unknown gate activation {self.activation!r}")
        if not 0 < self.top <= self.n_experts:
            raise ValueError(f"top {self.top} of {self.n_experts} experts")
        if self.activation == "swish_clamped" and (self.limit <= 0 or (self.shared_ffn and self.shared_limit <= 0)):
            raise ValueError("the clamped swish needs a positive limit")
        self.table = self.w_gate_up = self.w_down = self.shared_gate_up = self.shared_down = None

    def declare(self):
        n, H, F = self.names, self.hidden, self.ffn_dim
        out = {n["table"]: TensorDecl((self.vocab, self.top), "table", bound=self.n_experts)}
        for j in range(self.n_experts):
            out[n[f"gate{j}"]] = TensorDecl((F, H))
            out[n[f"up{j}"]] = TensorDecl((F, H))
            out[n[f"down{j}"]] = TensorDecl((H, F))
        if self.shared_ffn:
            out[n["shared_gate"]] = TensorDecl((self.shared_ffn, H))
            out[n["shared_up"]] = TensorDecl((self.shared_ffn, H))
            out[n["shared_down"]] = TensorDecl((H, self.shared_ffn))
        return out

    def bind(self, get, precision: Precision, device):
        n = self.names
        table = get(n["table"]).to(torch.int32)
        if int(table.min()) < 0 or int(table.max()) >= self.n_experts:
            raise ValueError(f"{n['table']} names an expert outside [0, {self.n_experts})")
        self.table = table.to(device).contiguous()
        mats = [get(n[f"{role}{j}"]) for j in range(self.n_experts) for role in ("gate", "up", "down")]
        dtype = torch.float32 if (precision.name == "float32" or len({m.dtype for m in mats}) > 1) else mats[0].dtype
        # [E][gate rows | up rows][H] and [E][H][F]: one stacked tensor per product
        self.w_gate_up = torch.stack([torch.cat([get(n[f"gate{j}"]).to(dtype), get(n[f"up{j}"]).to(dtype)], dim=0)
                                      for j in range(self.n_experts)]).to(device).contiguous()
        self.w_down = torch.stack([get(n[f"down{j}"]).to(dtype) for j in range(self.n_experts)]).to(device).contiguous()
        if self.shared_ffn:
            gate, up = get(n["shared_gate"]), get(n["shared_up"])
            if gate.dtype != up.dtype:
                gate, up = gate.to(torch.float32), up.to(torch.float32)
            self.shared_gate_up = precision.matrix(torch.cat([gate, up], dim=0), device)
            self.shared_down = precision.matrix(get(n["shared_down"]), device)

    def _shared_bytes(self):
        if not self.shared_ffn:
            return 0
        return (self.shared_gate_up.numel() * self.shared_gate_up.element_size()
                + self.shared_down.numel() * self.shared_down.element_size())

    def weight_bytes(self):
        return (self.table.numel() * 4 + self._shared_bytes()
                + self.w_gate_up.numel() * self.w_gate_up.element_size()
                + self.w_down.numel() * self.w_down.element_size())

    def active_weight_bytes(self, n_tokens):
        chosen = min(self.n_experts, n_tokens * self.top)
        per_expert = 3 * self.ffn_dim * self.hidden * self.w_gate_up.element_size()
        return n_tokens * self.top * 4 + chosen * per_expert + self._shared_bytes()

    def flops_per_token(self):
        return 2.0 * 3 * self.hidden * (self.top * self.ffn_dim + self.shared_ffn)

    def _shared_hidden(self, ctx, h):
        """act(gate h, up h) of the shared expert, in the products' dtype."""
        from ..kernels import tensorcore
        act = ctx.precision.act_dtype
        if tensorcore.swiglu_accepts(h, self.shared_gate_up):
            return tensorcore.swiglu_gate_up(h, self.shared_gate_up, activation=self.activation,
                                             limit=self.shared_limit)
        gate_up = ops.linear(h, self.shared_gate_up, torch.float32)
        return ops.gate_act_mul(gate_up, act, self.activation, self.shared_limit)

    def forward(self, ctx, h):
        ids, weights = expert_kernels.route_table(ctx.batch.token_ids, self.table, self.top)
        rows = h if h.dtype == self.w_gate_up.dtype else ops.cast(h, self.w_gate_up.dtype)
        out = expert_kernels.experts_forward(rows, ids, weights, self.w_gate_up, self.w_down, self.activation,
                                             limit=self.limit)
        if self.shared_ffn:
            a = self._shared_hidden(ctx, h)
            rest = ops.linear_into_residual(a, self.shared_down, out)      # out += down(a) where the product can
            if rest is not None:
                ops.add_(out, rest)
        return out

    def forward_add_normed(self, ctx, h, x, norm_weight, eps):
        """``x += norm_weight * unit(ff(h))``: the shared expert first, then the experts' weighted sum, the shared
        output, the output norm and the residual sum in one kernel."""
        shared = None
        if self.shared_ffn:
            shared = ops.linear(self._shared_hidden(ctx, h), self.shared_down, torch.float32)
        ids, weights = expert_kernels.route_table(ctx.batch.token_ids, self.table, self.top)
        rows = h if h.dtype == self.w_gate_up.dtype else ops.cast(h, self.w_gate_up.dtype)
        expert_kernels.experts_forward(rows, ids, weights, self.w_gate_up, self.w_down, self.activation,
                                       add_normed_into=(x, norm_weight, eps, shared), limit=self.limit)
