"""Grouped-query attention mixer with per-head q/k RMSNorm and rotary positions.

Order of operations (native/src/v2_runtime.cpp:28429-28478): q, k, v projections
without bias; RMSNorm over each head of q and of k with a [head_dim] weight shared by
all heads; rotary encoding of q and k; k and v appended to the cache; scores of query
head j against KV head j // (heads / kv_heads), scaled by head_dim^-1/2, causal,
softmax in fp32; output projection without gate.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import FixedState, Mixer, PagedKV, Precision, build_position, register_mixer


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm_eps (None: no
    q/k norm), position (PartSpec of a position encoding), window (0: all keys),
    shares_cache (True: reads the cache of another execution and projects q only).
    tensors: q, k, v, o, q_norm, k_norm.

    Further params, all optional: ``scale`` (head_dim^-1/2 when absent); ``chunk`` (> 0: the sequence
    is cut into runs of that many positions counted from position 0, and a query sees only the keys of
    its own run up to itself); ``qk_unit_rms_eps`` (not None: instead of the weighted norm in front of
    the rotation, every head of q and k is brought to unit root mean square behind it, without a
    weight; no ``q_norm``/``k_norm`` tensors); ``value_dim`` (the size of a value head when it differs
    from ``head_dim``: the pools and kernels then run at the larger of the two, the smaller heads padded
    with zero channels through zero rows and columns of the matrices); ``qk_norm`` ("head", the default:
    one weight of ``head_dim`` entries shared by the heads, the mean over each head; "whole": the RMS norm
    goes over all heads of q (and of k) at once, before they are split, with weights of the whole
    projection's size); ``sink`` (True: tensor ``sink`` [heads], a score per head that joins every softmax
    denominator without a value, neither scaled nor capped; "zero": that score is 0 for every head and there
    is no tensor, i.e. the denominator is one larger); ``conv`` (n > 0: a causal convolution of n taps over
    time on every channel of q, k and v right behind their projection, tensors ``q_conv``, ``k_conv``,
    ``v_conv`` [channels][n], the last tap on the token itself; a request's last n - 1 projected rows are
    kept in a ``FixedState`` beside the pages); ``softcap`` (> 0: score <- cap tanh(score /
    cap) behind the scale); ``gate`` ("head": tensor ``g`` [heads][H], every head's output times
    sigmoid(g h) of its head; "element": ``g`` [heads value_dim][H], channel by channel; both read the
    mixer's input); ``value_mix`` ("source": this layer's values, as cached, are also handed on to later
    layers of the step under ``value_mix_key``; "mixed": v <- (1 - lam) v + lam v_source with the
    tensor ``vmix``, one number, before v is cached)."""
    graph_safe = True
    takes_deferred_norm = True
    adds_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.eps = p.get("qk_norm_eps")
        self.window = int(p.get("window", 0) or 0)
        self.shares_cache = bool(p.get("shares_cache", False))
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.position = build_position(p["position"])
        self.chunk = int(p.get("chunk", 0) or 0)
        self.unit_rms_eps = p.get("qk_unit_rms_eps")
        # what the checkpoint's matrices have per head, and what the pools and kernels run at
        self.qk_dim = self.head_dim
        self.value_dim = int(p.get("value_dim", self.head_dim) or self.head_dim)
        if self.n_heads % self.n_kv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.chunk and self.window:
            raise ValueError("an attention mixer has a sliding window or chunks, not both")
        if self.unit_rms_eps is not None and self.eps is not None:
            raise ValueError("an attention mixer norms q and k in front of the rotation or behind it, not both")
        if self.value_dim != self.qk_dim or self.unit_rms_eps is not None or self.chunk:
            self.head_dim = -(-max(self.qk_dim, self.value_dim) // 16) * 16
        self.qk_norm = str(p.get("qk_norm", "head"))
        if self.qk_norm not in ("head", "whole"):
            raise ValueError(f"unknown q/k norm {self.qk_norm!r}; known: head, whole")
        if self.qk_norm == "whole" and self.eps is None:
            raise ValueError("a q/k norm over the whole projection needs qk_norm_eps")
        self.has_sink = bool(p.get("sink", False))
        self.zero_sink = p.get("sink") == "zero"
        self.conv_taps = int(p.get("conv", 0) or 0)
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        self.gate = p.get("gate")
        if self.gate not in (None, "head", "element"):
            raise ValueError(f"unknown output gate {self.gate!r}; known: head, element")
        self.value_mix = p.get("value_mix")
        if self.value_mix not in (None, "source", "mixed"):
            raise ValueError(f"unknown value mixing role {self.value_mix!r}; known: source, mixed")
        self.value_mix_key = str(p.get("value_mix_key", "values"))
        if self.value_mix and self.shares_cache:
            raise ValueError("a mixer that reads another's cache has no values of its own to mix")
        if self.softcap < 0:
            raise ValueError("softcap must not be negative")
        if self.value_dim != self.qk_dim or self.qk_dim % 16:
            self.head_dim = -(-max(self.qk_dim, self.value_dim) // 16) * 16
        # the launches LFM2 makes: nothing of the above, so the fused decode kernel and the native plan apply
        self._plain = not (self.has_sink or self.softcap or self.gate or self.value_mix or self.conv_taps
                           or self.qk_norm == "whole" or (self.head_dim != self.qk_dim and self.eps is not None))
        # q|k|v leave their product in fp32 when a norm over the whole projection works on them in place before
        # the head kernel reads them: one rounding, not two.  (Mixed values are rounded on both sides of the
        # mix in 16-bit runs: what the products' dtype means for a projection and for a cached value.)
        self._wide_qkv = self.qk_norm == "whole"
        # a gate per head behind a convolution: its rows ride in the q|k|v product (the convolution writes a
        # buffer of its own, so the gate's columns stay where the product left them)
        self._gate_in_projection = self.gate == "head" and self.conv_taps > 0
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.w_gate = self.sink = self.vmix = None
        self.taps = None

    @property
    def _kv_in(self) -> int:
        return 0 if self.shares_cache else self.n_kv

    def declare(self):
        n, hd, H = self.names, self.qk_dim, self.hidden
        out = {n["q"]: TensorDecl((self.n_heads * hd, H)),
               n["o"]: TensorDecl((H, self.n_heads * self.value_dim))}
        if not self.shares_cache:
            out[n["k"]] = TensorDecl((self.n_kv * hd, H))
            out[n["v"]] = TensorDecl((self.n_kv * self.value_dim, H))
        if self.eps is not None:
            whole = self.qk_norm == "whole"
            out[n["q_norm"]] = TensorDecl((self.n_heads * hd if whole else hd,), "norm")
            if not self.shares_cache:
                out[n["k_norm"]] = TensorDecl((self.n_kv * hd if whole else hd,), "norm")
        if self.has_sink and not self.zero_sink:
            out[n["sink"]] = TensorDecl((self.n_heads,), "bias")
        if self.conv_taps:
            out[n["q_conv"]] = TensorDecl((self.n_heads * hd, self.conv_taps), "taps")
            if not self.shares_cache:
                out[n["k_conv"]] = TensorDecl((self.n_kv * hd, self.conv_taps), "taps")
                out[n["v_conv"]] = TensorDecl((self.n_kv * self.value_dim, self.conv_taps), "taps")
        if self.gate:
            out[n["g"]] = TensorDecl((self.n_heads * (self.value_dim if self.gate == "element" else 1), H))
        if self.value_mix == "mixed":
            out[n["vmix"]] = TensorDecl((), "bias", also=((1,),))
        return out

    def bind(self, get, precision: Precision, device):
        n = self.names
        D = self.head_dim

        def rows_padded(matrix, per_head):
            """[heads * per_head][H] -> [heads * D][H]: zero rows behind every head's own."""
            if per_head == D:
                return matrix
            heads = matrix.shape[0] // per_head
            wide = matrix.new_zeros((heads, D, matrix.shape[1]))
            wide[:, :per_head] = matrix.view(heads, per_head, -1)
            return wide.view(heads * D, -1)

        mats = [rows_padded(get(n["q"]), self.qk_dim)]
        if not self.shares_cache:
            mats += [rows_padded(get(n["k"]), self.qk_dim), rows_padded(get(n["v"]), self.value_dim)]
        self._qkv_columns = sum(m.shape[0] for m in mats)
        if self._gate_in_projection:
            gate_rows = get(n["g"])
            pad = -gate_rows.shape[0] % 8                     # (a row count the products' tiles like)
            mats += [gate_rows] + ([gate_rows.new_zeros((pad, gate_rows.shape[1]))] if pad else [])
        dtypes = {m.dtype for m in mats}
        if len(dtypes) > 1:
            mats = [m.to(torch.float32) for m in mats]
        # one projection for q|k|v (|gate): the rows of the matrices, one after the other
        self.w_qkv = precision.matrix(torch.cat(mats, dim=0), device)
        w_o = get(n["o"])
        if self.value_dim != D:                   # zero columns where the padded channels of a head arrive
            wide = w_o.new_zeros((w_o.shape[0], self.n_heads, D))
            wide[:, :, :self.value_dim] = w_o.view(w_o.shape[0], self.n_heads, self.value_dim)
            w_o = wide.view(w_o.shape[0], self.n_heads * D)
        self.w_o = precision.matrix(w_o, device)
        def channels_padded(vector, per_head):
            """[heads * per_head] -> [heads * D]: zeros behind every head's own channels."""
            if per_head == D:
                return vector
            wide = vector.new_zeros((vector.numel() // per_head, D))
            wide[:, :per_head] = vector.view(-1, per_head)
            return wide.reshape(-1)

        if self.eps is not None:
            self.q_norm = precision.vector(channels_padded(get(n["q_norm"]), self.qk_dim), device)
            if not self.shares_cache:
                self.k_norm = precision.vector(channels_padded(get(n["k_norm"]), self.qk_dim), device)
        if self.has_sink:
            self.sink = (torch.zeros(self.n_heads, dtype=torch.float32, device=device) if self.zero_sink
                         else precision.vector(get(n["sink"]), device))
        if self.conv_taps:
            # the taps of q | k | v in the fused projection's channel order (zero taps on padding channels)
            taps = [rows_padded(get(n["q_conv"]), self.qk_dim)]
            if not self.shares_cache:
                taps += [rows_padded(get(n["k_conv"]), self.qk_dim), rows_padded(get(n["v_conv"]), self.value_dim)]
            self.taps = precision.vector(torch.cat([t.to(torch.float32) for t in taps], dim=0), device)
        if self.gate and not self._gate_in_projection:
            w_gate = get(n["g"])
            self.w_gate = precision.matrix(rows_padded(w_gate, self.value_dim) if self.gate == "element" else w_gate,
                                           device)
        if self.value_mix == "mixed":
            self.vmix = precision.vector(get(n["vmix"]).reshape(1), device)

    def _matrices(self):
        return tuple(m for m in (self.w_qkv, self.w_o, self.w_gate) if m is not None)

    def weight_bytes(self):
        return sum(m.numel() * m.element_size() for m in self._matrices())

    def flops_per_token(self):
        return 2.0 * sum(m.numel() for m in self._matrices())

    def context_flops(self, n_tokens):
        # QK^T and PV: 4 operations per (query, visible key, channel); half the pairs are masked
        if self.window and n_tokens > self.window:
            pairs = n_tokens * self.window - 0.5 * self.window * self.window
            return 4.0 * pairs * self.n_heads * self.head_dim
        if self.chunk and n_tokens > self.chunk:
            whole, rest = divmod(n_tokens, self.chunk)
            return 2.0 * (whole * self.chunk * self.chunk + rest * rest) * self.n_heads * self.head_dim
        return 2.0 * n_tokens * n_tokens * self.n_heads * self.head_dim

    @property
    def span(self) -> int:
        """The mask parameter of the attention kernels: a window (> 0), chunks (< 0), or all keys."""
        return -self.chunk if self.chunk else self.window

    def _encode_extra(self) -> dict:
        if self.unit_rms_eps is None:
            # (heads padded with zero channels: the mean of a weighted head norm goes over the true size)
            return {"norm_dim": self.qk_dim} if self.head_dim != self.qk_dim and self.eps is not None else {}
        return {"unit_rms_after": True, "norm_dim": self.qk_dim}

    def state_spec(self):
        paged = None if self.shares_cache else PagedKV(self.n_kv, self.head_dim, self.window)
        if self.conv_taps > 1:
            channels = (self.n_heads + 2 * self._kv_in) * self.head_dim
            rolling = FixedState((self.conv_taps - 1, channels))
            return rolling if paged is None else (paged, rolling)
        return paged

    def prepare(self, max_positions, device):
        self.position.prepare(max_positions, device)

    def forward(self, ctx, h, cache, residual=None):
        act = ctx.precision.act_dtype
        if not self._plain:
            return self._forward_general(ctx, h, cache, residual)
        # q|k|v in the activation dtype; the head norm and the rotation widen it to fp32
        qkv = ops.linear(h, self.w_qkv, act)
        block_table = ctx.batch.block_tables[cache.group]
        from ..kernels import attention as attention_kernels
        rotation = self.position.rotation() if self.unit_rms_eps is None else None
        if rotation is not None and attention_kernels.decode_fusable(ctx, qkv, cache, block_table, self.n_heads, rotation[1], self.window):
            # a step of single tokens whose position part is a plain rotation: the decode attention
            # kernel norms, turns and stores its own token's heads (one kernel and one pass less)
            table, rotary_dim, pairing = rotation
            out = attention_kernels.fused_decode_attention(
                ctx, qkv, cache, block_table, self.n_heads, self._kv_in, self.window, self.scale,
                self.q_norm, self.k_norm, self.eps, table, rotary_dim, pairing)
            return ops.linear_into_residual(out, self.w_o, residual)
        # positions are the position part's business: it norms, encodes and writes the pages
        q = self.position.encode(ctx, qkv, n_heads=self.n_heads, n_kv_in=self._kv_in,
                                 head_dim=self.head_dim, q_norm=self.q_norm, k_norm=self.k_norm,
                                 eps=self.eps if self.unit_rms_eps is None else self.unit_rms_eps,
                                 cache=cache, block_table=block_table, **self._encode_extra())
        out = attention_kernels.paged_attention(ctx, q, cache, block_table, self.n_heads,
                                                self.span, self.scale, act)
        return ops.linear_into_residual(out, self.w_o, residual)

    def _forward_general(self, ctx, h, cache, residual=None):
        """The mixer with any of: a norm over the whole projection, padded heads under a weighted norm,
        mixed values, a sink, capped scores, an output gate."""
        from ..kernels import attention as attention_kernels
        from ..kernels import mixing
        act = ctx.precision.act_dtype
        if not isinstance(h, torch.Tensor):
            h = h.materialize(act)
        D = self.head_dim
        qkv = ops.linear(h, self.w_qkv, torch.float32 if self._wide_qkv else act)
        block_table = ctx.batch.block_tables[cache.group]
        k_at, v_at = self.n_heads * D, (self.n_heads + self._kv_in) * D
        whole = self.qk_norm == "whole"
        ranges = None
        if whole:
            ranges = [(0, self.q_norm, self.n_heads * self.qk_dim, self.eps)]
            if self._kv_in:
                ranges.append((k_at, self.k_norm, self.n_kv * self.qk_dim, self.eps))
        projected = qkv
        if self.conv_taps:
            # the convolution (and the norm over the whole of q and of k behind it, in the same launch)
            fused = ranges if self._qkv_columns * 4 <= 160 * 1024 else None
            qkv = mixing.causal_conv(projected, self.taps, cache.state if self.conv_taps > 1 else None, ctx.batch,
                                     norm_ranges=fused)
            if fused is not None:
                ranges = None
        if ranges is not None:
            mixing.rmsnorm_ranges_(qkv, ranges)
        if self.value_mix == "source":
            first = torch.empty((qkv.shape[0], self.n_kv * D), dtype=qkv.dtype, device=qkv.device)
            mixing.value_mix_(qkv, v_at, self.n_kv * D, first, None)
            ctx.shared[self.value_mix_key] = first
        elif self.value_mix == "mixed":
            first = ctx.shared.get(self.value_mix_key)
            if first is None or tuple(first.shape) != (qkv.shape[0], self.n_kv * D) or first.dtype != qkv.dtype:
                raise ValueError(f"no values of this step under {self.value_mix_key!r} that fit "
                                 f"{self.n_kv} value heads of {D}: the source layer runs first and has the same shape")
            mixing.value_mix_(qkv, v_at, self.n_kv * D, first, self.vmix)
        extra = self._encode_extra()
        q = self.position.encode(ctx, qkv, n_heads=self.n_heads, n_kv_in=self._kv_in, head_dim=D,
                                 q_norm=None if whole else self.q_norm, k_norm=None if whole else self.k_norm,
                                 eps=None if whole else (self.eps if self.unit_rms_eps is None else self.unit_rms_eps),
                                 cache=cache, block_table=block_table, **extra)
        out = attention_kernels.paged_attention(ctx, q, cache, block_table, self.n_heads, self.span, self.scale,
                                                act, sink=self.sink, softcap=self.softcap)
        if self._gate_in_projection:
            mixing.sigmoid_gate_cols_mul_(out, projected, self._qkv_columns, self.n_heads, D)
        elif self.gate:
            mixing.sigmoid_gate_mul_(out, ops.linear(h, self.w_gate, act), self.n_heads, D)
        return ops.linear_into_residual(out, self.w_o, residual)

    def plan(self, builder, norm, cache):
        """The same operations for the native step plan (``engine/plan.py``)."""
        from ..engine.plan import EPI_ACT, NotPlannable
        if not self._plain:
            raise NotPlannable("sinks, capped scores, gates, mixed values and norms over the whole projection "
                               "have no native plan form")
        act = builder.act_dtype
        plan_position = getattr(self.position, "plan", None)
        if self.unit_rms_eps is not None:
            raise NotPlannable("the q/k norm behind the rotation has no native plan form")
        if plan_position is None:
            raise NotPlannable(f"position encoding {self.position.kind!r} has no native form")
        width = self.n_heads * self.head_dim
        qkv = builder.tokens(width + 2 * self._kv_in * self.head_dim, act)
        builder.norm_linear(norm, self.w_qkv, EPI_ACT, qkv, "q|k|v")
        q = builder.tokens(width, act)
        plan_position(builder, qkv, q, n_heads=self.n_heads, n_kv_in=self._kv_in, head_dim=self.head_dim,
                      q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps, cache=cache)
        builder.free(qkv)
        out = builder.tokens(width, act)
        builder.attention(q, cache, out, self.n_heads, self.span, self.scale)
        builder.free(q)
        builder.linear_residual(out, self.w_o, "attention out_proj")
        builder.free(out)
