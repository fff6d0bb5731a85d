"""Attention over a cached low-rank latent, with a softmax sink.

Per token one projection gives ``rank + rot`` numbers: the first ``rank``, RMS-normed with a
weight, are the latent c; the last ``rot``, turned by the token's position, are a key part r that
every head shares.  Head h has the key ``(U_h c | r)`` and the value ``V_h c``; its query has
``dim`` plain channels and ``rot`` turned ones; the score is ``scale * (q_plain . U_h c + q_rot . r)``
and the causal softmax's denominator also holds ``exp(sink_h)``.  Only (c | r) is cached: one row per
token for all heads, and a layer may read the rows another layer wrote (``shares_cache``) with
projections U, V of its own.

How it is computed: ``q_plain . U_h c = (U_h^T q_plain) . c``, so every query head is turned into a
row ``(U_h^T q_plain | q_rot)`` of the cache row's layout, attention runs between many query heads
and the one cached row per token, with the row's first ``rank`` columns as values, and V_h is
applied to the weighted sum of latents afterwards.  Nothing per head is ever built for a cached
token, whether the step is a whole prompt, a portion or one token.

In bfloat16 that attention is the engine's paged attention with one pool head that every query head
reads and that serves as key and as value (tcgen05 for prompt portions, the split-context kernel for
single tokens), so the cached row is padded to a head size those kernels have (64 or 128 entries when
it fits, which gives prompts the tcgen05 kernel); the per-head products run on tensor cores too.
Rows longer than 128 entries, and the 32-bit path, run the fp32 kernel of ``csrc/latent_attention.cu``.
"""
from __future__ import annotations

import torch

from ..kernels import attention as attention_kernels
from ..kernels import latent as latent_kernels
from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Mixer, PagedKV, Precision, build_position, register_mixer


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """params: hidden_size, num_heads, dim (plain query/key channels per head), rot_dim (turned
    ones), vdim, kv_rank, scale, eps (of the latent's norm), position (PartSpec of a rotary encoding
    whose ``rotary_dim`` <= rot_dim), sink (True: a learned number per head joins the softmax
    denominator), shares_cache (True: reads the rows of another execution; no latent projection), gate
    ("head": tensor ``g`` [heads][H], every head's output times sigmoid(g h) of its head, from the mixer's
    own input).  tensors: q, dkv, dkv_norm, uk, uv, o, sink, g."""
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.dim = int(p["dim"])
        self.rot = int(p["rot_dim"])
        self.vdim = int(p["vdim"])
        self.rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.has_sink = bool(p.get("sink", False))
        self.shares_cache = bool(p.get("shares_cache", False))
        self.gate = p.get("gate")
        if self.gate not in (None, "head"):
            raise ValueError(f"unknown output gate {self.gate!r}; known: head")
        self.position = build_position(p["position"])
        if self.position.rotary_dim > self.rot:
            raise ValueError(f"{self.position.rotary_dim} turning channels but a rotated part of {self.rot}")
        if min(self.n_heads, self.dim, self.vdim, self.rank) <= 0 or self.rot < 0:
            raise ValueError("latent attention: heads, dim, vdim and kv_rank must be positive")
        # a cache row: latent, turned key part, zero padding up to a multiple of 16 entries -- up to 64 or
        # 128 where that is near: the head sizes that every tensor-core attention kernel takes
        used = self.rank + self.rot
        self.row = 64 if used <= 64 else (128 if 96 < used <= 128 else _round_up(used, 16))
        self.q_width = self.n_heads * (self.dim + self.rot)
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.norm_w = self.sink = self.w_gate = None

    def declare(self):
        n, H = self.names, self.hidden
        out = {n["q"]: TensorDecl((self.q_width, H)),
               n["uk"]: TensorDecl((self.n_heads * self.dim, self.rank)),
               n["uv"]: TensorDecl((self.n_heads * self.vdim, self.rank)),
               n["o"]: TensorDecl((H, self.n_heads * self.vdim))}
        if not self.shares_cache:
            out[n["dkv"]] = TensorDecl((self.rank + self.rot, H))
            out[n["dkv_norm"]] = TensorDecl((self.rank,), "norm")
        if self.has_sink:
            out[n["sink"]] = TensorDecl((self.n_heads,), "bias")
        if self.gate:
            out[n["g"]] = TensorDecl((self.n_heads, H))
        return out

    def bind(self, get, precision: Precision, device):
        n = self.names
        mats = [get(n["q"])] + ([] if self.shares_cache else [get(n["dkv"])])
        self._gate_col = sum(m.shape[0] for m in mats)
        if self.gate:
            gate_rows = get(n["g"])
            pad = -(self._gate_col + gate_rows.shape[0]) % 8  # (a row count the products' tiles like)
            mats += [gate_rows] + ([gate_rows.new_zeros((pad, gate_rows.shape[1]))] if pad else [])
        if len({m.dtype for m in mats}) > 1:
            mats = [m.to(torch.float32) for m in mats]
        # one projection for the queries, the latent and the gates: the rows of the matrices, one after the other
        self.w_in = precision.matrix(torch.cat(mats, dim=0), device)
        # U as [heads][rank][dim]: the product that carries a plain query into the latent's space
        uk = get(n["uk"]).reshape(self.n_heads, self.dim, self.rank).transpose(1, 2)
        self.w_uk_t = precision.matrix(uk.contiguous(), device)
        self.w_uv = precision.matrix(get(n["uv"]).reshape(self.n_heads, self.vdim, self.rank), device)
        self.w_o = precision.matrix(get(n["o"]), device)
        if not self.shares_cache:
            self.norm_w = precision.vector(get(n["dkv_norm"]), device)
        if self.has_sink:
            self.sink = precision.vector(get(n["sink"]), device)

    def _matrices(self):
        return tuple(m for m in (self.w_in, self.w_uk_t, self.w_uv, self.w_o, self.w_gate) if m is not None)

    def weight_bytes(self):
        return sum(m.numel() * m.element_size() for m in self._matrices())

    def flops_per_token(self):
        return 2.0 * sum(m.numel() for m in self._matrices())

    def context_flops(self, n_tokens):
        # scores over rank + rot columns, weighted sums over rank; half the pairs are masked
        return 1.0 * n_tokens * n_tokens * self.n_heads * (2 * self.rank + self.rot)

    def state_spec(self):
        return None if self.shares_cache else PagedKV(1, self.row, 0, values=False)

    def prepare(self, max_positions, device):
        self.position.prepare(max_positions, device)

    def plan_stream(self, builder, h, cache, out):
        """The same operations for the native step plan: ``h`` (a buffer in the activation dtype) in,
        the mixer's output into ``out`` (fp32)."""
        from ..engine.plan import NotPlannable
        rotation = self.position.rotation()
        if rotation is None:
            raise NotPlannable(f"position encoding {self.position.kind!r} is no plain rotation")
        if self.gate:
            raise NotPlannable("an output gate on the latent attention has no native plan form")
        table, rot_dims, pairing = rotation
        act = builder.act_dtype
        proj = builder.tokens(self.w_in.shape[0], act)
        builder.linear(h, self.w_in, proj, "queries | latent")
        qa = builder.tokens(self.n_heads * self.row, act)
        builder.latent_prepare(proj, self.q_width, self.norm_w, table, qa, cache, not self.shares_cache,
                               self.n_heads, self.dim, self.rot, rot_dims, pairing, self.rank, self.row, self.eps)
        builder.head_linear(proj, self.dim + self.rot, self.w_uk_t, qa, self.row, "queries into the latent's space")
        builder.free(proj)
        heads_out = builder.tokens(self.n_heads * self.vdim, act)
        builder.latent_attention(qa, cache, self.sink, self.w_uv, heads_out, self.n_heads, self.rank,
                                 self.rank + self.rot, self.row, self.scale)
        builder.free(qa)
        builder.linear(heads_out, self.w_o, out, "latent attention out")
        builder.free(heads_out)

    def forward(self, ctx, h, cache):
        act = ctx.precision.act_dtype
        batch = ctx.batch
        rotation = self.position.rotation()
        if rotation is None:
            raise ValueError(f"latent attention turns its rotated part itself; position encoding "
                             f"{self.position.kind!r} is no plain rotation")
        table, rot_dims, pairing = rotation
        block_table = batch.block_tables[cache.group]
        proj = ops.linear(h, self.w_in, act)                     # [T][queries | latent + key part]
        qa = latent_kernels.latent_prepare(
            proj, self.q_width, self.norm_w, table, batch, block_table,
            None if self.shares_cache else cache.k_pool, self.n_heads, self.dim, self.rot, rot_dims, pairing,
            self.rank, self.row, self.eps)
        qa2 = qa.view(qa.shape[0], self.n_heads * self.row)
        latent_kernels.head_linear(proj, 0, self.dim + self.rot, self.dim, self.w_uk_t, qa2, 0, self.row)
        pool = cache.k_pool
        if (act == torch.bfloat16 and pool.dtype == torch.bfloat16 and latent_kernels.tensor_cores()
                and attention_kernels.tensor_core_shape_ok(self.n_heads, 1, self.row, pool.shape[2])):
            # many query heads over one pool head whose rows are keys and values: the paged attention
            # kernels; the weighted rows come back [T][heads][row], their first `rank` entries count
            mixed = attention_kernels.paged_attention(ctx, qa2, cache, block_table, self.n_heads, 0, self.scale,
                                                      act, sink=self.sink)
            stride = self.row
        else:
            mixed = latent_kernels.latent_attention(qa, pool, self.sink, batch, block_table, self.rank,
                                                    self.rank + self.rot, self.scale)
            stride = self.rank
        heads_out = torch.empty((mixed.shape[0], self.n_heads * self.vdim), dtype=act, device=mixed.device)
        latent_kernels.head_linear(mixed, 0, stride, self.rank, self.w_uv, heads_out, 0, self.vdim)
        if self.gate:
            from ..kernels import mixing
            mixing.sigmoid_gate_cols_mul_(heads_out, proj, self._gate_col, self.n_heads, self.vdim)
        return ops.linear(heads_out, self.w_o, torch.float32)
