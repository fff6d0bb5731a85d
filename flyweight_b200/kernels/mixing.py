"""Python faces of ``csrc/layer_mix.cu`` and ``csrc/linear_attention.cu``: the small fp32 kernels of
layers whose sublayers run side by side (norms over column ranges of a projection, values mixed between
layers, sigmoid gates, scaled residual sums, a token-indexed side input, the mean of two normed
outputs) and the decayed linear-attention recurrence with its gated norm."""
from __future__ import annotations

from typing import Optional

import torch

from . import lib
from .lib import KernelError, c_float, c_longlong, check_tensor, is_bf16, ptr, stream
from .ops import _i32

UNARY_ACTIVATIONS = {"relu_squared": 0, "silu": 1, "sigmoid": 2, "gelu_tanh": 3}


def _rows_2d(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be a CUDA matrix with contiguous rows")


def rmsnorm_ranges_(buf: torch.Tensor, ranges) -> torch.Tensor:
    """In place, per row of ``buf`` ([T][width], fp32 or bf16) and per range ``(col0, weight, count,
    eps)`` (one or two of them, one eps): columns ``col0 .. col0 + len(weight)`` become ``weight *
    c / sqrt(sum(c^2) / count + eps)``.  ``count`` is the number of channels the mean goes over: fewer than
    the range is wide when the range holds zero padding."""
    check_tensor("projection rows", buf)
    if buf.dim() != 2 or not 1 <= len(ranges) <= 2:
        raise KernelError("rmsnorm_ranges_ takes a matrix and one or two column ranges")
    args = []
    eps = float(ranges[0][3])
    for col0, weight, count, this_eps in ranges:
        check_tensor("range norm weight", weight, torch.float32)
        if float(this_eps) != eps:
            raise KernelError("the ranges of one launch share their eps")
        args += [int(col0), weight.numel(), int(count), ptr(weight)]
    if len(ranges) == 1:
        args += [0, 0, 0, None]
    lib.call("fwb_rmsnorm_ranges", ptr(buf), is_bf16(buf), c_longlong(buf.stride(0)), buf.shape[0], *args,
             c_float(eps), stream())
    return buf


def causal_conv(rows: torch.Tensor, taps: torch.Tensor, state: Optional[torch.Tensor], batch,
                norm_ranges=None) -> torch.Tensor:
    """A causal convolution over time on the first C channels of ``rows`` ([T][>= C], fp32 or bf16), ``taps`` fp32
    [C][n] with the last tap on the token itself: ``y[t] = sum_j taps[:, j] * rows[t - n + 1 + j]`` along each
    request's tokens.  ``state``: fp32 [slots][n - 1][C], every live request's last n - 1 inputs (zero when it
    starts), read in front of a portion and moved on by this call (None when n == 1).  ``norm_ranges``: one or two
    ``(col0, weight, count, eps)`` as ``rmsnorm_ranges_`` takes them; those column ranges of the result are
    normed by the same launch.  Returns a new buffer [T][C]; ``rows`` (and its columns from C on) stay."""
    check_tensor("convolution input", rows)
    T, ld = rows.shape
    C, n = taps.shape
    check_tensor("convolution taps", taps, torch.float32)
    if C > ld:
        raise KernelError(f"taps for {C} channels, rows of {ld}")
    stride = 0
    if n > 1:
        if state is None or state.dtype != torch.float32 or tuple(state.shape[1:]) != (n - 1, C) \
                or state.stride(2) != 1 or state.stride(1) != C:
            raise KernelError(f"the convolution's state must be fp32 [slots][{n - 1}][{C}] with contiguous slots")
        stride = state.stride(0) if state.shape[0] > 1 else (n - 1) * C
    norm_args = [0, 0, 0, None, 0, 0, 0, None]
    eps = 0.0
    if norm_ranges:
        if not 1 <= len(norm_ranges) <= 2 or C * 4 > 160 * 1024:
            raise KernelError("the convolution norms one or two column ranges of rows of at most 40,960 channels")
        eps = float(norm_ranges[0][3])
        for index, (col0, weight, count, this_eps) in enumerate(norm_ranges):
            check_tensor("range norm weight", weight, torch.float32)
            if float(this_eps) != eps:
                raise KernelError("the ranges of one launch share their eps")
            norm_args[4 * index:4 * index + 4] = [int(col0), weight.numel(), int(count), ptr(weight)]
    out = torch.empty((T, C), dtype=rows.dtype, device=rows.device)
    lib.call("fwb_causal_conv", ptr(rows), ptr(out), is_bf16(rows), c_longlong(ld), c_longlong(C), 0, C, ptr(taps), n,
             ptr(state) if n > 1 else None, c_longlong(stride), ptr(batch.tok_seg), ptr(batch.seg_start),
             ptr(batch.seg_slot), T, batch.n_segments, *norm_args, c_float(eps), stream(),
             launches=2 if n > 1 else 1)
    return out


def value_mix_(rows: torch.Tensor, col0: int, width: int, first: torch.Tensor,
               lam: Optional[torch.Tensor]) -> None:
    """``lam`` None: ``first[t][:] = rows[t][col0 : col0 + width]`` (the values a later layer mixes in).
    Else ``rows[t][col0 + i] <- (1 - lam) rows[t][col0 + i] + lam first[t][i]`` in fp32, in place; ``lam`` is one
    fp32 number on the device."""
    check_tensor("projection rows", rows)
    check_tensor("first values", first, rows.dtype, (rows.shape[0], width))
    if lam is not None:
        check_tensor("mixing weight", lam, torch.float32)
    lib.call("fwb_value_mix", ptr(rows), is_bf16(rows), c_longlong(rows.stride(0)), int(col0), int(width),
             ptr(first), ptr(lam), rows.shape[0], 0 if lam is None else 1, stream())


def sigmoid_gate_mul_(y: torch.Tensor, gate: torch.Tensor, heads: int, head_dim: int) -> torch.Tensor:
    """``y[t][h][c] *= sigmoid(gate[t][h])`` (gate [T][heads]) or ``sigmoid(gate[t][h][c])`` (gate
    [T][heads * head_dim]), in place; both of one dtype."""
    check_tensor("attention output", y)
    check_tensor("gate", gate, y.dtype)
    T = y.shape[0]
    if y.numel() != T * heads * head_dim:
        raise KernelError(f"the gated rows hold {y.numel()} entries, expected {T * heads * head_dim}")
    width = gate.numel() // max(T, 1)
    if width == heads:
        per_head = 1
    elif width == heads * head_dim:
        per_head = head_dim
    else:
        raise KernelError(f"a gate of {width} entries per token fits neither {heads} heads nor their channels")
    lib.call("fwb_sigmoid_gate_mul", ptr(y), ptr(gate), is_bf16(y), T, heads, head_dim, per_head, stream())
    return y


def sigmoid_gate_cols_mul_(y: torch.Tensor, rows: torch.Tensor, col0: int, heads: int, head_dim: int) -> torch.Tensor:
    """``y[t][h][c] *= sigmoid(rows[t][col0 + h])``: a gate per head that lies in columns of another buffer (a
    fused projection's last columns), of its own dtype; in place."""
    check_tensor("attention output", y)
    check_tensor("projection rows", rows)
    T = y.shape[0]
    if y.numel() != T * heads * head_dim or rows.shape[0] != T or col0 + heads > rows.shape[1]:
        raise KernelError("the gated rows and the gate's columns do not fit")
    if rows.dtype == torch.bfloat16 and y.dtype != torch.bfloat16:
        raise KernelError("a 16-bit gate on 32-bit rows has no kernel")
    lib.call("fwb_sigmoid_gate_mul_strided", ptr(y), is_bf16(y), rows.data_ptr() + col0 * rows.element_size(),
             is_bf16(rows), c_longlong(rows.shape[1]), T, heads, head_dim, 1, stream())
    return y


def scaled_add_(x: torch.Tensor, a: torch.Tensor, scale_a: Optional[torch.Tensor],
                b: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None,
                copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """``x += scale_a * a (+ scale_b * b)`` per channel, in place and in fp32 (a scale may be None: 1).
    ``copy_dtype`` bfloat16: also returns the new ``x`` rounded to bfloat16 (what a product that reads the
    stream next takes), written in the same pass; any other value returns None."""
    check_tensor("residual", x, torch.float32)
    H = x.shape[-1]
    check_tensor("sublayer output", a, torch.float32, x.shape)
    for name, t in (("scale", scale_a), ("second scale", scale_b)):
        if t is not None:
            check_tensor(name, t, torch.float32, (H,))
    if b is not None:
        check_tensor("second sublayer output", b, torch.float32, x.shape)
    copy = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if copy_dtype == torch.bfloat16 else None
    lib.call("fwb_scaled_add", ptr(x), ptr(a), ptr(scale_a), ptr(b), ptr(scale_b), ptr(copy), x.numel() // H, H,
             stream())
    return copy


def unary_act(x: torch.Tensor, activation: str, out_dtype: torch.dtype) -> torch.Tensor:
    """``act(x)`` element by element in fp32: "relu_squared", "silu", "sigmoid" or "gelu_tanh"."""
    check_tensor("activation input", x)
    try:
        code = UNARY_ACTIVATIONS[activation]
    except KeyError:
        raise KernelError(f"unknown activation {activation!r}; known: " + ", ".join(UNARY_ACTIVATIONS)) from None
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    lib.call("fwb_unary_act", ptr(x), is_bf16(x), ptr(out), is_bf16(out), c_longlong(x.numel()), code, stream())
    return out


def side_gate(g: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor,
              out_dtype: torch.dtype) -> torch.Tensor:
    """``gelu_tanh(g[t][c]) * table[tokens[t]][col0 + c]``: g [T][dim], table [vocab][width]."""
    check_tensor("side gate", g)
    check_tensor("side table", table)
    _i32("token ids", tokens, g.shape[0])
    T, dim = g.shape
    out = torch.empty((T, dim), dtype=out_dtype, device=g.device)
    lib.call("fwb_side_gate", ptr(g), is_bf16(g), ptr(table), is_bf16(table), table.shape[1], int(col0),
             ptr(tokens), table.shape[0], ptr(out), is_bf16(out), T, dim, stream())
    return out


def pair_norm_mean(a: torch.Tensor, weight_a: torch.Tensor, b: torch.Tensor, weight_b: torch.Tensor,
                   eps: float) -> torch.Tensor:
    """``0.5 (weight_a * unit(a) + weight_b * unit(b))`` per row, fp32."""
    check_tensor("left output", a, torch.float32)
    check_tensor("right output", b, torch.float32, a.shape)
    H = a.shape[-1]
    check_tensor("left weight", weight_a, torch.float32, (H,))
    check_tensor("right weight", weight_b, torch.float32, (H,))
    y = torch.empty_like(a)
    lib.call("fwb_pair_norm_mean", ptr(a), ptr(weight_a), ptr(b), ptr(weight_b), c_float(eps), ptr(y),
             a.numel() // H, H, stream())
    return y


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """``weight * o / sqrt(mean(o^2) + eps) * sigmoid(gate)`` per row.  o: fp32 [T][H]; ``gate``: [T][H],
    possibly a view of columns of a wider row-major tensor."""
    check_tensor("recurrence output", o, torch.float32)
    T, H = o.shape
    _rows_2d("gate", gate)
    if tuple(gate.shape) != (T, H):
        raise KernelError(f"the gate must be [{T}][{H}], got {tuple(gate.shape)}")
    check_tensor("norm weight", weight, torch.float32, (H,))
    out = torch.empty((T, H), dtype=out_dtype, device=o.device)
    lib.call("fwb_gated_rmsnorm", ptr(o), ptr(gate), is_bf16(gate), c_longlong(gate.stride(0)), ptr(weight),
             c_float(eps), ptr(out), is_bf16(out), T, H, stream())
    return out


def decay_scan(p: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, state: torch.Tensor,
               batch, heads: int, dim: int, vdim: int, act_silu: bool = True) -> torch.Tensor:
    """``S <- decay_h S + k v^T; o = S^T q`` over the step's ragged segments.  ``p``: fp32 [T][...] whose
    columns from ``q_col``, ``k_col`` (heads x dim each) and ``v_col`` (heads x vdim) are the projections
    (``act_silu``: silu on the way in); ``state``: fp32 [slots][>= heads dim vdim], read at the head of
    every segment and advanced.  Returns o, fp32 [T][heads vdim]."""
    check_tensor("projection", p, torch.float32)
    T, width = p.shape
    if max(q_col, k_col) + heads * dim > width or v_col + heads * vdim > width:
        raise KernelError("the projection's rows are shorter than the columns asked for")
    check_tensor("decay", decay, torch.float32, (heads,))
    size = heads * dim * vdim
    if (not state.is_cuda or state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < size
            or state.stride(1) != 1):
        raise KernelError(f"the recurrent state must be CUDA fp32 [slots][>= {size}], got {tuple(state.shape)}")
    stride = state.stride(0) if state.shape[0] > 1 else state.shape[1]
    S = batch.n_segments
    _i32("seg_start", batch.seg_start, S + 1)
    _i32("seg_slot", batch.seg_slot, S)
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=p.device)
    lib.call("fwb_decay_scan", ptr(p), c_longlong(width), int(q_col), int(k_col), int(v_col), 1 if act_silu else 0,
             ptr(decay), ptr(state), c_longlong(stride), ptr(batch.seg_start), ptr(batch.seg_slot), ptr(o), T, S,
             heads, dim, vdim, stream())
    return o


PIECE_TOKENS = 256      # tokens of a segment that one block of the tensor-core recurrence walks


def decay_runs(p: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, state: torch.Tensor,
               batch, heads: int, dim: int, vdim: int, act_silu: bool = True) -> torch.Tensor:
    """``decay_scan`` for steps that bring portions of prompts, on tensor cores: q, k and v enter the
    products as bfloat16, the state and every sum stay fp32.  Segments longer than ``PIECE_TOKENS`` are cut
    into pieces that run side by side (their contributions to the state are chained first)."""
    check_tensor("projection", p, torch.float32)
    T, width = p.shape
    if max(q_col, k_col) + heads * dim > width or v_col + heads * vdim > width:
        raise KernelError("the projection's rows are shorter than the columns asked for")
    check_tensor("decay", decay, torch.float32, (heads,))
    size = heads * dim * vdim
    if (not state.is_cuda or state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < size
            or state.stride(1) != 1):
        raise KernelError(f"the recurrent state must be CUDA fp32 [slots][>= {size}], got {tuple(state.shape)}")
    stride = state.stride(0) if state.shape[0] > 1 else state.shape[1]
    S = batch.n_segments
    _i32("seg_start", batch.seg_start, S + 1)
    _i32("seg_slot", batch.seg_slot, S)
    piece_seg, piece_tok0, pieces = batch.attention_tiles(PIECE_TOKENS, 0)
    chained = batch.max_segment > PIECE_TOKENS
    scratch = torch.empty((pieces, size), dtype=torch.float32, device=p.device) if chained else None
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=p.device)
    lib.call("fwb_decay_runs", ptr(p), c_longlong(width), int(q_col), int(k_col), int(v_col), 1 if act_silu else 0,
             ptr(decay), ptr(state), c_longlong(stride), ptr(batch.seg_start), ptr(batch.seg_slot),
             ptr(piece_seg), ptr(piece_tok0), PIECE_TOKENS, 1 if chained else 0,
             ptr(scratch) if chained else None, ptr(o), T, S, pieces, heads, dim, vdim, stream())
    if chained:
        lib.add_launches(2)
    return o
