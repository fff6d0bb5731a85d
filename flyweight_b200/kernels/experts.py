"""Python faces of the mixture-of-experts kernels (``csrc/moe.cu``): router, sorting of the
(token, expert) pairs, the experts' products over the sorted rows, the weighted sum."""
from __future__ import annotations

import torch

from . import lib
from .lib import KernelError, c_float, check_tensor, is_bf16, ptr, stream
from .ops import GATE_ACTIVATIONS


SIMT_TILE_ROWS = 64          # rows of a tile of fwb_moe_gemm
_use_tensor_cores = True


def set_tensor_cores(flag: bool) -> None:
    """Tests switch the grouped tcgen05 product off to compare it with the fp32-FMA kernel."""
    global _use_tensor_cores
    _use_tensor_cores = bool(flag)


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, n_groups: int, keep: int, top: int):
    """ids int32 [T][top] and weights fp32 [T][top]: softmax scores over all router outputs; the choice
    on score + correction inside the ``keep`` best of ``n_groups`` runs of neighbours; the weights are
    the chosen outputs' plain scores."""
    check_tensor("router input", h)
    T, W = h.shape
    N = router.shape[0]
    check_tensor("router", router, torch.float32, (N, W))
    check_tensor("router correction", correction, torch.float32, (N,))
    ids = torch.empty((T, top), dtype=torch.int32, device=h.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=h.device)
    lib.call("fwb_moe_route", ptr(h), is_bf16(h), ptr(router), ptr(correction), ptr(ids), ptr(weights), T, W, N,
             int(n_groups), int(keep), int(top), stream())
    return ids, weights


def route_table(token_ids: torch.Tensor, table: torch.Tensor, top: int):
    """ids int32 [T][top] and weights fp32 [T][top] of a router that is a table: row ``token_ids[t]`` of
    ``table`` (int32 [vocab][top]) names the token's experts, each with weight 1 / top."""
    check_tensor("token ids", token_ids, torch.int32)
    check_tensor("expert table", table, torch.int32)
    if table.dim() != 2 or table.shape[1] != top:
        raise KernelError(f"the expert table must be [vocab][{top}], got {tuple(table.shape)}")
    T = token_ids.numel()
    ids = torch.empty((T, top), dtype=torch.int32, device=table.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=table.device)
    lib.call("fwb_moe_route_table", ptr(token_ids), ptr(table), table.shape[0], int(top), T, ptr(ids), ptr(weights),
             stream())
    return ids, weights


def experts_forward(h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                    w_down: torch.Tensor, activation: str = "silu", add_normed_into=None, limit: float = 0.0):
    """``sum_slot weights * expert(h)`` as fp32 [T][W].  ``w_gate_up``: [E][2F][W] (gate rows, then up
    rows), ``w_down``: [E][W][F], both in the dtype of ``h``.  Router outputs from E on are identity
    experts: they pass ``h`` itself on.  ``add_normed_into`` = (x, norm weight, eps): the sum is not
    returned but normed and added, ``x += weight * sum / sqrt(mean(sum^2) + eps)`` in fp32, by the kernel
    that makes it (returns None); a fourth entry, fp32 [T][W], is added to every token's sum first (the output of an
    expert that every token shares)."""
    check_tensor("expert input", h)
    T, W = h.shape
    top = ids.shape[1]
    E, F2, _ = w_gate_up.shape
    F = F2 // 2
    check_tensor("expert gate|up", w_gate_up, h.dtype, (E, 2 * F, W))
    check_tensor("expert down", w_down, h.dtype, (E, W, F))
    check_tensor("expert ids", ids, torch.int32, (T, top))
    check_tensor("expert weights", weights, torch.float32, (T, top))
    act = GATE_ACTIVATIONS[activation]
    A = T * top
    bf16 = is_bf16(h)
    # bfloat16 rows whose lengths the tensor maps take run the grouped tcgen05 product, on token tiles
    # as wide as an expert's share of the step's rows; everything else the fp32-FMA kernel (tiles of 64)
    tensor_cores = bool(bf16 and _use_tensor_cores and E > 0 and W % 8 == 0 and F % 8 == 0)
    tile_rows = SIMT_TILE_ROWS
    if tensor_cores:
        share = -(-A // E)
        tile_rows = 16 if share <= 16 else (32 if share <= 32 else (64 if share <= 64 else 128))
    max_tiles = A // tile_rows + E + 1
    dev = h.device
    meta = torch.empty(E + 1 + 2 * A + 1 + 2 * max_tiles, dtype=torch.int32, device=dev)
    offsets, row_token = meta[:E + 1], meta[E + 1:E + 1 + A]
    pair_row, tiles = meta[E + 1 + A:E + 1 + 2 * A], meta[E + 1 + 2 * A:]
    lib.call("fwb_moe_sort", ptr(ids), A, top, E, tile_rows, ptr(offsets), ptr(row_token), ptr(pair_row), ptr(tiles),
             stream())
    a = torch.empty((A, F), dtype=h.dtype, device=dev)
    y = torch.empty((A, W), dtype=torch.float32, device=dev)
    if tensor_cores:
        from .tensorcore import EPI_F32, _gated_epilogue
        rows = torch.empty((A, W), dtype=h.dtype, device=dev)
        lib.call("fwb_moe_gather_rows", ptr(h), ptr(row_token), ptr(offsets), E, ptr(rows), A, W, stream())
        lib.call("fwb_gemm_tcgen05_grouped", ptr(rows), ptr(w_gate_up), ptr(a), ptr(offsets), ptr(tiles), max_tiles,
                 tile_rows, A, F, W, E, 2 * F, F, _gated_epilogue(activation), F, c_float(limit), stream(),
                 tag=f"experts gate|up {F}x{W}")
        lib.call("fwb_gemm_tcgen05_grouped", ptr(a), ptr(w_down), ptr(y), ptr(offsets), ptr(tiles), max_tiles,
                 tile_rows, A, W, F, E, W, W, EPI_F32, 0, c_float(0.0), stream(), tag=f"experts down {W}x{F}")
    elif E > 0:                                 # (a router may have identity experts only)
        lib.call("fwb_moe_gemm", ptr(h), ptr(w_gate_up), bf16, ptr(a), ptr(offsets), ptr(row_token), ptr(tiles),
                 max_tiles, F, W, 1, act, c_float(limit), stream())
        lib.call("fwb_moe_gemm", ptr(a), ptr(w_down), bf16, ptr(y), ptr(offsets), ptr(row_token), ptr(tiles),
                 max_tiles, W, F, 0, 0, c_float(0.0), stream())
    if add_normed_into is not None:
        x, norm_weight, eps = add_normed_into[:3]
        extra = add_normed_into[3] if len(add_normed_into) > 3 else None
        check_tensor("residual", x, torch.float32, (T, W))
        check_tensor("norm weight", norm_weight, torch.float32, (W,))
        if extra is not None:
            check_tensor("shared output", extra, torch.float32, (T, W))
        lib.call("fwb_moe_combine_norm_add", ptr(y), ptr(h), bf16, ptr(pair_row), ptr(ids), ptr(weights), ptr(x),
                 ptr(norm_weight), c_float(eps), T, W, top, E, ptr(extra), stream())
        return None
    out = torch.empty((T, W), dtype=torch.float32, device=dev)
    lib.call("fwb_moe_combine", ptr(y), ptr(h), bf16, ptr(pair_row), ptr(ids), ptr(weights), ptr(out), T, W, top,
             E, stream())
    return out
