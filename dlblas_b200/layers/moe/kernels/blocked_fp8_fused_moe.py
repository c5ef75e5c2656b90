"""`dlblas.layers.moe.kernels.blocked_fp8_fused_moe` (dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py of
the reference): the block-scaled FP8 fused MoE function (:261-338) and the grouped-GEMM launcher (:159-242).

Pipeline of `moe_expert_forward` (all kernels from the CUDA extension, one launch each):
  sort_by_expert -> build_tiles -> quantise+permute (or permute) the tokens into expert-contiguous order ->
  grouped GEMM w13 with the silu*up + FP8 re-quantisation epilogue -> grouped GEMM w2 with the routed-weight
  epilogue scattered back to (token, slot) order -> sum over the top-k slots.
"""
import os
from typing import Optional

import torch

from .... import _C, ops


def _renormalize(topk_weights: torch.Tensor, renormalize: bool):
    if renormalize:
        topk_weights = topk_weights / topk_weights.sum(dim=-1, keepdim=True)
    if not topk_weights.is_contiguous():
        topk_weights = topk_weights.contiguous()
    return topk_weights


def moe_expert_forward(hidden: Optional[torch.Tensor], x_q: Optional[torch.Tensor], x_s: Optional[torch.Tensor],
                       w1: torch.Tensor, w1_scale: torch.Tensor, w2: torch.Tensor, w2_scale: torch.Tensor,
                       topk_weights: torch.Tensor, topk_ids: torch.Tensor, topk: int, out_dtype: torch.dtype,
                       expert_offset: int = 0, num_experts: Optional[int] = None,
                       quant_mode: int = _C.QUANT_RECIP_MUL, weighted_combine: bool = False,
                       fuse_swiglu: bool = True, group_size: int = 128,
                       skip_unrouted_rows: bool = False, return_slot_rows: bool = False,
                       w2_column_parts: int = 1, on_columns_done=None, sm_margin: int = 0) -> torch.Tensor:
    """Expert computation for tokens that are either unquantised (`hidden` [M, H]) or already
    quantised (`x_q` e4m3 [M, H], `x_s` fp32 [M, H/128]).  topk_ids are global ids in
    [expert_offset, expert_offset + E_local) for the experts held in w1/w2; any other id (e.g. -1)
    contributes zero.  Returns [M, H] of out_dtype.

    With `return_slot_rows` and `w2_column_parts` > 1 the second GEMM runs in that many launches over windows of the
    hidden dimension; `on_columns_done(y, col_begin, col_count)` is called after each launch has been queued (the
    expert-parallel combine pushes those columns back from another stream), and every launch but the first leaves
    `sm_margin` SMs to that stream."""
    assert group_size == 128, "block size 128 is the only supported quantisation group"
    e_local, n, h = w1.shape
    inter = n // 2
    m = hidden.shape[0] if hidden is not None else x_q.shape[0]
    dev = w1.device
    if num_experts is None:
        num_experts = e_local
    if m == 0:
        return torch.empty(0, h, dtype=out_dtype, device=dev)
    s_rows = m * topk
    ids = topk_ids.contiguous()
    weights = topk_weights.contiguous()
    if weights.dtype != torch.float32:
        weights = weights.float()
    sorted_idx, exp_start, exp_end, pos = ops.sort_by_expert(ids, num_experts, want_pos=True)
    # DLBLAS_FP8_TILE_ROWS=256 runs the GEMMs on pairs of CTAs with 256-row tiles (tcgen05 cta_group::2).  Off by
    # default: the per-K-block hand-shake across the two CTAs costs more than the cheaper MMAs win (0.94 against
    # 1.85 PFLOP/s on 32 experts of 2048 rows); the variant is kept, bit-identical, for kernels with fewer hand-shakes.
    tile_rows = int(os.environ.get("DLBLAS_FP8_TILE_ROWS", "0")) or 128
    if out_dtype == torch.float32:
        tile_rows = 128
    max_tiles = ops.max_tiles_for(s_rows, e_local, tile_rows)
    tiles = ops.build_tiles(exp_start, exp_end, expert_offset, e_local, max_tiles, tile_rows)
    if hidden is not None:
        a1, a1_s = ops.quant_fp8(hidden, group_size, quant_mode, 1e-10, False, pos, topk, s_rows)
    else:
        a1, a1_s = ops.permute_rows(x_q, x_s.contiguous(), pos, topk, s_rows)
    h_q = torch.empty(s_rows, inter, dtype=ops.FP8, device=dev)
    h_s = torch.empty(s_rows, inter // 128, dtype=torch.float32, device=dev)
    if fuse_swiglu and n % 256 == 0:
        ops.grouped_gemm(a1, a1_s, w1, w1_scale, tiles, max_tiles, _C.EPI_SWIGLU_QUANT, h_q, q_scale=h_s,
                         round_dtype=out_dtype, quant_mode=quant_mode, quant_eps=1e-10, tile_rows=tile_rows)
    else:
        c1 = torch.empty(s_rows, n, dtype=out_dtype, device=dev)
        ops.grouped_gemm(a1, a1_s, w1, w1_scale, tiles, max_tiles, _C.EPI_STORE, c1, tile_rows=tile_rows)
        ops.silu_mul_quant(c1, quant_mode, 1e-10, False, None, h_q, h_s)
    y = torch.empty(s_rows, h, dtype=out_dtype, device=dev)
    parts = w2_column_parts if (return_slot_rows and h % (256 * max(w2_column_parts, 1)) == 0) else 1
    if parts > 1:
        step = h // parts
        for p in range(parts):
            ops.grouped_gemm(h_q, h_s, w2, w2_scale, tiles, max_tiles, _C.EPI_SCATTER_WEIGHT, y, sorted_idx=sorted_idx,
                             weights=weights, tile_rows=tile_rows, n_begin=p * step, n_count=step,
                             sm_margin=sm_margin if p > 0 else 0)
            if on_columns_done is not None:
                on_columns_done(y, p * step, step)
        return y
    ops.grouped_gemm(h_q, h_s, w2, w2_scale, tiles, max_tiles, _C.EPI_SCATTER_WEIGHT, y, sorted_idx=sorted_idx,
                     weights=weights, tile_rows=tile_rows)
    if return_slot_rows:
        # [M * topk, H] rows of the individual (token, slot) results, already weighted; the caller sums them
        # (the expert-parallel combine does it while pushing the rows to their source rank)
        return y
    return ops.sum_topk(y, m, topk, ids, expert_offset, expert_offset + e_local, skip_unrouted_rows)


def fused_moe_blocked_fp8_kernel_launcher(A: torch.Tensor, A_scale: torch.Tensor, B: torch.Tensor,
                                          B_scale: torch.Tensor, C: torch.Tensor, sorted_idx: torch.Tensor,
                                          exp_start: torch.Tensor, exp_end: torch.Tensor, weights: torch.Tensor,
                                          enable_weights: bool = False, top_k: int = 1, num_tokens: int = None,
                                          expert_offset: int = 0, reindex_a: bool = True, reindex_c: bool = True):
    """Grouped block-scaled GEMM over the expert segments [exp_start, exp_end) of the sorted order:
    A row = sorted_idx[p] // top_k if reindex_a else p; C row = sorted_idx[p] if reindex_c else p;
    optional multiply by weights.flatten()[sorted_idx[p]].  C is written in place."""
    assert A.dim() == 2 and A_scale.dim() == 2 and B.dim() == 3 and B_scale.dim() == 3
    e_local, n, k = B.shape
    assert k % A_scale.size(1) == 0 and k % B_scale.size(2) == 0 and n % B_scale.size(1) == 0
    assert k // A_scale.size(1) == 128 and k // B_scale.size(2) == 128 and n // B_scale.size(1) == 128, \
        "only 1x128 activation scales and 128x128 weight scales are supported"
    s_rows = sorted_idx.numel()
    c2 = C.flatten(0, -2)
    max_tiles = ops.max_tiles_for(s_rows, e_local)
    tiles = ops.build_tiles(exp_start, exp_end, expert_offset, e_local, max_tiles)
    if reindex_a:
        # host-side glue for this compatibility entry point: inverse permutation of sorted_idx
        pos = torch.empty(s_rows, dtype=torch.int32, device=A.device)
        pos[sorted_idx] = torch.arange(s_rows, dtype=torch.int32, device=A.device)
        a_sorted, as_sorted = ops.permute_rows(A.contiguous(), A_scale.contiguous(), pos, top_k, s_rows)
    else:
        a_sorted, as_sorted = A.contiguous(), A_scale.contiguous()
    if reindex_c:
        w = weights.contiguous().float() if enable_weights else torch.ones(s_rows, dtype=torch.float32, device=A.device)
        ops.grouped_gemm(a_sorted, as_sorted, B, B_scale, tiles, max_tiles, _C.EPI_SCATTER_WEIGHT, c2,
                         sorted_idx=sorted_idx, weights=w)
    else:
        assert not enable_weights, "routed weights need reindex_c=True"
        ops.grouped_gemm(a_sorted, as_sorted, B, B_scale, tiles, max_tiles, _C.EPI_STORE, c2)


def dlblas_fused_moe_blocked_fp8(input: torch.Tensor, input_scale: torch.Tensor, w1: torch.Tensor,
                                 w1_scale: torch.Tensor, w2: torch.Tensor, w2_scale: torch.Tensor,
                                 topk_weights: torch.Tensor, topk_ids: torch.Tensor, topk: int,
                                 out_dtype: torch.dtype = torch.float16, expert_offset: int = 0,
                                 num_experts: int = None, renormalize: bool = False, ep_size: int = 1) -> torch.Tensor:
    """Fused MoE on quantised activations.  As in the reference, `topk_ids` holds ids local to this rank
    (-1 = another rank's expert) and is shifted by `expert_offset` IN PLACE (:288)."""
    e_local = w1.shape[0]
    if num_experts is None:
        num_experts = e_local
        if ep_size > 1:
            num_experts = num_experts * ep_size
    topk_weights = _renormalize(topk_weights, renormalize)
    if expert_offset != 0:
        topk_ids[topk_ids != -1] += expert_offset
    return moe_expert_forward(None, input, input_scale, w1, w1_scale, w2, w2_scale, topk_weights, topk_ids, topk,
                              out_dtype, expert_offset, num_experts)
