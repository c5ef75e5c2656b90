"""Tensor-level wrappers over the C ABI: torch allocates every buffer (outputs and
workspaces) and passes raw pointers and the current stream; all arithmetic happens in
the CUDA extension.  The modules that mirror the reference's layout
(`dlblas_b200.kernels.*`, `dlblas_b200.layers.moe.*`) are built on these."""
from typing import Optional, Tuple

import os

import torch

from . import _C
from ._C import check, dtype_code, lib, ptr, require_cuda, stream

FP8 = torch.float8_e4m3fn


# --------------------------------------------------------------------------- sort
def sort_by_expert(topk_ids: torch.Tensor, num_experts: int, want_pos=False, want_rank=False, want_counts=False):
    """Stable token-by-expert sort.  Returns (sorted_idx int64 [S], exp_start, exp_end) with
    exp_start/exp_end two rows of one [2, E] int64 tensor, followed by the requested extras:
    slot_pos int32 [S], rank_in_expert int32 [S], counts int32 [E]."""
    require_cuda(topk_ids)
    assert topk_ids.dtype in (torch.int32, torch.int64), "topk_ids must be int32 or int64"
    flat = topk_ids.contiguous().view(-1)
    n = flat.numel()
    dev = flat.device
    sorted_idx = torch.empty(n, dtype=torch.int64, device=dev)
    start_end = torch.empty(2, num_experts, dtype=torch.int64, device=dev)
    pos = torch.empty(n, dtype=torch.int32, device=dev) if want_pos else None
    rank = torch.empty(n, dtype=torch.int32, device=dev) if want_rank else None
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev) if want_counts else None
    ws_bytes = lib().dlb_sort_by_expert_workspace_size(n, num_experts)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    check(lib().dlb_sort_by_expert(ptr(flat), dtype_code(flat.dtype), n, num_experts, ptr(sorted_idx),
                                   ptr(start_end[0]), ptr(start_end[1]), ptr(pos), ptr(rank), ptr(counts), ptr(ws),
                                   ws_bytes, stream(dev)))
    out = [sorted_idx, start_end[0], start_end[1]]
    for flag, t in ((want_pos, pos), (want_rank, rank), (want_counts, counts)):
        if flag:
            out.append(t)
    return tuple(out)


def max_tiles_for(num_rows: int, num_local_experts: int, tile_rows: int = 128) -> int:
    return num_rows // tile_rows + num_local_experts


def build_tiles(exp_start: torch.Tensor, exp_end: torch.Tensor, expert_offset: int, num_local_experts: int,
                max_tiles: int, tile_rows: int = 128) -> torch.Tensor:
    tiles = torch.empty((max_tiles + 1) * 4, dtype=torch.int32, device=exp_start.device)
    check(lib().dlb_moe_build_tiles_rows(ptr(exp_start), ptr(exp_end), expert_offset, num_local_experts, int(tile_rows),
                                         ptr(tiles), max_tiles, stream(exp_start.device)))
    return tiles


def build_tiles_masked(masked_m: torch.Tensor, rows_per_expert: int) -> Tuple[torch.Tensor, int]:
    assert masked_m.dtype == torch.int32
    e = masked_m.numel()
    max_tiles = e * ((rows_per_expert + 127) // 128)
    tiles = torch.empty((max_tiles + 1) * 4, dtype=torch.int32, device=masked_m.device)
    check(lib().dlb_moe_build_tiles_masked(ptr(masked_m), e, rows_per_expert, ptr(tiles), max_tiles,
                                           stream(masked_m.device)))
    return tiles, max_tiles


# --------------------------------------------------------------------------- quant
def quant_fp8(x: torch.Tensor, group_size: int = 128, mode: int = _C.QUANT_RECIP_MUL, eps: float = 1e-10,
              column_major_scales: bool = False, dst_pos: Optional[torch.Tensor] = None, fanout: int = 1,
              rows_out: Optional[int] = None, out_dtype: torch.dtype = FP8):
    """1xG quantisation of a 2-D tensor; with dst_pos, row t is written to rows dst_pos[t*fanout + j]."""
    require_cuda(x)
    assert x.dim() == 2 and x.stride(-1) == 1, "x must be 2-D with contiguous rows"
    assert out_dtype == FP8, "only torch.float8_e4m3fn is supported"
    m, k = x.shape
    assert k % group_size == 0, f"the last dimension of 'x' {k} must be divisible by 'group_size' {group_size}"
    rows = m if rows_out is None else rows_out
    g = k // group_size
    q = torch.empty(rows, k, dtype=FP8, device=x.device)
    if column_major_scales:
        s = torch.empty(g, rows, dtype=torch.float32, device=x.device).t()
    else:
        s = torch.empty(rows, g, dtype=torch.float32, device=x.device)
    check(lib().dlb_quant_fp8(ptr(x), dtype_code(x.dtype), m, k, x.stride(0), group_size, mode, eps, ptr(q), ptr(s),
                              s.stride(0), s.stride(1), ptr(dst_pos), fanout, stream(x.device)))
    return q, s


def permute_rows(q: torch.Tensor, scales: Optional[torch.Tensor], dst_pos: torch.Tensor, fanout: int, rows_out: int):
    require_cuda(q)
    assert q.dim() == 2 and q.is_contiguous()
    m = q.shape[0]
    row_bytes = q.shape[1] * q.element_size()
    out_q = torch.empty(rows_out, q.shape[1], dtype=q.dtype, device=q.device)
    out_s = None
    groups = 0
    if scales is not None:
        assert scales.is_contiguous() and scales.dtype == torch.float32
        groups = scales.shape[1]
        out_s = torch.empty(rows_out, groups, dtype=torch.float32, device=q.device)
    check(lib().dlb_permute_rows(ptr(q), row_bytes, ptr(scales), groups, m, ptr(dst_pos), fanout, ptr(out_q),
                                 ptr(out_s), stream(q.device)))
    return out_q, out_s


# --------------------------------------------------------------------------- activation
def silu_and_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    require_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.stride(-1) == 1
    rows, n2 = gate_up.shape
    n = n2 // 2
    if out is None:
        out = gate_up.new_empty((rows, n))
    assert out.stride(-1) == 1 and out.dtype == gate_up.dtype
    check(lib().dlb_silu_and_mul(ptr(gate_up), dtype_code(gate_up.dtype), rows, n, gate_up.stride(0), ptr(out),
                                 out.stride(0), stream(gate_up.device)))
    return out


def silu_mul_quant(gate_up: torch.Tensor, mode: int = _C.QUANT_RECIP_MUL, eps: float = 1e-10, round_silu: bool = False,
                   masked_m: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                   out_scale: Optional[torch.Tensor] = None):
    """[rows, 2n] (or [E, M, 2n] with masked_m) -> e4m3 [.., n] and fp32 scales [.., n/128]."""
    require_cuda(gate_up)
    assert gate_up.is_contiguous()
    n = gate_up.shape[-1] // 2
    lead = gate_up.shape[:-1]
    rows = gate_up.numel() // (2 * n)
    rpe = gate_up.shape[1] if masked_m is not None else 0
    if out is None:
        out = torch.empty(*lead, n, dtype=FP8, device=gate_up.device)
    if out_scale is None:
        out_scale = torch.empty(*lead, n // 128, dtype=torch.float32, device=gate_up.device)
    assert out.is_contiguous() and out_scale.is_contiguous()
    check(lib().dlb_silu_mul_quant(ptr(gate_up), dtype_code(gate_up.dtype), rows, n, mode, eps, int(round_silu),
                                   ptr(masked_m), rpe, ptr(out), ptr(out_scale), stream(gate_up.device)))
    return out, out_scale


# --------------------------------------------------------------------------- GEMMs
def fp8_gemm(a: torch.Tensor, b: torch.Tensor, a_s: torch.Tensor, b_s: torch.Tensor,
             out_dtype: torch.dtype = torch.bfloat16, tile_rows: Optional[int] = None) -> torch.Tensor:
    """tile_rows: 128 / 256 (pairs of CTAs) / None = DLBLAS_FP8_TILE_ROWS or the library's choice."""
    require_cuda(a, b, a_s, b_s)
    if tile_rows is None:
        tile_rows = int(os.environ.get("DLBLAS_FP8_TILE_ROWS", "0"))
    if out_dtype == torch.float32:
        tile_rows = 128
    assert a.is_contiguous() and b.is_contiguous(), "Input tensors must be contiguous"
    assert a_s.is_contiguous() and b_s.is_contiguous(), "Scaling factor tensors must be contiguous"
    k = a.size(-1)
    m = a.numel() // k
    n = b.size(0)
    c = torch.empty(*a.size()[:-1], n, dtype=out_dtype, device=a.device)
    kb = k // 128
    a_s2 = a_s.view(m, -1) if m > 0 else a_s
    assert a_s.numel() == m * kb and b_s.numel() == ((n + 127) // 128) * kb, "scale shapes do not match a / b"
    check(lib().dlb_fp8_gemm(ptr(a), ptr(b), ptr(a_s2), kb, 1, ptr(b_s), ptr(c), dtype_code(out_dtype), m, n, k,
                             int(tile_rows), ptr(_C.status_word(a.device)), stream(a.device)))
    return c


def grouped_gemm(a: torch.Tensor, a_s: torch.Tensor, b: torch.Tensor, b_s: torch.Tensor, tiles: torch.Tensor,
                 max_tiles: int, epilogue: int, c: torch.Tensor, q_scale: Optional[torch.Tensor] = None,
                 sorted_idx: Optional[torch.Tensor] = None, weights: Optional[torch.Tensor] = None,
                 round_dtype: Optional[torch.dtype] = None, quant_mode: int = _C.QUANT_RECIP_MUL,
                 quant_eps: float = 1e-10, tile_rows: int = 128, n_begin: int = 0, n_count: Optional[int] = None,
                 sm_margin: int = 0):
    """a [rows, k] e4m3 in expert-contiguous order, b [E, n, k]; `tiles` built with the same `tile_rows`;
    see dlb_moe_grouped_gemm.  n_begin / n_count: compute only that window of c's columns; sm_margin: SMs to leave to
    kernels of other streams."""
    require_cuda(a, b)
    assert a.is_contiguous() and a_s.is_contiguous() and b.is_contiguous() and b_s.is_contiguous()
    assert c.stride(-1) == 1
    rows, k = a.shape
    e, n, _ = b.shape
    if epilogue == _C.EPI_SWIGLU_QUANT:
        cdt = dtype_code(round_dtype or torch.bfloat16)
    else:
        cdt = dtype_code(c.dtype)
    if n_begin == 0 and n_count in (None, n) and sm_margin == 0:
        check(lib().dlb_moe_grouped_gemm(ptr(a), ptr(a_s), rows, ptr(b), ptr(b_s), e, n, k, ptr(tiles), max_tiles,
                                         int(tile_rows), epilogue,
                                         ptr(c), cdt, c.stride(0), ptr(q_scale), quant_mode, quant_eps, ptr(sorted_idx),
                                         ptr(weights),
                                         ptr(_C.status_word(a.device)), stream(a.device)))
        return c
    check(lib().dlb_moe_grouped_gemm_window(ptr(a), ptr(a_s), rows, ptr(b), ptr(b_s), e, n, k, ptr(tiles), max_tiles,
                                            int(tile_rows), epilogue, ptr(c), cdt, c.stride(0), ptr(q_scale), quant_mode,
                                            quant_eps, ptr(sorted_idx), ptr(weights), ptr(_C.status_word(a.device)),
                                            stream(a.device), int(n_begin), int(n if n_count is None else n_count),
                                            int(sm_margin)))
    return c


# --------------------------------------------------------------------------- combine
def grouped_gemm_16bit(a: torch.Tensor, b: torch.Tensor, tiles: torch.Tensor, max_tiles: int, tile_rows: int,
                       out: torch.Tensor) -> torch.Tensor:
    """out[rows of group g] = a[rows of g] @ b[g]^T on bf16 / fp16 operands, a [rows, k], b [groups, n, k]; `tiles` from
    build_tiles with the same tile_rows."""
    require_cuda(a, b, tiles, out)
    assert a.dtype == b.dtype == out.dtype and a.dtype in (torch.bfloat16, torch.float16)
    assert a.is_contiguous() and b.is_contiguous() and out.stride(-1) == 1
    rows, k = a.shape
    groups, n, bk = b.shape
    assert bk == k and out.shape == (rows, n)
    check(lib().dlb_grouped_gemm_16bit(ptr(a), ptr(b), dtype_code(a.dtype), rows, groups, n, k, ptr(tiles), max_tiles,
                                       tile_rows, ptr(out), out.stride(0), ptr(_C.status_word(a.device)), stream(a.device)))
    return out


def sum_topk(y: torch.Tensor, tokens: int, top_k: int, ids: Optional[torch.Tensor] = None, id_lo: int = 0,
             id_hi: int = 0, skip_unrouted_rows: bool = False) -> torch.Tensor:
    """out[t] = sum_j y[t*top_k + j]; with ids, slots whose id is outside [id_lo, id_hi) are skipped."""
    require_cuda(y)
    assert y.is_contiguous()
    h = y.shape[-1]
    out = torch.empty(tokens, h, dtype=y.dtype, device=y.device)
    idt = 0
    if ids is not None:
        assert ids.is_contiguous()
        idt = dtype_code(ids.dtype)
    check(lib().dlb_moe_sum_topk(ptr(y), dtype_code(y.dtype), tokens, top_k, h, ptr(ids), idt, id_lo, id_hi,
                                 int(skip_unrouted_rows), ptr(out), stream(y.device)))
    return out


def ep_gather(inp: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, index: torch.Tensor, out: torch.Tensor):
    require_cuda(inp, ids, weights, index, out)
    assert inp.is_contiguous() and out.is_contiguous() and ids.is_contiguous() and index.is_contiguous()
    assert ids.dtype == index.dtype and weights.dtype == torch.float32 and weights.is_contiguous()
    assert out.dtype == inp.dtype
    tokens, top_k = ids.shape
    check(lib().dlb_ep_gather(ptr(inp), dtype_code(inp.dtype), inp.shape[1], ptr(ids), ptr(index), dtype_code(ids.dtype),
                              ptr(weights), tokens, top_k, ptr(out), stream(inp.device)))
    return out


def ep_scatter(x, x_scale, ids, counts, expert_start_loc, out_x, out_scale, m_indices, output_index):
    require_cuda(x, ids, counts)
    assert x.is_contiguous() and ids.is_contiguous() and out_x.is_contiguous() and output_index.is_contiguous()
    assert counts.dtype == torch.int32 and expert_start_loc.dtype == torch.int32 and m_indices.dtype == torch.int32
    assert output_index.dtype == ids.dtype
    tokens, top_k = ids.shape
    e = counts.numel()
    groups = 0
    if x_scale is not None:
        assert x_scale.is_contiguous() and out_scale.is_contiguous()
        groups = x_scale.shape[1]
    ws_bytes = lib().dlb_ep_scatter_workspace_size(tokens, top_k, e)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
    check(lib().dlb_ep_scatter(ptr(x), x.shape[1] * x.element_size(), ptr(x_scale), groups, ptr(ids),
                               dtype_code(ids.dtype), tokens, top_k, ptr(counts), e, ptr(expert_start_loc), ptr(out_x),
                               ptr(out_scale), ptr(m_indices), m_indices.numel(), ptr(output_index), ptr(ws), ws_bytes,
                               stream(x.device)))


# --------------------------------------------------------------------------- routing
def eplb_map_hash(topk_idx: torch.Tensor, log2phy: torch.Tensor, logcnt: torch.Tensor, seed: int = 12345):
    """Hash choice of a physical replica per (token, slot); int32 [tokens, top_k]."""
    require_cuda(topk_idx, log2phy, logcnt)
    assert topk_idx.dim() == 2 and log2phy.dim() == 2 and logcnt.numel() == log2phy.shape[0]
    assert topk_idx.dtype in (torch.int32, torch.int64)
    topk_idx = topk_idx.contiguous()
    log2phy = log2phy.to(torch.int32).contiguous()
    logcnt = logcnt.to(torch.int32).contiguous()
    t, k = topk_idx.shape
    out = torch.empty(t, k, dtype=torch.int32, device=topk_idx.device)
    check(lib().dlb_eplb_map_hash(ptr(topk_idx), dtype_code(topk_idx.dtype), ptr(log2phy), ptr(logcnt), t, k,
                                  log2phy.shape[0], log2phy.shape[1], int(seed) & 0xFFFFFFFF, ptr(out),
                                  stream(topk_idx.device)))
    return out


def route_softmax_topk(logits: torch.Tensor, top_k: int, renormalize: bool = False, ids_dtype=torch.int64):
    require_cuda(logits)
    assert logits.dim() == 2 and logits.is_contiguous()
    t, e = logits.shape
    w = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    ids = torch.empty(t, top_k, dtype=ids_dtype, device=logits.device)
    check(lib().dlb_route_softmax_topk(ptr(logits), dtype_code(logits.dtype), t, e, top_k, int(renormalize), ptr(w),
                                       ptr(ids), dtype_code(ids_dtype), stream(logits.device)))
    return w, ids


def route_grouped_topk(logits: torch.Tensor, bias: torch.Tensor, top_k: int, renormalize: bool, num_expert_group: int,
                       topk_group: int):
    require_cuda(logits, bias)
    assert logits.dim() == 2 and logits.is_contiguous()
    t, e = logits.shape
    bias = bias.to(torch.float32).contiguous()
    assert bias.numel() == e
    w = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    ids = torch.empty(t, top_k, dtype=torch.int32, device=logits.device)
    check(lib().dlb_route_grouped_topk(ptr(logits), dtype_code(logits.dtype), ptr(bias), t, e, num_expert_group,
                                       topk_group, top_k, int(renormalize), ptr(w), ptr(ids), stream(logits.device)))
    return w, ids


def topk_gating_bwd(ws: torch.Tensor, dtype, tokens: int, experts: int, k: int, capacity: int, grad_l_aux: torch.Tensor,
                    grad_weights):
    """grad of (l_aux, token_exp_weights) w.r.t. the logits from the forward's workspace `ws`."""
    require_cuda(ws, grad_l_aux)
    dev = ws.device
    grad_l_aux = grad_l_aux.to(dtype).contiguous()
    gw = None if grad_weights is None else grad_weights.to(dtype).contiguous()
    out = torch.empty(tokens, experts, dtype=dtype, device=dev)
    check(lib().dlb_topk_gating_bwd(ptr(ws), ws.numel(), dtype_code(dtype), tokens, experts, k, capacity,
                                    ptr(grad_l_aux), 0 if gw is None else ptr(gw), ptr(out), stream(dev)))
    return out


def topk_gating(logits: torch.Tensor, k: int, capacity: int, return_workspace: bool = False):
    require_cuda(logits)
    assert logits.dim() == 2 and logits.is_contiguous()
    t, e = logits.shape
    dev = logits.device
    l_aux = torch.empty((), dtype=logits.dtype, device=dev)
    ec_idx = torch.empty(k * t, dtype=torch.int32, device=dev)
    w = torch.empty(k * t, dtype=logits.dtype, device=dev)
    sel = torch.empty(e * capacity, dtype=torch.int64, device=dev)
    ws_bytes = lib().dlb_topk_gating_workspace_size(t, e, k)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    check(lib().dlb_topk_gating(ptr(logits), dtype_code(logits.dtype), t, e, k, capacity, ptr(l_aux), ptr(ec_idx), ptr(w),
                                ptr(sel), ptr(ws), ws_bytes, stream(dev)))
    if return_workspace:
        return l_aux, ec_idx, w, sel, ws
    return l_aux, ec_idx, w, sel


def ep_dest_ranks(topk_ids: torch.Tensor, num_local_experts: int, world_size: int) -> torch.Tensor:
    """int32 [T * W]: entry t*W + r is r if token t routes to an expert of rank r, else W."""
    require_cuda(topk_ids)
    assert topk_ids.is_contiguous() and topk_ids.dtype in (torch.int32, torch.int64)
    t, k = topk_ids.shape
    out = torch.empty(t * world_size, dtype=torch.int32, device=topk_ids.device)
    check(lib().dlb_ep_dest_ranks(ptr(topk_ids), dtype_code(topk_ids.dtype), t, k, num_local_experts, world_size, ptr(out),
                                  stream(topk_ids.device)))
    return out
