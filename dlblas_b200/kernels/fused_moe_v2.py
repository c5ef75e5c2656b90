"""`dlblas.kernels.fused_moe_v2.fused_moe` of the reference (vLLM-style entry point,
dlblas/kernels/fused_moe_v2.py:323-471) for block-quantised FP8 weights: quantise 1x128
(`max(absmax, 1e-10) / 448` scales, :214-225) -> w1 grouped GEMM -> silu*up -> quantise -> w2 grouped GEMM
with the routing weight -> sum over top-k.  The block-aligned token layout of the reference
(moe_align_block_size) is an implementation detail of its Triton kernel; here the same function runs on
the library's expert path, whose tile list plays that role."""
from typing import List, Optional

import torch

from .. import _C
from ..layers.moe.kernels.blocked_fp8_fused_moe import moe_expert_forward


def fused_moe(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
              topk_ids: torch.Tensor, inplace: bool = False, activation: str = "silu", use_fp8_w8a8: bool = False,
              use_int8_w8a8: bool = False, use_int8_w8a16: bool = False, use_int4_w4a16: bool = False,
              per_channel_quant: bool = False, global_num_experts: int = -1, num_local_experts: int = -1,
              expert_map: Optional[torch.Tensor] = None, w1_scale: Optional[torch.Tensor] = None,
              w2_scale: Optional[torch.Tensor] = None, w1_zp: Optional[torch.Tensor] = None,
              w2_zp: Optional[torch.Tensor] = None, hidden_states_scale: Optional[torch.Tensor] = None,
              block_shape: Optional[List[int]] = None, chunk_size: Optional[int] = 32 * 1024,
              out_dtype: Optional[torch.dtype] = torch.bfloat16):
    assert hidden_states.shape[1] == w1.shape[2], "Hidden size mismatch"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.stride(-1) == 1, "Stride of last dimension must be 1"
    assert w2.stride(-1) == 1, "Stride of last dimension must be 1"
    assert hidden_states.dtype in [torch.float32, torch.float16, torch.bfloat16, torch.float8_e4m3fn]
    if activation != "silu":
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")
    if use_int8_w8a8 or use_int8_w8a16 or use_int4_w4a16 or per_channel_quant:
        raise NotImplementedError("the int8 / int4 and per-channel modes are not built: block-quantised FP8 "
                                  "(use_fp8_w8a8, block_shape [128, 128]) and unquantised bf16 / fp16 are")
    ids = topk_ids
    if expert_map is not None:
        # global -> local ids, -1 for experts of other ranks (:130-133 of moe_align_block_size.py)
        ids = torch.where(topk_ids >= 0, expert_map[topk_ids.clamp(min=0).long()].to(topk_ids.dtype),
                          torch.full_like(topk_ids, -1))
    if not use_fp8_w8a8:
        out = _fused_moe_16bit(hidden_states, w1, w2, topk_weights, ids, out_dtype)
        if inplace:
            hidden_states.copy_(out)
            return hidden_states
        return out
    assert block_shape is not None and list(block_shape) == [128, 128], "block_shape must be [128, 128]"
    assert w1_scale is not None and w2_scale is not None
    x_q, x_s, hidden = None, None, hidden_states
    if hidden_states.dtype == torch.float8_e4m3fn:
        assert hidden_states_scale is not None, "FP8 activations need hidden_states_scale"
        x_q, x_s, hidden = hidden_states, hidden_states_scale, None
    out = moe_expert_forward(hidden, x_q, x_s, w1, w1_scale, w2, w2_scale, topk_weights, ids, topk_ids.shape[1],
                             out_dtype=out_dtype, expert_offset=0, num_experts=w1.shape[0],
                             quant_mode=_C.QUANT_DIV_EPS, weighted_combine=False)
    if inplace:
        hidden_states.copy_(out)
        return hidden_states
    return out


def _fused_moe_16bit(hidden: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                     ids: torch.Tensor, out_dtype: Optional[torch.dtype]) -> torch.Tensor:
    """The unquantised mode (all `use_*` flags off; dlblas/kernels/fused_moe_v2.py:375-466 with compute type = the
    activations' 16-bit type): rows copied into expert order -> w1 grouped GEMM -> silu(gate) * up -> w2 grouped GEMM
    -> sum over top-k of weight * row in fp32, one rounding.  Both GEMMs run on the 16-bit tcgen05 kernel; ids outside
    [0, E) (other ranks' experts under `expert_map`) contribute nothing."""
    import os
    from .. import ops
    assert hidden.dtype in (torch.bfloat16, torch.float16), "the unquantised mode takes bf16 or fp16 activations"
    assert w1.dtype == hidden.dtype and w2.dtype == hidden.dtype, "weights must have the activations' type"
    m, h = hidden.shape
    e, n2, _ = w1.shape
    assert w2.shape == (e, h, n2 // 2), "w2 must be [E, H, I]"
    top_k = ids.shape[1]
    out_dtype = out_dtype or hidden.dtype
    if m == 0:
        return torch.empty(0, h, dtype=out_dtype, device=hidden.device)
    s_rows = m * top_k
    ids = ids.contiguous()
    _, exp_start, exp_end, pos = ops.sort_by_expert(ids, e, want_pos=True)
    tile_rows = int(os.environ.get("DLBLAS_GEMM16_TILE_ROWS", "256" if s_rows >= 512 * e else "128"))
    max_tiles = ops.max_tiles_for(s_rows, e, tile_rows)
    tiles = ops.build_tiles(exp_start, exp_end, 0, e, max_tiles, tile_rows)
    a1, _ = ops.permute_rows(hidden, None, pos, top_k, s_rows)
    c1 = torch.empty(s_rows, n2, dtype=hidden.dtype, device=hidden.device)
    ops.grouped_gemm_16bit(a1, w1.contiguous(), tiles, max_tiles, tile_rows, c1)
    act = ops.silu_and_mul(c1)
    y = torch.empty(s_rows, h, dtype=hidden.dtype, device=hidden.device)
    ops.grouped_gemm_16bit(act, w2.contiguous(), tiles, max_tiles, tile_rows, y)
    out = torch.empty(m, h, dtype=hidden.dtype, device=hidden.device)
    weights = topk_weights.contiguous().float()
    ops.ep_gather(y, ids.to(torch.int32), weights, pos.view(m, top_k), out)
    return out if out_dtype == hidden.dtype else out.to(out_dtype)
