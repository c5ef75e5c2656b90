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
    if not use_fp8_w8a8 or use_int8_w8a8 or use_int8_w8a16 or use_int4_w4a16 or per_channel_quant:
        raise NotImplementedError("only the block-quantised FP8 path (use_fp8_w8a8, block_shape [128, 128]) is built")
    assert block_shape is not None and list(block_shape) == [128, 128], "block_shape must be [128, 128]"
    assert w1_scale is not None and w2_scale is not None
    ids = topk_ids
    if expert_map is not None:
        # global -> local ids, -1 for experts of other ranks (:130-133 of moe_align_block_size.py)
        ids = torch.where(topk_ids >= 0, expert_map[topk_ids.clamp(min=0).long()].to(topk_ids.dtype),
                          torch.full_like(topk_ids, -1))
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
