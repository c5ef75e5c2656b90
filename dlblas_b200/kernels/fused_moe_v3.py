"""`dlblas.kernels.fused_moe_v3` (dlblas/kernels/fused_moe_v3.py of the reference): ep_scatter (:98-155),
ep_gather (:199-233) and the contiguous-layout expert computation fused_moe_v3 (:247-343)."""
from typing import List, Optional, Tuple

import torch

from .. import _C, ops


@torch.no_grad()
def ep_scatter(recv_x, recv_x_scale, recv_topk, num_recv_tokens_per_expert, expert_start_loc, output_tensor,
               output_tensor_scale, m_indices, output_index):
    """Permutes received rows (+ scales) into the expert-contiguous layout.  Destinations inside an
    expert are handed out in token-major, slot-minor order (the reference uses atomics, so its order
    varies from run to run).  expert_start_loc receives the exclusive cumsum of the counts."""
    assert m_indices.shape[0] % 128 == 0
    ops.ep_scatter(recv_x, recv_x_scale, recv_topk, num_recv_tokens_per_expert, expert_start_loc, output_tensor,
                   output_tensor_scale, m_indices, output_index)


@torch.no_grad()
def ep_gather(input_tensor, recv_topk_ids, recv_topk_weight, input_index, output_tensor):
    """output[t] = sum_k weight[t, k] * input[index[t, k]] over slots with id >= 0 (fp32 accumulate)."""
    ops.ep_gather(input_tensor, recv_topk_ids, recv_topk_weight, input_index, output_tensor)


def fused_moe_v3(hidden_states_fp8: Tuple[torch.Tensor, torch.Tensor], topk_idx, topk_weights,
                 w13_weight_fp8: Tuple[torch.Tensor, torch.Tensor], w2_weight_fp8: Tuple[torch.Tensor, torch.Tensor],
                 num_recv_tokens_per_expert: Optional[List[int]]):
    """Expert computation on received, already quantised tokens: topk_idx holds local expert ids (-1 =
    not on this rank).  Returns bf16 [R, H] = sum_k w[t,k] * expert_k(x[t]).  The per-expert counts are
    only used for the empty-input fast paths (:256-260); the layout is derived on the device."""
    x_q, x_s = hidden_states_fp8
    if num_recv_tokens_per_expert is None:
        return x_q.to(torch.bfloat16)
    if sum(num_recv_tokens_per_expert) <= 0:
        return x_q.to(torch.bfloat16)
    from ..layers.moe.kernels.blocked_fp8_fused_moe import moe_expert_forward
    w13, w13_s = w13_weight_fp8
    w2, w2_s = w2_weight_fp8
    return moe_expert_forward(None, x_q, x_s, w13, w13_s, w2, w2_s, topk_weights, topk_idx, topk_idx.shape[1],
                              out_dtype=torch.bfloat16, expert_offset=0, num_experts=w13.shape[0],
                              quant_mode=_C.QUANT_DIV_EPS, weighted_combine=True)
