"""`dlblas.kernels.moe` (dlblas/kernels/moe.py of the reference): quant_fp8 (:466-474),
silu_and_mul_masked_post_quant_fwd (:272-319), biased_grouped_topk (:477-521), renormalize (:368-373)."""
from typing import Optional

import torch

from .. import _C, ops


def renormalize(topk_weights: torch.Tensor, renormalize: bool):
    if renormalize:
        topk_weights = topk_weights / topk_weights.sum(dim=-1, keepdim=True)
    if not topk_weights.is_contiguous():
        topk_weights = topk_weights.contiguous()
    return topk_weights


def quant_fp8(A: torch.Tensor, group_size: int, dtype: torch.dtype = torch.float8_e4m3fn):
    """scale = absmax * (1/448) (no epsilon), q = clamp(A / scale); scales [M, K/group] fp32."""
    assert A.dim() == 2
    M, K = A.shape
    assert K % group_size == 0
    return ops.quant_fp8(A, group_size, _C.QUANT_RECIP_MUL, 0.0, out_dtype=dtype)


def silu_and_mul_masked_post_quant_fwd(input: torch.Tensor, output: torch.Tensor, output_scale: torch.Tensor,
                                       quant_group_size: int, masked_m: torch.Tensor):
    """input [E, M, 2N] -> output e4m3 [E, M, N], output_scale [E, M, N/128]; only rows < masked_m[e].
    silu(gate) is rounded to the input dtype before the multiply; scale = max(absmax, 1e-10) / 448."""
    assert input.is_contiguous()
    assert output.is_contiguous()
    assert len(input.shape) == 3
    assert input.shape[0] == masked_m.shape[0]
    assert input.shape[-1] % 2 == 0
    size_n = input.shape[-1] // 2
    assert size_n % quant_group_size == 0
    assert quant_group_size == 128, "the fused kernel quantises 1x128 groups"
    mm = masked_m if masked_m.dtype == torch.int32 else masked_m.to(torch.int32)
    ops.silu_mul_quant(input, _C.QUANT_DIV_EPS, 1e-10, True, mm, output, output_scale)


def biased_grouped_topk(hidden_states: torch.Tensor, gating_output: torch.Tensor, correction_bias: torch.Tensor,
                        topk: int, renormalize: bool, num_expert_group: int = 0, topk_group: int = 0,
                        n_share_experts_fusion: int = 0, routed_scaling_factor: Optional[float] = None):
    """DeepSeek-V3 grouped routing in one kernel.  Returns (weights fp32 [T, k], ids int32 [T, k]); slots
    are ordered by descending biased score with the lowest expert index winning ties (the reference's
    `topk(sorted=False)` leaves the order open).  Shared-expert fusion draws random ids in the reference
    (:506-514) and is not offered here."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    assert n_share_experts_fusion == 0, "n_share_experts_fusion is not supported"
    return ops.route_grouped_topk(gating_output.contiguous(), correction_bias, topk, renormalize, num_expert_group,
                                  topk_group)


def map_logic_to_physical_idx_hash_random(topk_idx: torch.Tensor, log2phy: torch.Tensor, logcnt: torch.Tensor,
                                          seed: int = 12345, block_size: int = 128) -> torch.Tensor:
    """Logical -> physical expert ids for replicated experts (:558-579 of the reference): slot (t, k) goes to
    replica hash32((t << 16) ^ (k << 8) ^ seed) mod logcnt[e]; -1 for negative ids / experts without replicas.
    `block_size` is the reference's launch parameter and has no effect here."""
    return ops.eplb_map_hash(topk_idx, log2phy, logcnt, seed)
