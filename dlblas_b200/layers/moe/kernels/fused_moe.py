"""`dlblas.layers.moe.kernels.fused_moe._dlblas_get_sorted_idx`
(dlblas/layers/moe/kernels/fused_moe.py:83-88 of the reference)."""
import torch

from .... import ops


def _dlblas_get_sorted_idx(topk_ids: torch.Tensor, num_experts: int):
    """sorted_idx = stable argsort of the flattened ids (-1 first); exp_start/exp_end per expert
    (two rows of one [2, E] tensor), both 0 for an expert without tokens."""
    return ops.sort_by_expert(topk_ids, num_experts)
