"""`dlblas.kernels.quant_dequant.tma_align_input_scale`
(dlblas/kernels/quant_dequant.py:22-83 of the reference).

The grouped GEMM of this package reads row-major scales, and the quantiser can write the
column-major layout directly (`per_token_group_quant_fp8(..., column_major_scales=True)`), so
nothing on the hot path calls this; it is kept for callers that hold row-major scales and
want the padded column-major view."""
import torch


def get_tma_aligned_size(x: int, element_size: int) -> int:
    alignment = 16 // element_size
    return (x + alignment - 1) // alignment * alignment


def tma_align_input_scale(input_scale: torch.Tensor) -> torch.Tensor:
    assert input_scale.dim() == 2
    m, g = input_scale.shape
    pad_m = get_tma_aligned_size(m, input_scale.element_size())
    out = torch.empty((g, pad_m), dtype=input_scale.dtype, device=input_scale.device)
    out[:, :m].copy_(input_scale.t())
    return out.t()[:m]
