"""`dlblas.kernels.fp8_gemm` (dlblas/kernels/fp8_gemm.py:68-89 of the reference)."""
import torch

from .. import ops


def fp8_gemm(a: torch.Tensor, b: torch.Tensor, a_s: torch.Tensor, b_s: torch.Tensor) -> torch.Tensor:
    """C = A @ B^T with 1x128 scales on A and 128x128 scales on B.

    a: [..., K] e4m3 contiguous, b: [N, K] e4m3 contiguous, a_s: [..., K/128] fp32,
    b_s: [N/128, K/128] fp32.  As in the reference the output dtype is
    `torch.get_default_dtype()` (callers set bf16).  Runs the tcgen05 kernel of the CUDA extension.
    """
    assert a.is_contiguous() and b.is_contiguous(), "Input tensors must be contiguous"
    assert a_s.is_contiguous() and b_s.is_contiguous(), "Scaling factor tensors must be contiguous"
    return ops.fp8_gemm(a, b, a_s, b_s, out_dtype=torch.get_default_dtype())
