"""`dlblas.kernels.fp8` (dlblas/kernels/fp8.py:108-182 of the reference)."""
from typing import Optional, Tuple

import torch

from .. import _C, ops


def per_token_group_quant_fp8(x: torch.Tensor, group_size: int, eps: float = 1e-10,
                              dtype: Optional[torch.dtype] = torch.float8_e4m3fn,
                              column_major_scales: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token-group FP8 quantisation: scale = max(absmax, eps) / 448, q = clamp(x / scale).
    Scales are [..., K/group] row-major, or for 2-D inputs a [M, G] view with strides (1, M)
    when `column_major_scales`."""
    assert x.shape[-1] % group_size == 0, \
        f"the last dimension of 'x' {x.shape[-1]} must be divisible by 'group_size' {group_size}"
    assert x.stride(-1) == 1, f"{x} groups must be contiguous"
    assert dtype == torch.float8_e4m3fn, "only torch.float8_e4m3fn is supported"
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if column_major_scales:
        assert x.dim() == 2, "column-major scales need a 2-D input"
    q, s = ops.quant_fp8(x2, group_size, _C.QUANT_DIV_EPS, eps, column_major_scales)
    q = q.view(shp)
    if not column_major_scales:
        s = s.view(shp[:-1] + (shp[-1] // group_size,))
    return q, s
