"""m_grouped_gemm (dlblas/kernels/grouped_gemm/BF16/m_grouped_gemm.py:235-352 of the reference):
C[rows of group g] = A[rows of g] @ B[g] for contiguous row groups of sizes `size_per_group`.

B is read where it lies in both layouts: [G, N, K] (`trans_b=True`) as a K-major operand, [G, K, N] (`trans_b=False`,
the reference's default) as an MN-major operand of the tensor cores; only a K that is not a multiple of 64 makes the
second layout fall back to one transposition of B per call.  Tile list and group offsets are built on the device;
nothing synchronises with the host."""
import os

import torch
from torch import Tensor

from .... import ops
from ...._C import check, check_status, dtype_code, lib, ptr, require_cuda, status_word, stream  # noqa: F401


def m_grouped_gemm(A: Tensor, B: Tensor, size_per_group: torch.Tensor, trans_b: bool = False, numSM: int = -1) -> Tensor:
    assert A.dim() == 2
    assert B.dim() == 3
    require_cuda(A, B, size_per_group)
    M, K = A.shape
    assert A.stride(-1) == 1, "Please make sure A is K-major"
    assert A.dtype == B.dtype and A.dtype in (torch.bfloat16, torch.float16)
    b_kn = False
    if trans_b:
        num_groups, N, BK = B.shape
        Bt = B.contiguous()
    else:
        num_groups, BK, N = B.shape
        b_kn = BK % 64 == 0
        Bt = B.contiguous() if b_kn else B.transpose(1, 2).contiguous()
    assert BK == K, "K of A should be equal to K of B"
    assert size_per_group.numel() == num_groups
    A = A.contiguous()
    C = A.new_empty(M, N)
    if M == 0:
        return C
    ends = torch.cumsum(size_per_group.to(torch.int64), 0)
    starts = ends - size_per_group.to(torch.int64)
    # pairs of CTAs on 256-row tiles when the groups are large enough to fill them (decided from the shapes,
    # no look at the group sizes on the host); DLBLAS_GEMM16_TILE_ROWS = 128 / 256 overrides
    tile_rows = int(os.environ.get("DLBLAS_GEMM16_TILE_ROWS", "256" if M >= 512 * num_groups else "128"))
    max_tiles = M // tile_rows + num_groups
    tiles = torch.empty((max_tiles + 1) * 4, dtype=torch.int32, device=A.device)
    check(lib().dlb_moe_build_tiles_rows(ptr(starts), ptr(ends), 0, num_groups, tile_rows, ptr(tiles), max_tiles,
                                         stream(A.device)))
    fn = lib().dlb_grouped_gemm_16bit_b_kn if b_kn else lib().dlb_grouped_gemm_16bit
    check(fn(ptr(A), ptr(Bt), dtype_code(A.dtype), M, num_groups, N, K, ptr(tiles), max_tiles,
             tile_rows, ptr(C), N, ptr(status_word(A.device)), stream(A.device)))
    return C
