"""k_grouped_gemm (dlblas/kernels/grouped_gemm/BF16/k_grouped_gemm.py:126-176 and :254-330 of the reference):
C[g] = A[rows of g]^T @ B[rows of g] for contiguous row groups of sizes `size_per_group` along the shared leading
(reduction) dimension; A [K, M], B [K, N], C [G, M, N] in the operands' 16-bit type, fp32 accumulation.  This is the
weight-gradient GEMM of a grouped linear layer.

The tcgen05 kernel reads A and B where they lie, as MN-major operands (a row of memory holds one k): nothing is
transposed or copied.  Group offsets, the tile list and the order in which the CTAs take the tiles are built on the
device in a small workspace; nothing synchronises with the host.  An empty group yields a zero C[g]."""
import os

import torch
from torch import Tensor

from ...._C import check, dtype_code, lib, ptr, require_cuda, status_word, stream


def k_grouped_gemm(A: Tensor, B: Tensor, size_per_group: torch.Tensor) -> Tensor:
    assert A.dim() == 2
    assert B.dim() == 2
    require_cuda(A, B, size_per_group)
    K, M = A.shape
    K_, N = B.shape
    assert A.stride(-1) == 1, "Please make sure A is K-major"
    assert B.stride(-1) == 1, "Please make sure B is K-major"
    assert K == K_, "Please make sure that A and B have the same seqlen"
    assert A.dtype == B.dtype and A.dtype in (torch.bfloat16, torch.float16), f"data type {A.dtype} not supported"
    num_groups = size_per_group.shape[0]
    A, B = A.contiguous(), B.contiguous()
    C = A.new_empty(num_groups, M, N)
    if num_groups == 0 or M == 0 or N == 0:
        return C
    sizes = size_per_group.to(torch.int64).contiguous()
    # pairs of CTAs on 256-row tiles of C unless M is smaller than one; DLBLAS_GEMM16_TILE_ROWS = 128 / 256 overrides
    tile_rows = int(os.environ.get("DLBLAS_GEMM16_TILE_ROWS", "256" if M >= 256 else "128"))
    need = lib().dlb_k_grouped_gemm_workspace_bytes(K, M, N, num_groups, tile_rows)
    assert need > 0, "k_grouped_gemm: bad sizes"
    work = torch.empty(need, dtype=torch.uint8, device=A.device)
    check(lib().dlb_k_grouped_gemm_16bit(ptr(A), ptr(B), dtype_code(A.dtype), K, M, N, ptr(sizes), num_groups, tile_rows,
                                         ptr(work), need, ptr(C), ptr(status_word(A.device)), stream(A.device)))
    return C
