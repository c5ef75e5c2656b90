"""Test helpers of the reference's BF16 grouped GEMM package (dlblas/kernels/grouped_gemm/BF16/utils.py:77-95)."""
import torch


def gmm(a, b, batch_sizes, trans_b=False):
    """Group-by-group torch matmul: the ground truth the reference's tests compare with."""
    out, start = [], 0
    for i, size in enumerate(batch_sizes.tolist()):
        rhs = b[i].t() if trans_b else b[i]
        out.append(a[start:start + size] @ rhs)
        start += size
    return torch.cat(out)


def allclose(x, y, pct=2.0):
    mask = torch.isclose(x, y, rtol=1e-5)
    return float((mask.numel() - mask.sum()) / mask.numel() * 100) <= pct


def gmm_dw(a, b, batch_sizes):
    """Group-by-group `a_g.T @ b_g` over row groups of the shared leading dimension: the ground truth of the
    reference's k_grouped_gemm test (tests/kernels/grouped_gemm/BF16/test_k_grouped_gemm.py:10-28)."""
    out = a.new_empty(batch_sizes.numel(), a.shape[1], b.shape[1])
    start = 0
    for g, size in enumerate(batch_sizes.tolist()):
        out[g] = a[start:start + size].t() @ b[start:start + size]
        start += size
    return out


def row_max_normalization(tensor):
    """Each row divided by its largest magnitude (dlblas/kernels/grouped_gemm/BF16/utils.py:113-116)."""
    return tensor / (tensor.abs().max(dim=-1).values + 1e-9).unsqueeze(-1)
