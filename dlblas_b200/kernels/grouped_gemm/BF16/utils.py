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
