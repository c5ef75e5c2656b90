"""16-bit grouped GEMM (tcgen05 kind::f16) against the oracle."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("tile_rows", [128, 256])      # one CTA per tile / pairs of CTAs (cta_group::2)
def test_m_grouped_gemm(dtype, trans_b, tile_rows, monkeypatch):
    monkeypatch.setenv("DLBLAS_GEMM16_TILE_ROWS", str(tile_rows))
    from dlblas_b200 import _C
    from dlblas_b200.kernels.grouped_gemm.BF16 import m_grouped_gemm
    g = torch.Generator().manual_seed(13)
    for (sizes, n, k) in [([5, 0, 130, 64, 257], 264, 200), ([128, 128], 512, 256), ([1], 8, 8), ([300, 211], 1000, 1096)]:
        sz = torch.tensor(sizes, dtype=torch.int64)
        m = int(sz.sum())
        a = (torch.randn(m, k, generator=g) * 0.5).to(dtype)
        b = (torch.randn(len(sizes), n, k, generator=g) * 0.5).to(dtype)
        b_in = b if trans_b else b.transpose(1, 2).contiguous()
        out = m_grouped_gemm(a.to(DEV), b_in.to(DEV), sz.to(DEV), trans_b=trans_b)
        _C.check_status()
        ref = O.m_grouped_gemm(a, b, sz, trans_b=True)
        assert out.shape == (m, n) and out.dtype == dtype
        assert O.rel_frobenius(out.cpu(), ref) < 2e-3
        assert float((out.cpu().float() - ref.float()).abs().max()) <= 2 ** -6 * float(ref.float().abs().max())


def test_m_grouped_gemm_large_and_empty():
    from dlblas_b200 import _C
    from dlblas_b200.kernels.grouped_gemm.BF16 import m_grouped_gemm, utils
    g = torch.Generator(device=DEV).manual_seed(1)
    sizes = torch.tensor([1000, 3000, 17, 4175], device=DEV)
    a = torch.randn(8192, 2048, generator=g, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(4, 1024, 2048, generator=g, device=DEV, dtype=torch.bfloat16) * 0.05
    ref = utils.gmm(a.float(), b.float(), sizes.cpu(), trans_b=True)
    out = m_grouped_gemm(a, b, sizes, trans_b=True)              # 2048 rows per group on average: the pair kernel
    _C.check_status()
    assert float((out.float() - ref).norm() / ref.norm()) < 3e-3
    import os
    os.environ["DLBLAS_GEMM16_TILE_ROWS"] = "128"
    try:
        out1 = m_grouped_gemm(a, b, sizes, trans_b=True)
    finally:
        del os.environ["DLBLAS_GEMM16_TILE_ROWS"]
    _C.check_status()
    assert torch.equal(out, out1)                                # same sums in the same order
    empty = m_grouped_gemm(a[:0], b, torch.zeros(4, dtype=torch.int64, device=DEV), trans_b=True)
    assert empty.shape == (0, 1024)
