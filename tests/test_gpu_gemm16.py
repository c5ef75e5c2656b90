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
    b_kn = b.transpose(1, 2).contiguous()                        # [G, K, N]: read as an MN-major operand, no transposition
    for tile_rows in ("128", "256"):
        os.environ["DLBLAS_GEMM16_TILE_ROWS"] = tile_rows
        try:
            out2 = m_grouped_gemm(a, b_kn, sizes, trans_b=False)
        finally:
            del os.environ["DLBLAS_GEMM16_TILE_ROWS"]
        _C.check_status()
        assert torch.equal(out, out2)
    empty = m_grouped_gemm(a[:0], b, torch.zeros(4, dtype=torch.int64, device=DEV), trans_b=True)
    assert empty.shape == (0, 1024)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tile_rows", [128, 256])
def test_k_grouped_gemm(dtype, tile_rows, monkeypatch):
    monkeypatch.setenv("DLBLAS_GEMM16_TILE_ROWS", str(tile_rows))
    from dlblas_b200 import _C
    from dlblas_b200.kernels.grouped_gemm.BF16 import k_grouped_gemm
    g = torch.Generator().manual_seed(17)
    # ragged K ranges (not multiples of the 64-element K block), empty groups first / in the middle / last,
    # m and n that are not multiples of the tile, a single group
    for (sizes, m, n) in [([5, 0, 130, 64, 257], 264, 200), ([128, 128], 512, 256), ([1], 8, 8), ([0, 300, 211, 0], 136, 1096),
                          ([0], 16, 24)]:
        sz = torch.tensor(sizes, dtype=torch.int64)
        k = int(sz.sum())
        a = (torch.randn(k, m, generator=g) * 0.5).to(dtype)
        b = (torch.randn(k, n, generator=g) * 0.5).to(dtype)
        out = k_grouped_gemm(a.to(DEV), b.to(DEV), sz.to(DEV))
        _C.check_status()
        ref = O.k_grouped_gemm(a, b, sz)
        assert out.shape == (len(sizes), m, n) and out.dtype == dtype
        assert O.rel_frobenius(out.cpu(), ref) < 2e-3
        assert float((out.cpu().float() - ref.float()).abs().max()) <= 2 ** -6 * max(float(ref.float().abs().max()), 1e-6)
        for i, size in enumerate(sizes):
            if size == 0:
                assert not out[i].any()                          # an empty group writes zeros


def test_k_grouped_gemm_like_the_reference_test():
    # tests/kernels/grouped_gemm/BF16/test_k_grouped_gemm.py of the reference at a sixteenth of its K: random group
    # sizes, row-max normalisation, rtol = atol = 0.01
    import random
    from dlblas_b200 import _C
    from dlblas_b200.kernels.grouped_gemm.BF16 import k_grouped_gemm, utils
    random.seed(3)
    groups = 16
    raw = [random.randint(0, 2 * 2560) for _ in range(groups)]
    sizes = torch.tensor(raw, dtype=torch.int64, device=DEV)
    k = int(sizes.sum())
    g = torch.Generator(device=DEV).manual_seed(2)
    for (m, n) in ((1536, 2048), (2048, 768)):
        a = torch.randn(k, m, generator=g, device=DEV, dtype=torch.bfloat16)
        b = torch.randn(k, n, generator=g, device=DEV, dtype=torch.bfloat16)
        out = k_grouped_gemm(a, b, sizes)
        _C.check_status()
        ref = utils.gmm_dw(a, b, sizes.cpu())
        torch.testing.assert_close(utils.row_max_normalization(out.float()), utils.row_max_normalization(ref.float()),
                                   rtol=0.01, atol=0.01)


def test_k_grouped_gemm_sizes_that_do_not_add_up():
    """Group sizes that stop short of the operands' rows leave the rest unused; sizes that run past them are clipped
    (the last groups shrink, down to empty), as the entry point documents."""
    from dlblas_b200 import _C
    from dlblas_b200.kernels.grouped_gemm.BF16 import k_grouped_gemm
    g = torch.Generator().manual_seed(23)
    k, m, n = 300, 256, 136
    a = (torch.randn(k, m, generator=g) * 0.5).to(torch.bfloat16)
    b = (torch.randn(k, n, generator=g) * 0.5).to(torch.bfloat16)
    for sizes, clipped in (([100, 50], [100, 50]), ([200, 150, 70], [200, 100, 0])):
        out = k_grouped_gemm(a.to(DEV), b.to(DEV), torch.tensor(sizes, dtype=torch.int64, device=DEV))
        _C.check_status()
        ref = O.k_grouped_gemm(a, b, torch.tensor(clipped, dtype=torch.int64))
        assert O.rel_frobenius(out.cpu(), ref) < 2e-3
        assert not out[-1].any() or clipped[-1] > 0
