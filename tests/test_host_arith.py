"""Host-side arithmetic that has to match the reference exactly, and properties of the oracle that the GPU
tests lean on.  No GPU needed."""
import torch

from oracle import moe_oracle as O


def test_capacity_uses_the_reference_single_precision_product():
    """dlblas/kernels/topk_gating.py:15-24: ceil((T / E) * float32(capacity_factor * k)) in float32.  The expected
    values were produced by that expression; a double-precision product gives one less / one more for each."""
    from dlblas_b200.kernels.topk_gating import _capacity
    pins = [(50290, 8, 1.2, 2, 2, 15088), (48400, 8, 0.9, 6, 2, 32670), (47660, 8, 1.2, 2, 4, 14299),
            (51055, 8, 1.2, 4, 2, 30634), (11780, 16, 1.2, 2, 2, 1768), (11300, 8, 1.2, 8, 2, 13561),
            (4096, 64, 1.0, 8, 2, 512), (3, 64, 1.0, 1, 2, 2), (100, 64, 1.0, 2, 4, 4)]
    for t, e, cf, k, mc, want in pins:
        ref = torch.ceil((t / e) * torch.tensor(cf * k)).to(torch.int64)
        ref = max(int(ref), mc)
        assert ref == want
        assert _capacity(t, e, cf * k, mc) == want, (t, e, cf, k)
        if t <= 12000 and want <= t:                              # the oracle sizes its outputs by the same capacity
            assert O.topk_gating(torch.zeros(t, e), k, cf, mc)[3].numel() == e * want


def test_zero_groups_quantise_to_finite_payloads():
    """scale = absmax * (1/448) is 0 for an all-zero group; the clamp of the compiled reference kernel turns the
    0 / 0 quotients into -448, and the group then contributes payload * 0 = 0."""
    x = torch.randn(6, 256).to(torch.bfloat16)
    x[2] = 0
    x[4, 128:] = 0
    q, s = O.quant_fp8(x)
    assert bool(torch.isfinite(q.float()).all())
    assert float(s[2].abs().max()) == 0.0 and bool((q[2].view(torch.uint8) == 0xFE).all())
    assert float(s[4, 1]) == 0.0 and float(s[4, 0]) > 0.0
    q2, s2 = O.per_token_group_quant_fp8(x, 128)                 # eps keeps this formula's scale positive
    assert bool((q2[2].float() == 0).all()) and float(s2[2, 0]) > 0.0
    _, _, w13, w13s, w2, w2s = O.make_layer_inputs(1, 256, 256, 4, seed=1)
    ow, oids = O.softmax_topk(torch.randn(6, 4), 2, True)
    out = O.moe_layer(x, ow, oids, w13, w13s, w2, w2s, top_k=2)
    assert bool(torch.isfinite(out.float()).all()) and float(out[2].float().abs().max()) == 0.0


def test_canonical_sigmoid_is_the_correctly_rounded_one():
    x = torch.cat([torch.randn(200000) * 4, torch.tensor([0.0, -0.0, 88.0, -88.0, 104.0, -104.0, 1e30, -1e30,
                                                           float("inf"), -float("inf")])])
    s = O.sigmoid_exact(x)
    assert s.dtype == torch.float32 and torch.equal(s, torch.sigmoid(x.double()).float())
    # torch's own fp32 sigmoid is a library function good to an ulp or two: that is all the slack there is
    d = (s.view(torch.int32).long() - torch.sigmoid(x).view(torch.int32).long()).abs()
    assert int(d[:200000].max()) <= 2
    assert torch.equal(O.sigmoid_exact(x.to(torch.bfloat16)), O.sigmoid_exact(x.to(torch.bfloat16).float()))


def test_tma_aligned_scale_layout():
    """dlblas/kernels/quant_dequant.py:65-83: same values, column-major storage, rows padded to 16 bytes."""
    for m, g in [(7, 4), (128, 56), (1, 1), (130, 16)]:
        s = torch.rand(m, g)
        a = O.tma_align_input_scale(s)
        assert a.shape == (m, g) and torch.equal(a, s)
        assert a.stride() == (1, (m + 3) // 4 * 4)
