"""Full-size configurations of the benchmark set on the GPU, checked through properties that do
not need the oracle on every row: a sample of tokens against the CPU oracle, permutation
invariance over tokens, and bit-exact routing / sort at full size."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP8 = torch.float8_e4m3fn


def _weights_on_device(e, inter, h, seed):
    """N(0, 0.02^2) weights quantised per 128x128 block, generated on the device in chunks."""
    g = torch.Generator(device=DEV).manual_seed(seed)

    def quant(w):
        n, k = w.shape[1:]
        blk = w.view(w.shape[0], n // 128, 128, k // 128, 128)
        s = blk.abs().amax(dim=(2, 4), keepdim=True) / 448.0
        return (blk / s).clamp_(-448, 448).view(w.shape).to(FP8), s.view(w.shape[0], n // 128, k // 128).float()

    w13 = torch.empty(e, 2 * inter, h, dtype=FP8, device=DEV)
    w13s = torch.empty(e, 2 * inter // 128, h // 128, device=DEV)
    w2 = torch.empty(e, h, inter, dtype=FP8, device=DEV)
    w2s = torch.empty(e, h // 128, inter // 128, device=DEV)
    for i in range(e):
        w13[i:i + 1], w13s[i:i + 1] = quant(torch.randn(1, 2 * inter, h, generator=g, device=DEV) * 0.02)
        w2[i:i + 1], w2s[i:i + 1] = quant(torch.randn(1, h, inter, generator=g, device=DEV) * 0.02)
    return w13, w13s, w2, w2s


def test_mixtral_shaped_layer_sample_against_oracle():
    """Config 3: 4096 tokens, hidden 4096, intermediate 14336, 8 experts top-2 softmax."""
    from dlblas_b200 import _C, ops
    from dlblas_b200.layers.moe.ep_moe import DlblasTritonFusedMoEBlockedF8Impl
    t, h, inter, e, k = 4096, 4096, 14336, 8, 2
    g = torch.Generator().manual_seed(0)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g)
    w13, w13s, w2, w2s = _weights_on_device(e, inter, h, 1)
    w, ids = ops.route_softmax_topk(logits.to(DEV), k, True)
    ow, oids = O.softmax_topk(logits, k, True)
    assert torch.equal(ids.cpu(), oids)                                   # routing bit-exact at full size
    sidx, st, en = ops.sort_by_expert(ids, e)
    o_sidx, o_st, o_en = O.stable_sort_by_expert(oids, e)
    assert torch.equal(sidx.cpu(), o_sidx) and torch.equal(st.cpu(), o_st) and torch.equal(en.cpu(), o_en)
    layer = DlblasTritonFusedMoEBlockedF8Impl(top_k=k, num_experts=e, out_dtype=torch.bfloat16)
    out = layer.forward(x.to(DEV), w, ids, w13, w13s, w2, w2s)
    _C.check_status()
    # the layer acts on every token independently: a permuted batch gives the permuted result, bit for bit
    perm = torch.randperm(t, generator=g)
    out_p = layer.forward(x[perm].to(DEV), w[perm.to(DEV)], ids[perm.to(DEV)], w13, w13s, w2, w2s)
    assert torch.equal(out_p.cpu(), out.cpu()[perm])
    # 48 sampled tokens against the oracle (only the experts they hit are dequantised on the host)
    rows = torch.arange(0, t, t // 48)[:48]
    ref = O.moe_layer(x[rows], ow[rows], oids[rows], w13.cpu(), w13s.cpu(), w2.cpu(), w2s.cpu(), top_k=k)
    err = O.rel_frobenius(out.cpu()[rows], ref)
    assert err < 2e-2, err


def test_deepseek_shaped_layer_sample_against_oracle():
    """Config 4 at batch size on one GPU, as the benchmark runs it: 8192 tokens, hidden 7168, intermediate 2048,
    256 routed experts top-8 with grouped routing (8 groups, 4 kept, sigmoid + bias) and the shared expert as a
    ninth slot of weight 1.  48 rows OF THE FULL-BATCH OUTPUT against the oracle (routed experts + dense shared
    expert); the ragged ~256-row expert segments, two or three row tiles per expert and 257 groups are the ones
    of the timed run."""
    from dlblas_b200 import _C, ops
    from dlblas_b200.layers.moe.kernels.blocked_fp8_fused_moe import moe_expert_forward
    t, h, inter, e, k = 8192, 7168, 2048, 256, 8
    g = torch.Generator().manual_seed(11)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g)
    bias = torch.randn(e, generator=g) * 0.01
    w13, w13s, w2, w2s = _weights_on_device(e + 1, inter, h, 5)          # expert number e = the shared expert
    w, ids = ops.route_grouped_topk(logits.to(DEV), bias.to(DEV), k, True, 8, 4)
    ow, oids = O.biased_grouped_topk(logits, bias, k, True, 8, 4)
    assert torch.equal(ids.cpu(), oids)
    ids9 = torch.cat([ids.long(), torch.full((t, 1), e, dtype=torch.int64, device=DEV)], dim=1)
    w9 = torch.cat([w, torch.ones(t, 1, device=DEV)], dim=1)
    out = moe_expert_forward(x.to(DEV), None, None, w13, w13s, w2, w2s, w9, ids9, k + 1, torch.bfloat16, 0, e + 1)
    _C.check_status()
    assert out.shape == (t, h) and bool(torch.isfinite(out.float()).all())
    rows = torch.cat([torch.arange(0, t, t // 46)[:46], torch.tensor([t - 2, t - 1])])
    assert rows.numel() == 48
    hit = torch.unique(oids[rows].long())
    remap = torch.full((e,), -1, dtype=torch.int64)
    remap[hit] = torch.arange(hit.numel())
    hd = hit.to(DEV)
    ref = O.moe_layer(x[rows], ow[rows], remap[oids[rows].long()], w13[hd].cpu(), w13s[hd].cpu(), w2[hd].cpu(),
                      w2s[hd].cpu(), top_k=k)
    ref = ref + O.dense_swiglu_mlp(x[rows], w13[e].cpu(), w13s[e].cpu(), w2[e].cpu(), w2s[e].cpu())
    err = O.rel_frobenius(out.cpu()[rows], ref)
    assert err < 2e-2, err
    # every sampled row on its own, so that one bad row cannot hide in the norm of the other 47
    per_row = (out.cpu()[rows].float() - ref.float()).norm(dim=1) / ref.float().norm(dim=1)
    assert float(per_row.max()) < 2e-2, per_row


def test_all_zero_token_rows_give_zero_output_rows():
    """A zero (padding) token has scale 0 in every 1x128 group under the `absmax * (1/448)` formula; the clamp in
    front of the cast keeps its payload finite, so the row comes out as zeros, not NaN."""
    from dlblas_b200 import _C, ops
    from dlblas_b200.layers.moe.ep_moe import DlblasTritonFusedMoEBlockedF8Impl
    x, logits, w13, w13s, w2, w2s = O.make_layer_inputs(130, 512, 256, 8, seed=3)
    x[5] = 0
    x[129] = 0
    x[7, 128:256] = 0                                             # one zero group inside a live row
    ow, oids = O.softmax_topk(logits, 2, True)
    q, s = ops.quant_fp8(x.to(DEV), 128, _C.QUANT_RECIP_MUL, 0.0)
    oq, os_ = O.quant_fp8(x)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8)) and torch.equal(s.cpu(), os_)
    assert float(s[5].abs().max()) == 0.0 and int(q[5].view(torch.uint8)[0]) == 0xFE      # -448, not NaN (0x7F / 0xFF)
    layer = DlblasTritonFusedMoEBlockedF8Impl(top_k=2, num_experts=8, out_dtype=torch.bfloat16)
    out = layer.forward(x.to(DEV), ow.to(DEV), oids.to(DEV), w13.to(DEV), w13s.to(DEV), w2.to(DEV), w2s.to(DEV))
    _C.check_status()
    assert bool(torch.isfinite(out.float()).all())
    assert float(out[5].float().abs().max()) == 0.0 and float(out[129].float().abs().max()) == 0.0
    ref = O.moe_layer(x, ow, oids, w13, w13s, w2, w2s, top_k=2)
    assert bool(torch.isfinite(ref.float()).all()) and O.rel_frobenius(out.cpu(), ref) < 2e-2


def test_deepseek_routing_and_sort_bit_exact_at_full_size():
    """Config 4 sizes: 8192 tokens, 256 experts, 8 groups / 4 kept, top-8, sigmoid + bias."""
    from dlblas_b200 import ops
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(8192, 256, generator=g)
    bias = torch.randn(256, generator=g) * 0.01
    w, ids = ops.route_grouped_topk(logits.to(DEV), bias.to(DEV), 8, True, 8, 4)
    ow, oids = O.biased_grouped_topk(logits, bias, 8, True, 8, 4)
    assert torch.equal(ids.cpu(), oids)                                   # all 8192 rows, bit for bit
    torch.testing.assert_close(w.cpu(), ow, rtol=1e-5, atol=1e-7)
    assert bool((w.sum(dim=1) - 1).abs().max() < 1e-5)                    # renormalised
    assert bool(((ids // 32).cpu().unsqueeze(2) == (ids // 32).cpu().unsqueeze(1)).sum(dim=2).max() <= 8)
    groups_used = torch.zeros(8192, 8, dtype=torch.bool).scatter_(1, (ids.cpu() // 32).long(), True).sum(dim=1)
    assert int(groups_used.max()) <= 4                                     # at most topk_group groups per token
    sidx, st, en, pos, rank, cnt = ops.sort_by_expert(ids, 256, True, True, True)
    o_sidx, o_st, o_en = O.stable_sort_by_expert(ids.cpu(), 256)
    assert torch.equal(sidx.cpu(), o_sidx) and torch.equal(st.cpu(), o_st) and torch.equal(en.cpu(), o_en)
    assert int(cnt.sum()) == 8192 * 8 and torch.equal(torch.sort(sidx.cpu()).values, torch.arange(65536))


def test_fp16_layer_path():
    from dlblas_b200 import _C
    from dlblas_b200.layers.moe.kernels.blocked_fp8_fused_moe import moe_expert_forward
    x, logits, w13, w13s, w2, w2s = O.make_layer_inputs(130, 256, 256, 8, seed=9)
    x = x.to(torch.float16)
    ow, oids = O.softmax_topk(logits, 2, True)
    out = moe_expert_forward(x.to(DEV), None, None, w13.to(DEV), w13s.to(DEV), w2.to(DEV), w2s.to(DEV), ow.to(DEV),
                             oids.to(DEV), 2, torch.float16)
    _C.check_status()
    ref = O.moe_layer(x, ow, oids, w13, w13s, w2, w2s, top_k=2)
    assert out.dtype == torch.float16 and O.rel_frobenius(out.cpu(), ref) < 2e-2


def test_decode_shape_masked_layout_layer():
    """Config 5 on one GPU: 128 tokens, 256 experts, top-8 with Zipf-skewed routing, through the low-latency
    (masked layout) layer with a world of one; a sample of tokens against the oracle."""
    from dlblas_b200 import _C, ops
    from dlblas_b200.layers.moe.ep_moe import build_deepep_moe
    t, h, inter, e, k = 128, 7168, 2048, 256, 8
    g = torch.Generator().manual_seed(3)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    ranks = torch.randperm(e, generator=g).float() + 1.0
    logits = torch.randn(t, e, generator=g) + torch.log(ranks ** -1.2 / (ranks ** -1.2).sum())   # Zipf alpha = 1.2
    w13, w13s, w2, w2s = _weights_on_device(e, inter, h, 2)
    w, ids = ops.route_softmax_topk(logits.to(DEV), k, True)
    ow, oids = O.softmax_topk(logits, k, True)
    assert torch.equal(ids.cpu(), oids)
    layer = build_deepep_moe(True, 1, None, e, h, 128, k, torch.bfloat16)
    out = layer.forward(x.to(DEV), w, ids, w13, w13s, w2, w2s)
    _C.check_status()
    assert out.shape == (t, h)
    rows = torch.tensor([0, 17, 64, 127])
    hit = torch.unique(oids[rows])
    # oracle on the sampled tokens, restricted to the experts they hit (renumbered), with the scale formula of
    # the low-latency path's quantiser
    remap = torch.full((e,), -1, dtype=torch.int64)
    remap[hit] = torch.arange(hit.numel())
    ref = O.fused_moe_v2(x[rows], w13[hit.to(DEV)].cpu(), w13s[hit.to(DEV)].cpu(), w2[hit.to(DEV)].cpu(),
                         w2s[hit.to(DEV)].cpu(), ow[rows], remap[oids[rows]])
    err = O.rel_frobenius(out.cpu()[rows], ref)
    assert err < 2e-2, err
