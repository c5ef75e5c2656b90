"""GPU parity tests of the bandwidth kernels (sort, quantisers, activation, permutation, combine,
routing) against the CPU oracle and the committed golden fixtures.  Integer / byte results are
compared bit-exactly."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rand_ids(t, k, e, g, neg_frac=0.0):
    ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]) if t else torch.zeros(0, k, dtype=torch.int64)
    if neg_frac:
        ids[torch.rand(t, k, generator=g) < neg_frac] = -1
    return ids


# ------------------------------------------------------------------------------- sort
def _check_sort(ids, e, dtype=torch.int64):
    from dlblas_b200 import ops
    sidx, st, en, pos, rank, cnt = ops.sort_by_expert(ids.to(dtype).to(DEV), e, True, True, True)
    o_sidx, o_st, o_en = O.stable_sort_by_expert(ids, e)
    assert torch.equal(sidx.cpu(), o_sidx)
    assert torch.equal(st.cpu(), o_st) and torch.equal(en.cpu(), o_en)
    flat = ids.flatten()
    n = flat.numel()
    inv = torch.empty(n, dtype=torch.int64)
    inv[o_sidx] = torch.arange(n)
    exp_pos = torch.where(flat < 0, -(inv + 1), inv)
    assert torch.equal(pos.cpu().long(), exp_pos)
    valid = flat >= 0
    first = torch.zeros(e + 1, dtype=torch.int64)
    c = torch.bincount(flat[valid], minlength=e)
    assert torch.equal(cnt.cpu().long(), c)
    base = torch.cumsum(c, 0) - c + int((~valid).sum())
    exp_rank = torch.where(valid, inv - base[flat.clamp(min=0)], torch.full_like(inv, -1))
    assert torch.equal(rank.cpu().long(), exp_rank)
    assert st.data_ptr() + e * 8 == en.data_ptr()        # two rows of one [2, E] tensor, as in the reference


def test_sort_reference_vectors(golden):
    from dlblas_b200.layers.moe.kernels.fused_moe import _dlblas_get_sorted_idx
    for c in golden("sort.pt"):
        ids, e = c["topk_ids"], c["num_experts"]
        sidx, st, en = _dlblas_get_sorted_idx(ids.to(DEV), e)
        assert torch.equal(st.cpu(), c["run_exp_start"]) and torch.equal(en.cpu(), c["run_exp_end"])
        flat = ids.flatten()
        assert torch.equal(flat[sidx.cpu()], flat[c["run_sorted_idx"]])
        if "test_exp_start" in c:
            assert torch.equal(st.cpu(), c["test_exp_start"]) and torch.equal(en.cpu(), c["test_exp_end"])
            assert torch.equal(flat[sidx.cpu()], flat[c["test_sorted_idx"]])
        _check_sort(ids, e)


@pytest.mark.parametrize("t,k,e,neg", [(1, 1, 4, 0), (7, 2, 8, 0), (64, 2, 8, 0), (300, 8, 256, 0.3), (2048, 8, 256, 0),
                                       (2049, 8, 256, 0.5), (8192, 8, 256, 0), (10000, 6, 160, 0.1), (515, 4, 1000, 0)])
def test_sort_random(t, k, e, neg):
    g = torch.Generator().manual_seed(t * 31 + k)
    ids = _rand_ids(t, k, e, g, neg)
    _check_sort(ids, e)
    _check_sort(ids, e, torch.int32)


def test_sort_edge_cases():
    from dlblas_b200 import ops
    _check_sort(torch.full((64, 8), 3, dtype=torch.int64), 16)        # all tokens on one expert
    _check_sort(torch.full((40, 2), -1, dtype=torch.int64), 4)        # nothing routed here
    _check_sort(torch.full((70000, 1), 5, dtype=torch.int64), 8)      # large path, one bucket
    sidx, st, en = ops.sort_by_expert(torch.zeros(0, 8, dtype=torch.int64, device=DEV), 16)
    assert sidx.numel() == 0 and int(st.sum()) == 0 and int(en.sum()) == 0


def test_build_tiles():
    from dlblas_b200 import ops
    g = torch.Generator().manual_seed(5)
    ids = _rand_ids(1000, 4, 32, g, 0.2)
    ids[ids == 7] = 9                                                   # an empty expert
    sidx, st, en = ops.sort_by_expert(ids.to(DEV), 32)
    for off, nloc in [(0, 32), (8, 8), (24, 8)]:
        mt = ops.max_tiles_for(ids.numel(), nloc)
        tiles = ops.build_tiles(st, en, off, nloc, mt).cpu().view(-1, 4)
        n = int(tiles[0, 0])
        exp = []
        for e in range(nloc):
            s, t = int(st[e + off]), int(en[e + off])
            for r in range(s, t, 128):
                exp.append([e, r, min(128, t - r), 0])
        assert n == len(exp) and tiles[1:1 + n].tolist() == exp
    mm = torch.tensor([0, 5, 128, 129, 300], dtype=torch.int32, device=DEV)
    tiles, mt = ops.build_tiles_masked(mm, 384)
    tiles = tiles.cpu().view(-1, 4)
    assert int(tiles[0, 0]) == 7
    assert tiles[1:8].tolist() == [[1, 384, 5, 0], [2, 768, 128, 0], [3, 1152, 128, 0], [3, 1280, 1, 0],
                                   [4, 1536, 128, 0], [4, 1664, 128, 0], [4, 1792, 44, 0]]


# ------------------------------------------------------------------------------- quant
def test_quant_golden_scales(golden):
    from dlblas_b200.kernels.fp8 import per_token_group_quant_fp8
    from dlblas_b200.kernels.moe import quant_fp8
    g = golden("quant.pt")
    x = g["x"].to(DEV)
    q, s = quant_fp8(x, 128)
    assert torch.equal(s.cpu(), g["scale_quant_fp8"])
    oq, _ = O.quant_fp8(g["x"], 128)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))
    q2, s2 = per_token_group_quant_fp8(x, 128)
    assert torch.equal(s2.cpu(), g["scale_per_token_group"])
    q3, s3 = per_token_group_quant_fp8(x, 128, column_major_scales=True)
    assert tuple(s3.stride()) == tuple(g["colmajor_stride"]) and torch.equal(s3.cpu().contiguous(), g["scale_colmajor"])
    oq2, _ = O.per_token_group_quant_fp8(g["x"], 128)
    assert torch.equal(q2.cpu().view(torch.uint8), oq2.view(torch.uint8))
    assert torch.equal(q3.cpu().view(torch.uint8), oq2.view(torch.uint8))


@pytest.mark.parametrize("m,k,dtype", [(1, 128, torch.bfloat16), (33, 512, torch.bfloat16), (257, 7168, torch.bfloat16),
                                       (64, 1024, torch.float16), (19, 256, torch.float32)])
@pytest.mark.parametrize("group", [128, 64])
def test_quant_bit_exact(m, k, dtype, group):
    from dlblas_b200 import _C, ops
    g = torch.Generator().manual_seed(m + k)
    x = (torch.randn(m, k, generator=g) * torch.rand(m, 1, generator=g) * 10).to(dtype)
    for mode, ofn in [(_C.QUANT_RECIP_MUL, O.quant_fp8), (_C.QUANT_DIV_EPS, O.per_token_group_quant_fp8)]:
        q, s = ops.quant_fp8(x.to(DEV), group, mode, 1e-10)
        oq, os_ = ofn(x, group)
        assert torch.equal(s.cpu(), os_)
        assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))
    # 3-D input through the reference-shaped wrapper
    from dlblas_b200.kernels.fp8 import per_token_group_quant_fp8
    if m % 3 == 0:
        q, s = per_token_group_quant_fp8(x.view(3, m // 3, k).to(DEV), group)
        assert q.shape == (3, m // 3, k) and s.shape == (3, m // 3, k // group)


def test_quant_zero_group():
    from dlblas_b200.kernels.fp8 import per_token_group_quant_fp8
    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    x[1, 5] = 3.0
    q, s = per_token_group_quant_fp8(x.to(DEV), 128)
    oq, os_ = O.per_token_group_quant_fp8(x, 128)
    assert torch.equal(s.cpu(), os_) and torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))


def test_quant_zero_group_under_the_reciprocal_formula():
    """`quant_fp8` (scale = absmax * (1/448), no epsilon): an all-zero group has scale 0 and its payload is the
    clamped -448 of the reference's compiled kernel, never NaN; fused fan-out and the silu*up quantiser agree."""
    from dlblas_b200 import _C, ops
    x = torch.randn(6, 384).to(torch.bfloat16)
    x[1] = 0
    x[3, 128:256] = 0
    q, s = ops.quant_fp8(x.to(DEV), 128, _C.QUANT_RECIP_MUL, 0.0)
    oq, os_ = O.quant_fp8(x)
    assert torch.equal(s.cpu(), os_) and torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))
    assert bool((q[1].view(torch.uint8) == 0xFE).all()) and bool(torch.isfinite(q.float()).all())
    gu = torch.randn(5, 512).to(torch.bfloat16)
    gu[2] = 0                                                       # silu(0) * 0 = 0 in every group
    hq, hs = ops.silu_mul_quant(gu.to(DEV), _C.QUANT_RECIP_MUL, 0.0, False)
    assert bool(torch.isfinite(hq.float()).all()) and float(hs[2].abs().max()) == 0.0
    assert bool((hq[2].view(torch.uint8) == 0xFE).all())


def test_tma_align_input_scale():
    """dlblas/kernels/quant_dequant.py:65-83: same values in a column-major buffer whose rows are padded to 16 B;
    and the quantiser's own column-major output carries the same values."""
    from dlblas_b200.kernels.fp8 import per_token_group_quant_fp8
    from dlblas_b200.kernels.quant_dequant import tma_align_input_scale
    for m, k in [(7, 512), (130, 7168), (1, 128)]:
        x = torch.randn(m, k).to(torch.bfloat16)
        q, s = per_token_group_quant_fp8(x.to(DEV), 128)
        a = tma_align_input_scale(s)
        o = O.tma_align_input_scale(s.cpu())
        assert a.shape == o.shape and a.stride() == o.stride() and torch.equal(a.cpu(), o)
        assert a.stride(0) == 1 and a.stride(1) % 4 == 0
        _, sc = per_token_group_quant_fp8(x.to(DEV), 128, column_major_scales=True)
        assert sc.stride(0) == 1 and torch.equal(sc.cpu(), s.cpu())


def test_quant_fused_with_permutation():
    from dlblas_b200 import _C, ops
    g = torch.Generator().manual_seed(9)
    t, k, h, e = 100, 4, 512, 16
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    ids = _rand_ids(t, k, e, g, 0.25)
    sidx, st, en, pos = ops.sort_by_expert(ids.to(DEV), e, want_pos=True)
    q, s = ops.quant_fp8(x.to(DEV), 128, _C.QUANT_RECIP_MUL, 0.0, False, pos, k, t * k)
    oq, os_ = O.quant_fp8(x, 128)
    o_sidx, _, _ = O.stable_sort_by_expert(ids, e)
    n_neg = int((ids < 0).sum())
    src = (o_sidx // k)[n_neg:]
    assert torch.equal(q.cpu().view(torch.uint8)[n_neg:], oq.view(torch.uint8)[src])
    assert torch.equal(s.cpu()[n_neg:], os_[src])
    # same movement for rows that are already quantised
    q2, s2 = ops.permute_rows(oq.to(DEV), os_.to(DEV), pos, k, t * k)
    assert torch.equal(q2.cpu().view(torch.uint8)[n_neg:], oq.view(torch.uint8)[src])
    assert torch.equal(s2.cpu()[n_neg:], os_[src])


# ------------------------------------------------------------------------------- activation
def test_silu_and_mul(golden):
    from dlblas_b200.kernels.activation import silu_and_mul
    from dlblas_b200.layers.moe.kernels.activation import silu_and_mul as silu2
    g = golden("silu_and_mul.pt")
    out = silu_and_mul(g["gate_up"].to(DEV))
    torch.testing.assert_close(out.cpu(), g["out_fp32"], rtol=2e-6, atol=2e-6)
    gu = (g["gate_up"]).to(torch.bfloat16)
    out = silu2(gu.to(DEV))
    ref = O.silu_and_mul(gu)
    # __expf vs exp: at most one bf16 ulp apart, on a tiny fraction of elements
    diff = (out.cpu().float() - ref.float()).abs()
    assert float(diff.max()) <= float(ref.float().abs().max()) * 2 ** -7
    assert float((diff > 0).float().mean()) < 0.02
    buf = torch.empty(24, 256, dtype=torch.bfloat16, device=DEV)
    assert silu2(gu.to(DEV), buf) is buf and torch.equal(buf, out)


@pytest.mark.parametrize("round_silu", [False, True])
def test_silu_mul_quant(round_silu):
    from dlblas_b200 import _C, ops
    g = torch.Generator().manual_seed(11)
    e, m, n = 3, 40, 256
    inp = (torch.randn(e, m, 2 * n, generator=g) * 2).to(torch.bfloat16)
    masked_m = torch.tensor([40, 0, 17], dtype=torch.int32)
    if round_silu:
        from dlblas_b200.kernels.moe import silu_and_mul_masked_post_quant_fwd
        out = torch.zeros(e, m, n, dtype=torch.float8_e4m3fn, device=DEV)
        out_s = torch.zeros(e, m, n // 128, dtype=torch.float32, device=DEV)
        silu_and_mul_masked_post_quant_fwd(inp.to(DEV), out, out_s, 128, masked_m.to(DEV))
        oq, os_ = O.silu_and_mul_masked_post_quant(inp, masked_m)
    else:
        out, out_s = ops.silu_mul_quant(inp.view(e * m, 2 * n).to(DEV), _C.QUANT_RECIP_MUL)
        oq, os_ = O.quant_fp8(O.silu_and_mul(inp.view(e * m, 2 * n)), 128)
        out, out_s, oq, os_ = out.view(e, m, n), out_s.view(e, m, -1), oq.view(e, m, n), os_.view(e, m, -1)
        masked_m = torch.tensor([m, m, m])
    for i in range(e):
        r = int(masked_m[i])
        a = out.cpu()[i, :r].float() * out_s.cpu()[i, :r].repeat_interleave(128, dim=1)
        b = oq[i, :r].float() * os_[i, :r].repeat_interleave(128, dim=1)
        if r:
            assert O.rel_frobenius(a, b) < 5e-3         # exp flavour differs: rare one-ulp flips before quantisation
            torch.testing.assert_close(out_s.cpu()[i, :r], os_[i, :r], rtol=2 ** -7, atol=0)
        if round_silu and r < m:
            assert float(out.cpu()[i, r:].float().abs().max()) == 0.0   # rows beyond masked_m untouched


# ------------------------------------------------------------------------------- combine / scatter / gather
def test_sum_topk_and_masked_variant():
    from dlblas_b200 import ops
    g = torch.Generator().manual_seed(12)
    t, k, h = 37, 4, 512
    y = torch.randn(t * k, h, generator=g).to(torch.bfloat16)
    out = ops.sum_topk(y.to(DEV), t, k)
    assert torch.equal(out.cpu(), y.view(t, k, h).sum(dim=1))
    ids = _rand_ids(t, k, 8, g)
    out = ops.sum_topk(y.to(DEV), t, k, ids.to(DEV), 2, 6)
    keep = ((ids >= 2) & (ids < 6))[..., None]
    assert torch.equal(out.cpu(), torch.where(keep, y.view(t, k, h).float(), torch.zeros(())).sum(dim=1).to(torch.bfloat16))


def test_scatter_gather(golden):
    from dlblas_b200.kernels.fused_moe_v3 import ep_gather, ep_scatter
    g = golden("scatter_gather.pt")
    x, xs, topk, counts = g["x"], g["xs"], g["topk"], g["counts"]
    total = int(counts.sum())
    out_x = torch.zeros(total, x.shape[1], dtype=x.dtype, device=DEV)
    out_s = torch.zeros(total, xs.shape[1], device=DEV)
    m_idx = torch.zeros(total, dtype=torch.int32, device=DEV)
    out_index = torch.zeros_like(topk, device=DEV)
    start = torch.zeros_like(counts, device=DEV)
    ep_scatter(x.to(DEV), xs.to(DEV), topk.to(DEV), counts.to(DEV), start, out_x, out_s, m_idx, out_index)
    o_x, o_s, o_m, o_index, o_start = O.ep_scatter(x, xs, topk, counts)
    assert torch.equal(m_idx.cpu(), g["m_indices"]) and torch.equal(m_idx.cpu(), o_m)
    assert torch.equal(start.cpu().long(), o_start)
    ok = topk >= 0
    assert torch.equal(out_index.cpu()[ok], o_index[ok])                 # canonical (deterministic) slots
    assert torch.equal(out_x.cpu().view(torch.uint8), o_x.view(torch.uint8)) and torch.equal(out_s.cpu(), o_s)
    # against the reference run: same rows behind its own index map
    gi = g["output_index"]
    assert torch.equal(out_x.cpu().view(torch.uint8)[out_index.cpu()[ok].long()],
                       g["out_x"].view(torch.uint8)[gi[ok].long()])
    gat = torch.empty(topk.shape[0], x.shape[1], dtype=torch.float32, device=DEV)
    ep_gather(g["y"].float().to(DEV), topk.to(DEV), g["wt"].to(DEV), g["output_index"].to(DEV), gat)
    torch.testing.assert_close(gat.cpu(), g["gather_fp32"], rtol=1e-5, atol=1e-5)
    gat16 = torch.empty(topk.shape[0], x.shape[1], dtype=torch.bfloat16, device=DEV)
    ep_gather(g["y"].to(DEV), topk.to(DEV), g["wt"].to(DEV), g["output_index"].to(DEV), gat16)
    assert torch.equal(gat16.cpu(), O.ep_gather(g["y"], topk, g["wt"], g["output_index"]))


# ------------------------------------------------------------------------------- routing
def _margin_ok(scores, k, rel=1e-5):
    top = torch.topk(scores, min(k + 1, scores.shape[1]), dim=1).values
    gap = (top[:, :-1] - top[:, 1:]).abs() / top[:, :-1].abs().clamp_min(1e-30)
    return gap.min(dim=1).values > rel


@pytest.mark.parametrize("t,e,k", [(64, 8, 2), (4096, 8, 2), (1000, 64, 8), (333, 256, 8), (50, 1000, 16), (0, 8, 2)])
@pytest.mark.parametrize("renorm", [False, True])
def test_softmax_topk(t, e, k, renorm):
    from dlblas_b200 import ops
    g = torch.Generator().manual_seed(t + e)
    logits = torch.randn(t, e, generator=g)
    w, ids = ops.route_softmax_topk(logits.to(DEV), k, renorm)
    if t == 0:
        return
    ow, oids = O.softmax_topk(logits, k, renorm)
    ok = _margin_ok(torch.softmax(logits, 1), k)
    assert float(ok.float().mean()) > 0.99
    assert torch.equal(ids.cpu()[ok], oids[ok])
    torch.testing.assert_close(w.cpu()[ok], ow[ok], rtol=2e-6, atol=1e-8)
    w32, ids32 = ops.route_softmax_topk(logits.to(DEV), k, renorm, torch.int32)
    assert ids32.dtype == torch.int32 and torch.equal(ids32.long(), ids)


def test_softmax_topk_ties_take_the_lowest_index():
    from dlblas_b200 import ops
    logits = torch.zeros(5, 64)
    logits[1, 40:] = 1.0
    logits[2] = torch.arange(64).float().flip(0) // 8          # eight-way ties
    w, ids = ops.route_softmax_topk(logits.to(DEV), 4)
    ow, oids = O.softmax_topk(logits, 4)
    assert torch.equal(ids.cpu(), oids)
    assert ids.cpu()[0].tolist() == [0, 1, 2, 3] and ids.cpu()[1].tolist() == [40, 41, 42, 43]
    lb = torch.randint(0, 4, (64, 32)).to(torch.bfloat16)      # bf16 logits tie in almost every row
    w, ids = ops.route_softmax_topk(lb.to(DEV), 8)
    assert torch.equal(ids.cpu(), O.softmax_topk(lb, 8)[1])


def _grouped_decision_gap(logits, bias, topk, num_groups, topk_group):
    """Per row, the smallest gap of a routing decision on the canonical scores: between the last kept and the
    first dropped group score, and between the k-th and (k+1)-th biased score inside the kept groups."""
    sc = O.sigmoid_exact(logits.float())
    ch = sc + bias.float()[None, :]
    t, e = ch.shape
    gs = ch.view(t, num_groups, -1).topk(2, dim=-1).values.sum(-1)
    gsort = gs.sort(dim=1, descending=True).values
    ggap = gsort[:, topk_group - 1] - gsort[:, topk_group] if topk_group < num_groups else torch.full((t,), 1.0)
    keep = torch.zeros(t, num_groups, dtype=torch.bool).scatter_(1, gs.topk(topk_group, dim=1).indices, True)
    masked = ch.masked_fill(~keep[:, :, None].expand(t, num_groups, e // num_groups).reshape(t, e), -float("inf"))
    top = masked.topk(topk + 1, dim=1).values
    return torch.minimum(ggap, top[:, topk - 1] - top[:, topk])


def test_grouped_topk(golden):
    """Ids equal the oracle on every row (the scores are reproducible bit for bit); against the reference's own
    run, whose fp32 sigmoid is only defined to an ulp or two, every row that differs is a proven near-tie."""
    from dlblas_b200.kernels.moe import biased_grouped_topk
    for c in golden("grouped_topk.pt"):
        lg = c["logits"].to(DEV)
        w, ids = biased_grouped_topk(lg, lg, c["bias"].to(DEV), c["topk"], True, c["num_expert_group"], c["topk_group"])
        assert w.dtype == torch.float32 and ids.dtype == torch.int32
        ow, oids = O.biased_grouped_topk(c["logits"], c["bias"], c["topk"], True, c["num_expert_group"], c["topk_group"])
        assert torch.equal(ids.cpu(), oids)
        torch.testing.assert_close(w.cpu(), ow, rtol=1e-5, atol=1e-7)
        # against the reference's own output: same expert sets, same weights, except on near-ties
        a, ia = torch.sort(ids.cpu().long(), dim=1)
        b, ib = torch.sort(c["ids"].long(), dim=1)
        rows = (a == b).all(dim=1)
        gap = _grouped_decision_gap(c["logits"], c["bias"], c["topk"], c["num_expert_group"], c["topk_group"])
        assert bool((gap[~rows] <= 1e-6).all()), gap[~rows]          # a few ulps of a score near 0.5 .. 1
        assert float(rows.float().mean()) > 0.99
        torch.testing.assert_close(w.cpu().gather(1, ia)[rows], c["weights"].gather(1, ib)[rows], rtol=1e-5, atol=1e-6)


def test_grouped_topk_large_and_ties():
    from dlblas_b200 import ops
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(8192, 256, generator=g)
    bias = torch.randn(256, generator=g) * 0.01
    w, ids = ops.route_grouped_topk(logits.to(DEV), bias.to(DEV), 8, True, 8, 4)
    ow, oids = O.biased_grouped_topk(logits, bias, 8, True, 8, 4)
    assert torch.equal(ids.cpu(), oids)                          # every row, bit for bit
    torch.testing.assert_close(w.cpu(), ow, rtol=1e-5, atol=1e-7)
    for dt in (torch.bfloat16, torch.float16):                   # 16-bit logits tie in most rows
        lb = logits.to(dt)
        _, ids16 = ops.route_grouped_topk(lb.to(DEV), bias.to(DEV), 8, True, 8, 4)
        assert torch.equal(ids16.cpu(), O.biased_grouped_topk(lb, bias, 8, True, 8, 4)[1])
    z = torch.zeros(4, 256)
    w, ids = ops.route_grouped_topk(z.to(DEV), torch.zeros(256, device=DEV), 8, False, 8, 4)
    assert ids.cpu()[0].tolist() == list(range(8))               # all equal: lowest groups, lowest experts
    assert torch.equal(ids.cpu(), O.biased_grouped_topk(z, torch.zeros(256), 8, False, 8, 4)[1])
    big = torch.tensor([[-1e30, 1e30, 800.0, -800.0] * 64])      # saturated scores stay finite and ordered
    _, idb = ops.route_grouped_topk(big.to(DEV), torch.zeros(256, device=DEV), 8, False, 8, 4)
    assert torch.equal(idb.cpu(), O.biased_grouped_topk(big, torch.zeros(256), 8, False, 8, 4)[1])


def test_topk_gating(golden):
    import dlblas_b200
    for c in golden("topk_gating.pt"):
        out = dlblas_b200.topk_gating(c["logits"].to(DEV), c["k"], c["capacity_factor"], c["min_capacity"],
                                      c["higher_precision"])
        l_aux, ec, w, sel = [o.cpu() for o in out]
        o_l, o_ec, o_w, o_sel = O.topk_gating(c["logits"], c["k"], c["capacity_factor"], c["min_capacity"])
        torch.testing.assert_close(l_aux, c["l_aux"], rtol=1e-5, atol=1e-7)
        assert ec.dtype == torch.int32 and torch.equal(ec, c["ec_idx"]) and torch.equal(ec, o_ec)
        torch.testing.assert_close(w, c["weights"], rtol=1e-5, atol=1e-7)
        assert sel.dtype == torch.int64 and torch.equal(sel, o_sel)


@pytest.mark.parametrize("t,e,k,cf", [(4096, 64, 8, 1.0), (1000, 8, 2, 0.5), (512, 256, 8, 2.0)])
def test_topk_gating_random(t, e, k, cf):
    import dlblas_b200
    g = torch.Generator().manual_seed(t)
    logits = torch.randn(t, e, generator=g)
    l_aux, ec, w, sel = [o.cpu() for o in dlblas_b200.topk_gating(logits.to(DEV), k, cf, 2)]
    o_l, o_ec, o_w, o_sel = O.topk_gating(logits, k, cf, 2)
    ok = _margin_ok(torch.softmax(logits, 1), k)
    if bool(ok.all()):
        assert torch.equal(ec, o_ec) and torch.equal(sel, o_sel)
        torch.testing.assert_close(w, o_w, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(l_aux, o_l, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("higher_precision", [False, True])
def test_topk_gating_backward(golden, higher_precision):
    import dlblas_b200
    for c in golden("topk_gating_bwd.pt"):
        logits = c["logits"].to(DEV).requires_grad_(True)
        l_aux, ec, w, sel = dlblas_b200.topk_gating(logits, c["k"], c["capacity_factor"], c["min_capacity"],
                                                    higher_precision)
        gw = c["grad_weights"].to(DEV)
        (l_aux * 0.7 + (w * gw).sum()).backward()
        ref = O.topk_gating_grad(c["logits"], c["k"], c["capacity_factor"], c["min_capacity"], c["grad_l_aux"],
                                 c["grad_weights"] if higher_precision else None)
        torch.testing.assert_close(logits.grad.cpu(), ref, rtol=2e-4, atol=1e-6)
        if not higher_precision:
            torch.testing.assert_close(logits.grad.cpu(), c["grad_logits_default"], rtol=2e-4, atol=1e-6)
    # fp16 logits, larger case
    g = torch.Generator().manual_seed(5)
    lg = torch.randn(300, 64, generator=g)
    x = lg.half().to(DEV).requires_grad_(True)
    l_aux, ec, w, sel = dlblas_b200.topk_gating(x, 4, 1.0, 2, higher_precision)
    gw = torch.randn(4 * 300, generator=g)
    (l_aux.float() * 0.7 + (w.float() * gw.to(DEV)).sum()).backward()
    ref = O.topk_gating_grad(lg.half().float(), 4, 1.0, 2, 0.7, gw.half().float() if higher_precision else None)
    assert x.grad.dtype == torch.float16
    tol = 2e-2 * float(ref.abs().max()) + 1e-6
    assert float((x.grad.cpu().float() - ref).abs().max()) <= tol
