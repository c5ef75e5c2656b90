"""The expert-parallel data path with several ranks emulated on ONE GPU.

Every emulated rank gets its own receive / return buffers (ordinary device tensors standing in for the symmetric
memory of a real rank) and the exchange kernels are given the addresses of all of them as "peer" pointers, exactly as
on several GPUs.  The phases of all ranks run one after the other on one stream, so stream order takes the place of
the barrier between the push phases (kernels that wait on one another must not share a GPU, and none runs here).
What is checked is what the multi-GPU tests check: the layer output of every rank against the CPU oracle of the full
layer, through the same kernels (quantise-and-push, metadata unpack, expert GEMMs on the receive buffer, sum-and-push,
gather; and the masked-layout variants of the decode path) and the same planning functions."""
import ctypes

import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP8 = torch.float8_e4m3fn


def _peers(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _problem(world, e, k, h, inter, tokens):
    _, _, w13, w13s, w2, w2s = O.make_layer_inputs(1, h, inter, e, seed=0)
    xs, ws, idss, refs = [], [], [], []
    for r in range(world):
        g = torch.Generator().manual_seed(20 + r)
        x = torch.randn(tokens[r], h, generator=g).to(torch.bfloat16)
        logits = torch.randn(tokens[r], e, generator=g)
        ow, oids = O.softmax_topk(logits, k, True)
        if tokens[r] > 3:
            oids[3, 1] = -1                                   # a slot without an expert
        xs.append(x.to(DEV))
        ws.append(ow.to(DEV))
        idss.append(oids.to(DEV))
        refs.append(O.moe_layer(x, ow, oids, w13, w13s, w2, w2s, top_k=k))
    nle = e // world
    local = [[t[r * nle:(r + 1) * nle].to(DEV).contiguous() for t in (w13, w13s, w2, w2s)] for r in range(world)]
    return xs, ws, idss, refs, local


@pytest.mark.parametrize("world,parts", [(2, 1), (4, 1), (2, 2)])
def test_prefill_exchange_with_emulated_ranks(world, parts):
    from dlblas_b200 import _C, ops
    from dlblas_b200.layers.moe.kernels.blocked_fp8_fused_moe import moe_expert_forward
    lib = _C.lib()
    e, k, h, inter, region = 16, 4, 512, 256, 160
    tokens = [96, 128, 8, 57][:world]
    xs, ws, idss, refs, local = _problem(world, e, k, h, inter, tokens)
    nle = e // world
    rows = world * region
    kp = (k + 1) // 2 * 2
    meta_ints = 2 * kp
    st = torch.cuda.current_stream().cuda_stream
    q = [torch.zeros(rows, h, dtype=torch.uint8, device=DEV) for _ in range(world)]
    s = [torch.zeros(rows, h // 128, dtype=torch.float32, device=DEV) for _ in range(world)]
    meta_b = [torch.zeros(rows, meta_ints, dtype=torch.int32, device=DEV) for _ in range(world)]
    counts_b = [torch.zeros(64, dtype=torch.int32, device=DEV) for _ in range(world)]
    comb = [torch.zeros(rows, h, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    pq, ps, pm, pc, pcomb = _peers(q), _peers(s), _peers(meta_b), _peers(counts_b), _peers(comb)
    within_all = []
    for r in range(world):                                     # phase 1: every rank pushes its tokens
        t = tokens[r]
        ids = idss[r]
        dest = ops.ep_dest_ranks(ids.contiguous(), nle, world)
        _, _, _, within, counts = ops.sort_by_expert(dest, world, want_rank=True, want_counts=True)
        meta = torch.zeros(t, meta_ints, dtype=torch.int32, device=DEV)
        meta[:, :k] = ids
        meta[:, kp:kp + k] = ws[r].view(torch.int32)
        _C.check(lib.dlb_p2p_quant_push(_C.ptr(xs[r]), _C.dtype_code(xs[r].dtype), t, h, h, _C.QUANT_DIV_EPS, 1e-10,
                                        _C.ptr(within), world, r, region, pq, ps, pm, _C.ptr(meta), meta_ints, pc,
                                        _C.ptr(counts), st))
        within_all.append(within.view(t, world))
    for r in range(world):                                     # phase 2: experts on the receive buffer, push back
        rids = torch.empty(rows, k, dtype=torch.int64, device=DEV)
        rw = torch.empty(rows, k, dtype=torch.float32, device=DEV)
        _C.check(lib.dlb_p2p_unpack_meta(_C.ptr(meta_b[r]), meta_ints, k, _C.ptr(counts_b[r]), world, region, r * nle,
                                         nle, _C.ptr(rids), _C.ptr(rw), st))
        assert int(counts_b[r][:world].sum()) == sum(int((within_all[src][:, r] >= 0).sum()) for src in range(world))
        slot_rows = moe_expert_forward(None, q[r].view(FP8), s[r], *local[r], rw, rids, k, torch.bfloat16, 0, nle,
                                       _C.QUANT_DIV_EPS, skip_unrouted_rows=True, return_slot_rows=True)
        if parts == 1:
            _C.check(lib.dlb_p2p_sum_push(_C.ptr(slot_rows), _C.dtype_code(slot_rows.dtype), _C.ptr(rids), k, h,
                                          _C.ptr(counts_b[r]), world, r, region, pcomb, st))
        for p in range(parts if parts > 1 else 0):               # the same, one window of the columns at a time
            _C.check(lib.dlb_p2p_sum_push_cols(_C.ptr(slot_rows), _C.dtype_code(slot_rows.dtype), _C.ptr(rids), k, h,
                                               _C.ptr(counts_b[r]), world, r, region, pcomb, st, p * (h // parts),
                                               h // parts, 8 if p == 0 else 0))
    _C.check_status()
    base = (torch.arange(world, device=DEV, dtype=torch.int32) * region)[None, :]
    for r in range(world):                                     # phase 3: every rank gathers its tokens' results
        t = tokens[r]
        if t == 0:
            continue
        within = within_all[r]
        idx = torch.where(within >= 0, within + base, torch.full_like(within, -1)).contiguous()
        out = torch.empty(t, h, dtype=torch.bfloat16, device=DEV)
        ops.ep_gather(comb[r], idx, torch.ones(t, world, device=DEV), idx, out)
        err = O.rel_frobenius(out.cpu(), refs[r])
        assert err < 2e-2, (r, err)


@pytest.mark.parametrize("world,max_tokens", [(2, 128), (4, 64)])
def test_decode_exchange_with_emulated_ranks(world, max_tokens):
    from dlblas_b200 import _C, ops
    from dlblas_b200.layers.moe.ep_moe import FusedMoELowLatency
    from dlblas_b200.layers.moe.token_dispatcher import make_low_latency_p2p_plan
    lib = _C.lib()
    e, k, h, inter = 16, 4, 512, 256
    tokens = [max_tokens, 40, 5, 17][:world]
    xs, ws, idss, refs, local = _problem(world, e, k, h, inter, tokens)
    nle = e // world
    rpe = max_tokens * world
    st = torch.cuda.current_stream().cuda_stream
    allcnt = [torch.zeros(world, e, dtype=torch.int32, device=DEV) for _ in range(world)]
    q = [torch.zeros(nle, rpe, h, dtype=torch.uint8, device=DEV) for _ in range(world)]
    s = [torch.zeros(nle, rpe, h // 128, dtype=torch.float32, device=DEV) for _ in range(world)]
    comb = [torch.zeros(max_tokens * k, h, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    pcnt, pq, ps, pcomb = _peers(allcnt), _peers(q), _peers(s), _peers(comb)
    rank_in = []
    for r in range(world):                                     # phase 0: pair counts to everybody
        _, _, _, rk, counts = ops.sort_by_expert(idss[r], e, want_rank=True, want_counts=True)
        rank_in.append(rk)
        _C.check(lib.dlb_p2p_all_gather_small(_C.ptr(counts), e * 4, world, r, pcnt, st))
    assert all(torch.equal(allcnt[0], a) for a in allcnt)
    plans = []
    for r in range(world):                                     # phase 1: quantise and store into the owners' layouts
        plan = make_low_latency_p2p_plan(allcnt[r].to(torch.int64), r, nle, rpe, idss[r], rank_in[r])
        plans.append(plan)
        pair_rank, pair_row = plan[0], plan[1]
        _C.check(lib.dlb_p2p_ll_quant_push(_C.ptr(xs[r]), _C.dtype_code(xs[r].dtype), tokens[r], h, h, _C.QUANT_DIV_EPS,
                                           1e-10, _C.ptr(pair_rank), _C.ptr(pair_row), k, world, pq, ps, st))
    layer = object.__new__(FusedMoELowLatency)                 # only the masked-layout expert MLP of the class is used
    layer.out_dtype, layer.block_size = torch.bfloat16, 128
    for r in range(world):                                     # phase 2: masked-layout experts, rows back to their source
        masked_m, row_rank, row_pos = plans[r][4], plans[r][5], plans[r][6]
        out_states = layer.experts([q[r].view(FP8), s[r]], *local[r], masked_m, 0)
        if world == 2:
            _C.check(lib.dlb_p2p_push_rows_indexed(_C.ptr(out_states), h * 2, nle * rpe, _C.ptr(row_rank),
                                                   _C.ptr(row_pos), world, pcomb, st))
        else:                                                  # the same walk over the valid rows only
            _C.check(lib.dlb_p2p_push_rows_masked(_C.ptr(out_states), h * 2, _C.ptr(masked_m), nle, rpe,
                                                  _C.ptr(row_rank), _C.ptr(row_pos), world, pcomb, st))
    _C.check_status()
    for r in range(world):                                     # phase 3: weighted gather on the source
        t = tokens[r]
        if t == 0:
            continue
        pair_pos, sent = plans[r][2].view(t, k), plans[r][3].view(t, k)
        assert bool((sent == (idss[r] >= 0)).all())            # nothing overflowed in this case
        ids32 = torch.where(sent, idss[r], torch.full_like(idss[r], -1)).to(torch.int32).contiguous()
        out = torch.empty(t, h, dtype=torch.bfloat16, device=DEV)
        ops.ep_gather(comb[r], ids32, ws[r].contiguous(), pair_pos.contiguous(), out)
        err = O.rel_frobenius(out.cpu(), refs[r])
        assert err < 2e-2, (r, err)


@pytest.mark.parametrize("world,me,e,rpe,t,k", [(4, 2, 16, 12, 40, 4), (1, 0, 8, 16, 33, 2), (8, 7, 64, 24, 128, 8),
                                                (2, 0, 6, 64, 5, 3)])
def test_plan_kernel_equals_the_tensor_arithmetic(world, me, e, rpe, t, k):
    """`dlb_p2p_ll_plan` against `make_low_latency_p2p_plan` (the same index arithmetic in plain tensor operations,
    which the CPU tests cover): every output equal, with experts whose blocks overflow (rows dropped), experts
    nobody chose and slots without an expert."""
    from dlblas_b200 import _C, ops
    from dlblas_b200.layers.moe.token_dispatcher import make_low_latency_p2p_plan
    g = torch.Generator().manual_seed(world * 100 + me)
    nle = e // world
    ids = torch.randint(0, e, (t, k), generator=g)
    ids[::7, 0] = -1
    ids[:, -1] = torch.where(torch.rand(t, generator=g) < 0.5, torch.zeros(t, dtype=torch.int64), ids[:, -1])  # crowd expert 0
    ids = ids.to(DEV)
    _, _, _, rank_in, counts = ops.sort_by_expert(ids, e, want_rank=True, want_counts=True)
    stride = (e + 3) // 4 * 4
    allcnt = torch.randint(0, max(2, 2 * rpe // max(world, 1)), (world, stride), generator=g, dtype=torch.int32).to(DEV)
    allcnt[:, 1] = 0                                              # an expert nobody chose
    allcnt[me, :e] = counts
    want = make_low_latency_p2p_plan(allcnt[:, :e].to(torch.int64), me, nle, rpe, ids, rank_in)
    pairs = t * k
    outs = [torch.full((n,), -7, dtype=torch.int32, device=DEV) for n in (pairs, pairs, pairs, pairs, nle, nle * rpe,
                                                                          nle * rpe)]
    pair_rank, pair_row, pair_pos, ids_sent, masked_m, row_rank, row_pos = outs
    _C.check(_C.lib().dlb_p2p_ll_plan(_C.ptr(allcnt), stride, world, e, me, nle, rpe, _C.ptr(ids.view(-1)),
                                      _C.ptr(rank_in), pairs, _C.ptr(pair_rank), _C.ptr(pair_row), _C.ptr(pair_pos),
                                      _C.ptr(ids_sent), _C.ptr(masked_m), _C.ptr(row_rank), _C.ptr(row_pos),
                                      torch.cuda.current_stream().cuda_stream))
    w_rank, w_row, w_pos, w_sent, w_m, w_rrank, w_rpos = want
    assert torch.equal(pair_rank, w_rank) and torch.equal(pair_row, w_row) and torch.equal(pair_pos, w_pos)
    assert torch.equal(ids_sent, torch.where(w_sent, ids.view(-1), torch.full_like(ids.view(-1), -1)).to(torch.int32))
    assert torch.equal(masked_m, w_m) and torch.equal(row_rank, w_rrank) and torch.equal(row_pos, w_rpos)
    assert bool((~w_sent & (ids.view(-1) >= 0)).any()) or world == 2    # the crowded expert overflowed somewhere
