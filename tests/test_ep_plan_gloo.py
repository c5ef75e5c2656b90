"""Expert-parallel exchange planning on CPU: two gloo ranks run the same planning code the GPU
path uses (token_dispatcher.make_normal_plan / make_low_latency_plan), move rows with plain torch
indexing in place of the CUDA permutation kernels, and check that dispatch followed by combine
is the identity on a per-expert tagging function."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _expert_fn(rows, expert):
    """Stand-in for an expert: a function of (row content, global expert id)."""
    return rows * (1.0 + expert.float()[:, None]) + expert.float()[:, None]


def _worker(rank, world, port, ret):
    from dlblas_b200.layers.moe import token_dispatcher as td
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100 + rank)
        e, k, h = 8, 3, 4
        nle = e // world
        t = 17 + 5 * rank
        x = torch.randn(t, h, generator=g)
        ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)])
        ids[0, 1] = -1                                           # an unrouted slot
        w = torch.rand(t, k, generator=g)
        # ---- normal mode -------------------------------------------------------------------
        plan = td.make_normal_plan(ids, world, rank, nle, dist.group.WORLD, expert_alignment=4)
        assert plan.dst_pos.shape == (t, world) and plan.num_send == int((plan.dst_pos >= 0).sum())
        send = torch.zeros(plan.num_send, h)
        send_ids = torch.zeros(plan.num_send, k, dtype=torch.int64)
        send_w = torch.zeros(plan.num_send, k)
        for tok in range(t):
            for r in range(world):
                d = int(plan.dst_pos[tok, r])
                if d >= 0:
                    send[d] = x[tok]
                    send_ids[d] = td.localize_ids(ids[tok:tok + 1], torch.tensor([r]), nle)[0]
                    send_w[d] = w[tok]
        # rows for one destination are contiguous and in token order
        flat = plan.dst_pos.t()[plan.dst_pos.t() >= 0]
        assert torch.equal(flat, torch.arange(plan.num_send, dtype=torch.int32))
        recv = torch.zeros(plan.num_recv, h)
        recv_ids = torch.zeros(plan.num_recv, k, dtype=torch.int64)
        recv_w = torch.zeros(plan.num_recv, k)
        td._a2a(recv, send, plan.recv_splits, plan.send_splits, dist.group.WORLD, world)
        td._a2a(recv_ids, send_ids, plan.recv_splits, plan.send_splits, dist.group.WORLD, world)
        td._a2a(recv_w, send_w, plan.recv_splits, plan.send_splits, dist.group.WORLD, world)
        assert int(((recv_ids >= nle) | (recv_ids < -1)).sum()) == 0       # ids are local to this rank
        cnt = torch.bincount(recv_ids[recv_ids >= 0], minlength=nle)
        assert plan.recv_tokens_per_expert == [int((c + 3) // 4 * 4) for c in cnt]
        # "experts": weighted sum over the local slots of every received row
        part = torch.zeros(plan.num_recv, h)
        for j in range(k):
            ok = recv_ids[:, j] >= 0
            part += torch.where(ok[:, None], _expert_fn(recv, recv_ids[:, j] + rank * nle) * recv_w[:, j:j + 1],
                                torch.zeros(()))
        back = torch.zeros(plan.num_send, h)
        td._a2a(back, part, plan.send_splits, plan.recv_splits, dist.group.WORLD, world)
        out = torch.zeros(t, h)
        for tok in range(t):
            for r in range(world):
                d = int(plan.dst_pos[tok, r])
                if d >= 0:
                    out[tok] += back[d]
        ref = torch.zeros(t, h)
        for j in range(k):
            ok = ids[:, j] >= 0
            ref += torch.where(ok[:, None], _expert_fn(x, ids[:, j]) * w[:, j:j + 1], torch.zeros(()))
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)

        # ---- low-latency mode ----------------------------------------------------------------
        ids2 = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)])
        flat_ids = ids2.flatten()
        counts = torch.bincount(flat_ids, minlength=e)
        rpe = 64
        lp = td.make_low_latency_plan(counts, world, rank, nle, dist.group.WORLD, rpe)
        order = torch.argsort(flat_ids, stable=True)               # send order: pairs sorted by expert
        send = x[order // k]
        tag = flat_ids[order].float()
        recv = torch.zeros(lp.num_recv, h)
        recv_tag = torch.zeros(lp.num_recv)
        td._a2a(recv, send, lp.recv_splits, lp.send_splits, dist.group.WORLD, world)
        td._a2a(recv_tag, tag, lp.recv_splits, lp.send_splits, dist.group.WORLD, world)
        packed = torch.full((nle * rpe, h), float("nan"))
        packed_tag = torch.full((nle * rpe,), -1.0)
        packed[lp.recv_dst.long()] = recv
        packed_tag[lp.recv_dst.long()] = recv_tag
        assert lp.recv_dst.unique().numel() == lp.num_recv
        for j in range(nle):                                        # rows of expert j are the first masked_m[j] of its slab
            m = int(lp.masked_m[j])
            assert bool((packed_tag[j * rpe: j * rpe + m] == rank * nle + j).all())
            assert bool((packed_tag[j * rpe + m: (j + 1) * rpe] == -1).all())
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_plans_on_gloo():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert dict(ret) == {0: "ok", 1: "ok"}
    assert all(p.exitcode == 0 for p in procs)


def test_single_rank_plan_without_process_group():
    from dlblas_b200.layers.moe import token_dispatcher as td
    ids = torch.tensor([[0, 3], [2, -1], [1, 1]])
    plan = td.make_normal_plan(ids, 1, 0, 4, None, expert_alignment=128)
    assert plan.send_splits == [3] and plan.recv_splits == [3]
    assert plan.dst_pos.flatten().tolist() == [0, 1, 2]
    assert plan.recv_tokens_per_expert == [128, 128, 128, 128]
    lp = td.make_low_latency_plan(torch.tensor([1, 2, 0, 1]), 1, 0, 4, None, 8)
    assert lp.masked_m.tolist() == [1, 2, 0, 1] and lp.recv_dst.tolist() == [0, 8, 9, 24]
    # the device-side plan of a world of one: same destinations, buffers sized for every (token, slot) pair,
    # pairs without an expert (they sort to the end of the send order) dropped
    sp = td.make_single_rank_plan(torch.tensor([1, 2, 0, 1]), 6, 8)
    assert sp.masked_m.tolist() == [1, 2, 0, 1] and sp.num_send == sp.num_recv == 6
    assert sp.recv_dst.tolist() == [0, 8, 9, 24, -1, -1]


def test_host_free_low_latency_plan_round_trip():
    """The index arithmetic of the peer-to-peer low-latency exchange, with the ranks emulated in one process: every
    sent pair lands in a distinct row of its expert's block on the owner, the block is filled without holes in
    (source rank, rank inside the source) order, and the owner's return addresses lead back to the pair's own row
    of the source's return buffer.  Includes unrouted slots, an empty expert and an overfull block."""
    from dlblas_b200.layers.moe.token_dispatcher import make_low_latency_p2p_plan
    for w, e, k, tokens, rpe in [(4, 16, 4, [7, 0, 12, 5], 16), (2, 8, 2, [9, 9], 4), (8, 32, 8, [3] * 8, 24)]:
        nle = e // w
        g = torch.Generator().manual_seed(w * 100 + e)
        ids, rank_in, counts = [], [], []
        for r in range(w):
            t = tokens[r]
            x = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]) if t else torch.zeros(0, k).long()
            x[x == 1] = 0                                             # expert 1 stays empty, expert 0 is crowded
            if t:
                x[0, 0] = -1                                          # a slot without an expert
            flat = x.reshape(-1)
            rk = torch.full_like(flat, -1)
            seen = {}
            for f, ex in enumerate(flat.tolist()):
                if ex >= 0:
                    rk[f] = seen.get(ex, 0)
                    seen[ex] = rk[f] + 1
            ids.append(x)
            rank_in.append(rk.to(torch.int32))
            counts.append(torch.bincount(flat[flat >= 0], minlength=e))
        c = torch.stack(counts).to(torch.int64)
        plans = [make_low_latency_p2p_plan(c, r, nle, rpe, ids[r], rank_in[r]) for r in range(w)]
        # dispatch: every owner's masked layout records (source, flat pair index)
        layout = [dict() for _ in range(w)]
        for r in range(w):
            pair_rank, pair_row, pair_pos, sent, _, _, _ = plans[r]
            flat = ids[r].reshape(-1)
            for f in range(flat.numel()):
                if flat[f] < 0:
                    assert not sent[f] and pair_rank[f] == -1 and pair_pos[f] == -1
                    continue
                if not sent[f]:
                    continue
                owner, row = int(pair_rank[f]), int(pair_row[f])
                assert owner == int(flat[f]) // nle and row // rpe == int(flat[f]) % nle
                assert row not in layout[owner], "two pairs in one row"
                layout[owner][row] = (r, f)
        for o in range(w):
            _, _, _, _, masked_m, row_rank, row_pos = plans[o]
            total = c[:, o * nle:(o + 1) * nle].sum(0)
            assert torch.equal(masked_m.long(), total.clamp(max=rpe))
            for le in range(nle):
                rows = [layout[o].get(le * rpe + i) for i in range(rpe)]
                filled = [x for x in rows if x is not None]
                assert rows[:len(filled)] == filled and len(filled) == int(masked_m[le])   # no holes
                assert filled == sorted(filled)                                              # source, then rank order
                for i in range(rpe):
                    rr = int(row_rank[le * rpe + i])
                    if i < int(total[le]):
                        assert rr >= 0
                    else:
                        assert rr == -1
                    if i < len(filled):
                        src, f = filled[i]
                        assert rr == src and int(row_pos[le * rpe + i]) == int(plans[src][2][f])
        for r in range(w):                                            # return rows of a source are distinct and dense
            pos = plans[r][2][plans[r][3]]
            assert pos.numel() == torch.unique(pos).numel()
            assert pos.numel() == 0 or int(pos.max()) < int(c[r].sum())
