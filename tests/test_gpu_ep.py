"""Expert-parallel layers on 2 GPUs (NCCL): FusedMoENormal and FusedMoELowLatency against the CPU
oracle of the full layer.  Skipped when fewer than 2 GPUs are visible."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    from dlblas_b200 import _C
    from dlblas_b200.layers.moe.ep_moe import build_deepep_moe
    from oracle import moe_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        e, k, h, inter = 16, 4, 512, 256
        nle = e // world
        # every rank builds the same weights (seed 0) and its own tokens
        _, _, w13, w13s, w2, w2s = O.make_layer_inputs(1, h, inter, e, seed=0)
        t = 96 + 32 * rank
        g = torch.Generator().manual_seed(10 + rank)
        x = torch.randn(t, h, generator=g).to(torch.bfloat16)
        logits = torch.randn(t, e, generator=g)
        ow, oids = O.softmax_topk(logits, k, True)
        ref = O.moe_layer(x, ow, oids, w13, w13s, w2, w2s, top_k=k)
        ids_u = oids.clone()
        ids_u[::3, 1] = -1
        ids_u[5] = -1
        ref_u = O.moe_layer(x, ow, ids_u, w13, w13s, w2, w2s, top_k=k)
        sl = slice(rank * nle, (rank + 1) * nle)
        local = [w13[sl].to(dev), w13s[sl].to(dev), w2[sl].to(dev), w2s[sl].to(dev)]
        os.environ["DLBLAS_EP_MAX_TOKENS"] = "256"
        first_p2p = None
        for backend, low_latency in (("p2p", False), ("p2p-parts", False), ("p2p-chunked", False), ("nccl", False),
                                     ("nccl", True), ("p2p", True)):
            # two token chunks on two streams (ranks hold 96 and 128 tokens: chunks of 48 / 64)
            os.environ["DLBLAS_EP_MIN_CHUNK_ROWS"] = "32" if backend == "p2p-chunked" else "1024"
            os.environ["DLBLAS_EP_CHUNKS"] = "2" if backend == "p2p-chunked" else "1"
            # the chunked run also takes the unfused combine (sum kernel, then push) so that both stay covered
            os.environ["DLBLAS_EP_FUSED_COMBINE"] = "0" if backend == "p2p-chunked" else "1"
            # second GEMM in two windows of the hidden dimension, the first window pushed back while the second runs
            os.environ["DLBLAS_EP_W2_PARTS"] = "2" if backend == "p2p-parts" else "1"
            parts_run = backend == "p2p-parts"
            backend = backend.split("-")[0]
            os.environ["DLBLAS_EP_BACKEND"] = backend
            layer = build_deepep_moe(low_latency, world, dist.group.WORLD, e, h, 128, k, torch.bfloat16)
            if low_latency:
                assert type(layer.token_dispatcher).__name__ == ("TokenDispatcherLowLatencyP2P" if backend == "p2p"
                                                                 else "TokenDispatcherLowLatency")
            else:
                assert (getattr(layer, "p2p_dispatcher", None) is not None) == (backend == "p2p")
            if backend == "p2p" and not low_latency:
                assert len(layer.p2p_chunks) == (2 if os.environ["DLBLAS_EP_MIN_CHUNK_ROWS"] == "32" else 1)
            for _ in range(3):                      # repeated steps reuse the symmetric buffers
                out = layer.forward(x.to(dev), ow.to(dev), oids.to(dev), *local)
            _C.check_status(dev)
            err = O.rel_frobenius(out.cpu(), ref)
            assert out.shape == (t, h) and err < 2e-2, (backend, low_latency, err)
            if backend == "p2p" and not low_latency and first_p2p is None:
                first_p2p = out.clone()
            if parts_run:
                assert torch.equal(out, first_p2p)   # same sums in the same order, column window by column window
            # slots without an expert (id -1) are dropped by every exchange
            out_u = layer.forward(x.to(dev), ow.to(dev), ids_u.to(dev), *local)
            _C.check_status(dev)
            err_u = O.rel_frobenius(out_u.cpu(), ref_u)
            assert err_u < 2e-2, (backend, low_latency, "unrouted slots", err_u)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def _setup(rank, world, port):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    return dev


def _inputs(rank, world, dev, e=16, k=4, h=512, inter=256):
    from oracle import moe_oracle as O
    nle = e // world
    _, _, w13, w13s, w2, w2s = O.make_layer_inputs(1, h, inter, e, seed=0)
    t = 96 + 32 * rank
    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g)
    ow, oids = O.softmax_topk(logits, k, True)
    sl = slice(rank * nle, (rank + 1) * nle)
    local = [w13[sl].to(dev), w13s[sl].to(dev), w2[sl].to(dev), w2s[sl].to(dev)]
    ref = O.moe_layer(x, ow, oids, w13, w13s, w2, w2s, top_k=k)
    return x.to(dev), ow.to(dev), oids.to(dev), local, ref


def _worker_async_api(rank, world, port, ret):
    """The split API of both layer classes (dlblas/layers/moe/ep_moe.py:100-152, 301-347 of the reference):
    dispatch_async -> wait -> fusedmoe_forward -> combine_async -> wait gives the bits of forward()."""
    import torch.distributed as dist

    from dlblas_b200 import _C
    from dlblas_b200.layers.moe.ep_moe import build_deepep_moe
    from oracle import moe_oracle as O
    dev = _setup(rank, world, port)
    try:
        e, k, h = 16, 4, 512
        x, w, ids, local, ref = _inputs(rank, world, dev, e, k, h)
        os.environ["DLBLAS_EP_BACKEND"] = "nccl"
        normal = build_deepep_moe(False, world, dist.group.WORLD, e, h, 128, k, torch.bfloat16)
        whole = normal.forward(x, w, ids, *local)
        start = normal.capture()
        recv_x, recv_idx, recv_w, per_expert, handle, ev = normal.dispatch_async(x, ids, w, e, previous_event=start,
                                                                               async_finish=True)
        normal.wait(ev)
        state = {"recv_hidden_states": recv_x, "recv_topk_idx": recv_idx, "recv_topk_weights": recv_w,
                 "recv_tokens_per_expert": per_expert}
        out_states = normal.fusedmoe_forward(state, *local)
        out, ev2 = normal.combine_async(out_states, handle, previous_event=normal.capture(), async_finish=True)
        normal.wait(ev2)
        assert normal.release() is True
        _C.check_status(dev)
        assert torch.equal(out.view_as(whole), whole), "FusedMoENormal: split API differs from forward"
        assert O.rel_frobenius(out.view_as(whole).cpu(), ref) < 2e-2
        # the already quantised input form of dispatch_async
        xq = normal.per_token_group_quant_fp8(x)
        r2 = normal.dispatch_async(xq, ids, w, e)
        normal.wait(r2[5])
        assert torch.equal(r2[0][0].view(torch.uint8), recv_x[0].view(torch.uint8)) and torch.equal(r2[1], recv_idx)

        outs = {}
        for ll_backend in ("nccl", "p2p"):
            os.environ["DLBLAS_EP_BACKEND"] = ll_backend
            low = build_deepep_moe(True, world, dist.group.WORLD, e, h, 128, k, torch.bfloat16)
            outs[ll_backend] = low.forward(x, w, ids, *local)
            outs[ll_backend] = low.forward(x, w, ids, *local)        # a second step reuses the symmetric buffers
        _C.check_status(dev)
        assert torch.equal(outs["nccl"], outs["p2p"]), "the two low-latency exchanges give different bits"
        whole = outs["p2p"]
        packed, masked_m, handle, ev, hook = low.dispatch_async(x, ids, e, True, True)
        low.wait(ev)
        hook()
        state = {"recv_hidden_states": packed, "recv_expert_count": masked_m, "raw_hidden_shape": x.shape,
                 "topk_idx": ids}
        out_states = low.fusedmoe_forward(state, *local)
        out, ev2, hook2 = low.combine_async(out_states, ids, w, handle, True)
        low.wait(ev2)
        hook2()
        _C.check_status(dev)
        assert torch.equal(out, whole), "FusedMoELowLatency: split API differs from forward"
        assert O.rel_frobenius(out.cpu(), ref) < 2e-2
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def _worker_barrier_timeout(rank, world, port, ret):
    """A rank that misses a barrier costs its peers one bounded wait and an exception on the host, and the
    group carries on afterwards.  The failure is made on the host (rank 1 simply does not call the barrier);
    nothing on a GPU faults, traps or spins without a limit."""
    import time

    import torch.distributed as dist

    from dlblas_b200 import _C
    from dlblas_b200.layers.moe.ep_moe import build_deepep_moe
    from dlblas_b200.layers.moe.token_dispatcher import TokenDispatcherP2P
    from oracle import moe_oracle as O
    dev = _setup(rank, world, port)
    try:
        e, k, h = 16, 4, 512
        os.environ["DLBLAS_EP_BARRIER_TIMEOUT_MS"] = "300"
        d = TokenDispatcherP2P(dist.group.WORLD, e, e // world, h, torch.bfloat16, max_tokens_per_rank=64, max_top_k=k)
        for ch in (0, 1, 0):
            d.barrier(ch)
        _C.check_status(dev)                                  # everybody arrived: nothing to report
        if rank == 0:
            t0 = time.time()
            d.barrier(0)                                      # rank 1 never makes this call
            try:
                _C.check_status(dev)
                ret[rank] = "no time-out reported"
                return
            except RuntimeError as exc:
                assert "gave up" in str(exc)
            waited = time.time() - t0
            assert 0.25 < waited < 5.0, waited
        else:
            time.sleep(0.5)
        d.resync()
        d.barrier(0)
        d.barrier(1)
        _C.check_status(dev)
        # and the layer built on these barriers still runs
        os.environ["DLBLAS_EP_BARRIER_TIMEOUT_MS"] = "10000"
        os.environ["DLBLAS_EP_BACKEND"] = "p2p"
        os.environ["DLBLAS_EP_MAX_TOKENS"] = "256"
        x, w, ids, local, ref = _inputs(rank, world, dev, e, k, h)
        layer = build_deepep_moe(False, world, dist.group.WORLD, e, h, 128, k, torch.bfloat16)
        out = layer.forward(x, w, ids, *local)
        _C.check_status(dev)
        assert O.rel_frobenius(out.cpu(), ref) < 2e-2
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def _run(worker, world=2, timeout=300):
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert dict(ret) == {r: "ok" for r in range(world)}


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_layers_two_gpus():
    _run(_worker)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_split_api_matches_forward_two_gpus():
    _run(_worker_async_api)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_missed_barrier_times_out_and_group_recovers_two_gpus():
    _run(_worker_barrier_timeout)
