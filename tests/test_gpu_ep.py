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
        for backend, low_latency in (("p2p", False), ("p2p-chunked", False), ("nccl", False), ("nccl", True)):
            # two token chunks on two streams (ranks hold 96 and 128 tokens: chunks of 48 / 64)
            os.environ["DLBLAS_EP_MIN_CHUNK_ROWS"] = "32" if backend == "p2p-chunked" else "1024"
            os.environ["DLBLAS_EP_CHUNKS"] = "2" if backend == "p2p-chunked" else "1"
            # the chunked run also takes the unfused combine (sum kernel, then push) so that both stay covered
            os.environ["DLBLAS_EP_FUSED_COMBINE"] = "0" if backend == "p2p-chunked" else "1"
            backend = backend.split("-")[0]
            os.environ["DLBLAS_EP_BACKEND"] = backend
            layer = build_deepep_moe(low_latency, world, dist.group.WORLD, e, h, 128, k, torch.bfloat16)
            assert (getattr(layer, "p2p_dispatcher", None) is not None) == (backend == "p2p")
            if backend == "p2p":
                assert len(layer.p2p_chunks) == (2 if os.environ["DLBLAS_EP_MIN_CHUNK_ROWS"] == "32" else 1)
            for _ in range(3):                      # repeated steps reuse the symmetric buffers
                out = layer.forward(x.to(dev), ow.to(dev), oids.to(dev), *local)
            _C.check_status(dev)
            err = O.rel_frobenius(out.cpu(), ref)
            assert out.shape == (t, h) and err < 2e-2, (backend, low_latency, err)
            # slots without an expert (id -1) are dropped by every exchange
            out_u = layer.forward(x.to(dev), ow.to(dev), ids_u.to(dev), *local)
            _C.check_status(dev)
            err_u = O.rel_frobenius(out_u.cpu(), ref_u)
            assert err_u < 2e-2, (backend, low_latency, "unrouted slots", err_u)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_layers_two_gpus():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert dict(ret) == {0: "ok", 1: "ok"}
