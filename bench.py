"""Benchmark of the FP8 MoE expert path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--tokens T]

Workload ("step" = one MoE layer forward over one batch of synthetic tokens): the
DeepSeek-V3-shaped prefill layer of the benchmark set — 8192 tokens per GPU, hidden 7168,
expert intermediate 2048, 256 routed experts top-8 with grouped routing (8 groups, 4 kept,
sigmoid scores + N(0, 0.01^2) bias), one shared expert, FP8 e4m3 weights with 128x128 block
scales, bf16 in/out.  With N > 1 GPUs the layer runs expert-parallel (256 / N experts per rank,
8192 tokens per rank: weak scaling) with the NCCL dispatch / combine of this package.

One JSON line is printed by rank 0.  `value` = tokens/s with inputs resident in HBM, `e2e` = the
same through host buffers (pinned host -> device copy of the step's inputs and device -> host
read of the result inside the timed region).  `--impl reference` times the CPU restatement of
the reference path (oracle/) on the host cores on a bounded sample of the same workload.
"""
import argparse
import json
import os

# torchrun exports OMP_NUM_THREADS=1 to every rank; the CPU baseline leg (rank 0 only) should use the host's cores
if os.environ.get("LOCAL_RANK") is not None and os.environ.get("OMP_NUM_THREADS") == "1":
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

T_PER_GPU, H, INTER, E, TOPK, GROUPS, TOPK_GROUP = 8192, 7168, 2048, 256, 8, 8, 4
FP8 = torch.float8_e4m3fn
METRIC = "moe_layer_tokens_per_s"
WORKLOAD = "deepseek_v3_moe_prefill"


def layer_flops(tokens: int) -> float:
    return 6.0 * tokens * TOPK * H * INTER + 6.0 * tokens * H * INTER     # routed + shared expert


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------------
# synthetic inputs
# --------------------------------------------------------------------------------------------
def quantize_blocks_gpu(w: torch.Tensor):
    e, n, k = w.shape
    blk = w.view(e, n // 128, 128, k // 128, 128)
    s = blk.abs().amax(dim=(2, 4), keepdim=True) / 448.0
    q = (blk / s).clamp_(-448.0, 448.0).view(e, n, k).to(FP8)
    return q, s.view(e, n // 128, k // 128).float()


def make_weights(num_experts: int, seed: int, dev, chunk: int = 8):
    """Random-init expert weights ~ N(0, 0.02^2), quantised per 128x128 block (generated on the
    device in chunks: the full fp32 tensors would not fit in host memory)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    w13 = torch.empty(num_experts, 2 * INTER, H, dtype=FP8, device=dev)
    w13s = torch.empty(num_experts, 2 * INTER // 128, H // 128, dtype=torch.float32, device=dev)
    w2 = torch.empty(num_experts, H, INTER, dtype=FP8, device=dev)
    w2s = torch.empty(num_experts, H // 128, INTER // 128, dtype=torch.float32, device=dev)
    for e0 in range(0, num_experts, chunk):
        n = min(chunk, num_experts - e0)
        a = torch.randn(n, 2 * INTER, H, generator=g, device=dev) * 0.02
        w13[e0:e0 + n], w13s[e0:e0 + n] = quantize_blocks_gpu(a)
        b = torch.randn(n, H, INTER, generator=g, device=dev) * 0.02
        w2[e0:e0 + n], w2s[e0:e0 + n] = quantize_blocks_gpu(b)
        del a, b
    return w13, w13s, w2, w2s


def make_tokens(tokens: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(tokens, E, generator=g)
    bias = torch.randn(E, generator=torch.Generator().manual_seed(1234)) * 0.01
    return x, logits, bias


def measured_traffic(kernel: str, experts: int):
    """DRAM bytes per launch of `kernel` from the tracked table of ncu captures (dlblas_b200/ncu_traffic.json):
    dram__bytes_read.sum + dram__bytes_write.sum of a small capture, scaled by the number of experts (the
    weights dominate and every expert is streamed once).  An entry is used only while the kernel's source file
    still has the hash it was captured with; otherwise the field is null rather than stale."""
    import hashlib
    path = os.path.join(ROOT, "dlblas_b200", "ncu_traffic.json")
    if not os.path.exists(path):
        return None, "no capture on record"
    ent = json.load(open(path)).get(kernel)
    if ent is None:
        return None, "no capture on record"
    src = os.path.join(ROOT, ent["source"])
    digest = hashlib.sha256(open(src, "rb").read()).hexdigest()[:16]
    if digest != ent["source_sha256_16"]:
        return None, f"the capture on record predates the current {ent['source']}"
    return ent["dram_bytes_per_launch"] * experts / ent["experts"], ent["note"]


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples `nvidia-smi` every 50 ms in the background; stop(t0, t1) keeps the samples whose
    timestamp falls inside the timed region [t0, t1] (wall clock)."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, t0: float, t1: float):
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        for line in open(self.path):
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), float(f[2]), f[5:9]))
            except ValueError:
                continue
        os.unlink(self.path)
        inside = [r for r in rows if t0 - 0.05 <= r[0] <= t1 + 0.05] or rows[-3:]
        reasons = set()
        for r in inside:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if inside:
            sm = sorted(r[1] for r in inside)
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(r[2] for r in inside), reasons=sorted(reasons),
                       samples=len(inside))
        return out


# --------------------------------------------------------------------------------------------
# reference arm: CPU restatement on the host cores
# --------------------------------------------------------------------------------------------
def cpu_sample(rows, w_cpu, x, logits, bias, remap=None):
    """One pass of the oracle over the tokens `rows` (an int = the first so many tokens, or an index tensor) of
    the workload; returns (seconds, output).  `remap` renumbers global expert ids into the positions of a
    reduced weight list (only the experts the sample hits)."""
    from oracle import moe_oracle as O
    w13, w13s, w2, w2s, sw13, sw13s, sw2, sw2s = w_cpu
    if isinstance(rows, int):
        rows = torch.arange(rows)
    xs = x[rows]
    t0 = time.perf_counter()
    # routing is decided on the whole batch's logits row by row, so a row's choice does not depend on the sample
    w, ids = O.biased_grouped_topk(logits[rows], bias, TOPK, True, GROUPS, TOPK_GROUP)
    ids = ids.long()
    if remap is not None:
        ids = remap[ids]
    out = O.moe_layer(xs, w, ids, w13, w13s, w2, w2s, top_k=TOPK)
    out = out + O.dense_swiglu_mlp(xs, sw13, sw13s, sw2, sw2s)
    return time.perf_counter() - t0, out


def cpu_weights(seed=0, distinct=8):
    """e4m3 weights of all 256 routed experts + the shared expert on the host.  Generating 11 GB of
    random weights on the CPU would take minutes, so `distinct` experts are drawn and repeated
    (expert e uses draw e % distinct); the cost of the CPU path does not depend on the values."""
    from oracle import moe_oracle as O
    g = torch.Generator().manual_seed(seed)
    w13, w13s = O.quantize_weight_blocks(torch.randn(distinct, 2 * INTER, H, generator=g) * 0.02)
    w2, w2s = O.quantize_weight_blocks(torch.randn(distinct, H, INTER, generator=g) * 0.02)
    sw13, sw13s = O.quantize_weight_blocks(torch.randn(1, 2 * INTER, H, generator=g) * 0.02)
    sw2, sw2s = O.quantize_weight_blocks(torch.randn(1, H, INTER, generator=g) * 0.02)
    idx = torch.arange(E) % distinct
    return [w13.view(torch.uint8)[idx].view(FP8), w13s[idx], w2.view(torch.uint8)[idx].view(FP8), w2s[idx],
            sw13[0], sw13s[0], sw2[0], sw2s[0]]


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, logits, bias = make_tokens(max(args.cpu_tokens, 8), 100)
    w_cpu = cpu_weights(0)
    # size the per-step sample so that warm-up + timed steps stay near two minutes of CPU work
    t8, _ = cpu_sample(8, w_cpu, x, logits, bias)
    budget = 120.0 / max(args.warmup + args.steps, 1)
    sample = max(1, min(args.cpu_tokens, int(budget / (t8 / 8.0))))
    times = []
    for i in range(args.warmup + args.steps):
        dt, _ = cpu_sample(sample, w_cpu, x, logits, bias)
        if i >= args.warmup:
            times.append(dt)
    total = sum(times)
    tps = sample * len(times) / total
    line = {
        "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic", "impl": "reference",
        "config": {"workload": WORKLOAD, "tokens_per_gpu": T_PER_GPU, "hidden": H, "intermediate": INTER,
                   "experts": E, "top_k": TOPK, "shared_experts": 1},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{sample} tokens of the workload per step through oracle/moe_oracle.py "
                                   f"(torch CPU restatement of the reference path)"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# B200 arm
# --------------------------------------------------------------------------------------------
class Layer:
    """The benchmarked layer on one rank: routing + routed experts + shared expert."""

    def __init__(self, world: int, rank: int, dev, group):
        from dlblas_b200.layers.moe.ep_moe import FusedMoENormal
        self.world, self.rank, self.dev = world, rank, dev
        self.e_local = E // world
        w13, w13s, w2, w2s = make_weights(self.e_local + 1, 1000 + rank, dev)    # last one = shared expert
        self.weights = (w13, w13s, w2, w2s)
        self.ep = None
        if world > 1:
            self.ep = FusedMoENormal(world, group, E, H, top_k=TOPK, out_dtype=torch.bfloat16)
            self.side = torch.cuda.Stream(device=dev)
        self.shared_col_ids = torch.full((T_PER_GPU, 1), self.e_local, dtype=torch.int64, device=dev)
        self.shared_col_w = torch.ones(T_PER_GPU, 1, dtype=torch.float32, device=dev)

    def step(self, x, logits, bias):
        from dlblas_b200 import _C, ops
        from dlblas_b200.kernels.fp8 import per_token_group_quant_fp8
        from dlblas_b200.layers.moe.kernels.blocked_fp8_fused_moe import moe_expert_forward
        w13, w13s, w2, w2s = self.weights
        t = x.shape[0]
        w, ids = ops.route_grouped_topk(logits, bias, TOPK, True, GROUPS, TOPK_GROUP)
        if self.world == 1:
            # the shared expert rides along as expert number E with weight 1 for every token
            ids9 = torch.cat([ids.long(), self.shared_col_ids[:t]], dim=1)
            w9 = torch.cat([w, self.shared_col_w[:t]], dim=1)
            return moe_expert_forward(x, None, None, w13, w13s, w2, w2s, w9, ids9, TOPK + 1, torch.bfloat16, 0,
                                      self.e_local + 1)
        nl = self.e_local
        box = {}

        # The shared expert works on local tokens only: its w13 half is enqueued between this rank's dispatch pushes
        # and the wait for the peers' tokens, its w2 half between the combine pushes and the wait for the peers'
        # results, so it runs while rows are in flight over NVLink instead of beside the routed GEMMs.
        def shared_up():
            xq, xs = ops.quant_fp8(x, 128, _C.QUANT_RECIP_MUL, 0.0)
            c1 = ops.fp8_gemm(xq, w13[nl], xs, w13s[nl], torch.bfloat16)
            box["h"] = ops.silu_mul_quant(c1, _C.QUANT_RECIP_MUL)

        def shared_down():
            hq, hs = box["h"]
            box["out"] = ops.fp8_gemm(hq, w2[nl], hs, w2s[nl], torch.bfloat16)

        # (measured at N = 4: 5.46 ms per step this way against 5.41 ms with the shared expert on a side stream,
        # so the side stream stays the default; DLBLAS_BENCH_OVERLAP=1 selects the hooks)
        if self.ep.p2p_dispatcher is not None and os.environ.get("DLBLAS_BENCH_OVERLAP", "0") == "1":
            self.ep.during_dispatch, self.ep.during_combine = shared_up, shared_down
            routed = self.ep.forward(x, w, ids.long(), w13[:nl], w13s[:nl], w2[:nl], w2s[:nl])
            return routed.add_(box["out"])
        cur = torch.cuda.current_stream()
        self.side.wait_stream(cur)
        with torch.cuda.stream(self.side):           # shared expert on the local tokens, beside the exchange
            shared_up()
            shared_down()
        self.ep.during_dispatch = self.ep.during_combine = None
        routed = self.ep.forward(x, w, ids.long(), w13[:nl], w13s[:nl], w2[:nl], w2s[:nl])
        cur.wait_stream(self.side)
        return routed.add_(box["out"])


def time_steps(fn, steps, dev, before_end=None):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    start.record()
    for _ in range(steps):
        fn()
    if before_end is not None:
        before_end()                 # e.g. make the timing stream wait for side streams
    end.record()
    torch.cuda.synchronize(dev)
    return start.elapsed_time(end)


def run_b200(args):
    import torch.distributed as dist

    from dlblas_b200 import _C, ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    tokens = args.tokens
    layer = Layer(world, rank, dev, group)
    x_h, logits_h, bias_h = make_tokens(tokens, 100 + rank)
    x_pin, logits_pin = x_h.pin_memory(), logits_h.pin_memory()
    out_pin = torch.empty(tokens, H, dtype=torch.bfloat16).pin_memory()
    x_d, logits_d, bias_d = x_h.to(dev), logits_h.to(dev), bias_h.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def step_resident():
        return layer.step(x_d, logits_d, bias_d)

    # End-to-end step: every step copies its inputs from pinned host memory and its result back.
    # The copies run on their own streams over double-buffered device inputs, so the upload of
    # step i + 1 and the download of step i - 1 overlap the kernels of step i (PCIe is full duplex).
    h2d_stream, d2h_stream = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    in_bufs = [(torch.empty_like(x_d), torch.empty_like(logits_d)) for _ in range(2)]
    out_pins = [out_pin, torch.empty_like(out_pin).pin_memory()]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    e2e_state = {"i": 0}

    def step_e2e():
        i = e2e_state["i"]
        e2e_state["i"] = i + 1
        b = i & 1
        cur = torch.cuda.current_stream(dev)
        xb, lb = in_bufs[b]
        with torch.cuda.stream(h2d_stream):
            if i >= 2:
                h2d_stream.wait_event(in_free[b])         # step i - 2 has consumed this buffer
            xb.copy_(x_pin, non_blocking=True)
            lb.copy_(logits_pin, non_blocking=True)
            in_ready[b].record(h2d_stream)
        cur.wait_event(in_ready[b])
        out = layer.step(xb, lb, bias_d)
        in_free[b].record(cur)
        done = torch.cuda.Event()
        done.record(cur)
        with torch.cuda.stream(d2h_stream):
            d2h_stream.wait_event(done)
            if i >= 2:
                d2h_stream.wait_event(out_done[b])        # keep the pinned buffer's copies in order
            out_pins[b].copy_(out, non_blocking=True)
            out.record_stream(d2h_stream)
            out_done[b].record(d2h_stream)

    def drain_e2e():
        cur = torch.cuda.current_stream(dev)
        cur.wait_stream(d2h_stream)
        cur.wait_stream(h2d_stream)

    for _ in range(max(args.warmup, 3)):
        step_resident()
    _C.check_status(dev)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(3):
        step_resident()              # every rank (the step has collectives); the sampler comes up meanwhile
    time.sleep(0.3)
    barrier()
    _C.launch_count(reset=True)
    wall0 = time.time()
    ms = time_steps(step_resident, args.steps, dev)
    wall1 = time.time()
    launches = _C.launch_count(reset=True)
    barrier()
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    for _ in range(2):
        step_e2e()
    drain_e2e()
    barrier()
    ms_e2e = time_steps(step_e2e, args.steps, dev, before_end=drain_e2e)
    barrier()
    _C.check_status(dev)
    if world > 1:
        tmax = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(tmax[0]), float(tmax[1])

    # ---- end-to-end ceiling: the step's host copies alone (same pinned buffers, same streams, no kernels) ----
    def copies_only():
        with torch.cuda.stream(h2d_stream):
            in_bufs[0][0].copy_(x_pin, non_blocking=True)
            in_bufs[0][1].copy_(logits_pin, non_blocking=True)
        with torch.cuda.stream(d2h_stream):
            out_pins[0].copy_(in_bufs[1][0], non_blocking=True)

    for _ in range(2):
        copies_only()
    drain_e2e()
    barrier()
    ms_copy = time_steps(copies_only, max(args.steps, 5), dev, before_end=drain_e2e) / max(args.steps, 5)
    barrier()
    if world > 1:
        tc = torch.tensor([ms_copy], dtype=torch.float64, device=dev)
        dist.all_reduce(tc, op=dist.ReduceOp.MAX)
        ms_copy = float(tc[0])

    # ---- dominant kernel: the w13 grouped GEMM with the fused silu*up + quantisation epilogue, on the rows this
    # rank really works on (at N > 1: the receive buffer after a real dispatch, which every rank takes part in) ----
    peaks = load_peaks()
    e_loc = layer.e_local + (1 if world == 1 else 0)
    w13, w13s, w2, w2s = layer.weights
    w_r, ids_r = ops.route_grouped_topk(logits_d, bias_d, TOPK, True, GROUPS, TOPK_GROUP)
    if world == 1:
        ids_k = torch.cat([ids_r.long(), layer.shared_col_ids[:tokens]], dim=1)
        s_rows = tokens * (TOPK + 1)
        sidx, st, en, pos = ops.sort_by_expert(ids_k, e_loc, want_pos=True)
        a1, a1s = ops.quant_fp8(x_d, 128, _C.QUANT_RECIP_MUL, 0.0, False, pos, TOPK + 1, s_rows)
    else:
        disp = layer.ep.p2p_dispatcher
        assert disp is not None, "the roofline leg times the peer-to-peer exchange's receive buffer"
        (rq, rs), ids_k, _rw = disp.dispatch_from_hidden(x_d, ids_r.long(), w_r, 128)
        s_rows = ids_k.numel()
        sidx, st, en, pos = ops.sort_by_expert(ids_k, e_loc, want_pos=True)
        a1, a1s = ops.permute_rows(rq, rs.contiguous(), pos, TOPK, s_rows)
    mt = ops.max_tiles_for(s_rows, e_loc)
    tiles = ops.build_tiles(st, en, 0, e_loc, mt)
    hq = torch.empty(s_rows, INTER, dtype=FP8, device=dev)
    hs = torch.empty(s_rows, INTER // 128, dtype=torch.float32, device=dev)
    routed_rows = int((ids_k >= 0).sum())
    tile_rows_issued = int(tiles[0]) * 128

    def gemm1():
        ops.grouped_gemm(a1, a1s, w13[:e_loc], w13s[:e_loc], tiles, mt, _C.EPI_SWIGLU_QUANT, hq, q_scale=hs,
                         round_dtype=torch.bfloat16)

    for _ in range(3):
        gemm1()
    n_roof = max(args.steps, 5)
    kms = time_steps(gemm1, n_roof, dev) / n_roof
    _C.check_status(dev)
    roof = None
    cpu_base = None
    parity = None
    if rank == 0:
        flops = 2.0 * routed_rows * (2 * INTER) * H
        achieved = flops / (kms * 1e-3) / 1e12
        # a long back-to-back loop of this kernel runs under the power cap like the step itself:
        # compare it with the sustained figure; a short loop with the burst figure
        sustained = kms * n_roof > 1000.0
        bf16_peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
        fp8_peak = 2.0 * bf16_peak
        traffic, traffic_note = measured_traffic("gemm_fp8_w13_grouped", e_loc)
        roof = {"kernel": "gemm_fp8 w13 grouped GEMM with the silu*up + quantise epilogue", "bound": "tensor",
                "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak,
                "traffic": traffic, "ms_per_launch": kms, "launches_timed": n_roof,
                "rows": routed_rows, "tile_fill": routed_rows / max(tile_rows_issued, 1),
                "rows_note": "the rows of the step itself" if world == 1 else
                             "this rank's receive buffer after a real dispatch of the step's tokens",
                "peak_note": f"2 x {peaks['source']} cuBLAS bf16 {'sustained' if sustained else 'burst'} figure "
                             f"({bf16_peak} TFLOP/s): e4m3 tensor rate is twice bf16 on B200; no FP8 figure is "
                             f"measured on this pool",
                "traffic_note": traffic_note}

    # ---- parity of the timed configuration: rows of a full-batch step against the CPU oracle ----
    if not args.no_cpu:
        from oracle import moe_oracle as O
        full_out = layer.step(x_d, logits_d, bias_d)           # every rank: the step has collectives
        _C.check_status(dev)
        if rank == 0:
            torch.set_num_threads(os.cpu_count() or 1)
            n_s = max(args.cpu_tokens, 1)
            rows = torch.unique(torch.linspace(0, tokens - 1, n_s).long())
            _, ids_o = O.biased_grouped_topk(logits_h[rows], bias_h, TOPK, True, GROUPS, TOPK_GROUP)
            assert torch.equal(ids_o, ids_r.cpu()[rows]), "routing ids of the sampled rows differ from the oracle"
            hit = torch.unique(ids_o.long())
            remap = torch.full((E,), -1, dtype=torch.int64)
            remap[hit] = torch.arange(hit.numel())
            nl = layer.e_local
            parts = {k_: [] for k_ in range(4)}
            for r in range(world):                              # weights of rank r: seeded, regenerated here
                mine = hit[(hit >= r * nl) & (hit < (r + 1) * nl)] - r * nl
                if mine.numel() == 0:
                    continue
                wr = layer.weights if r == rank else make_weights(nl + 1, 1000 + r, dev)
                for k_ in range(4):
                    parts[k_].append(wr[k_][mine.to(dev)].cpu())
                del wr
            w_cpu = [torch.cat(parts[k_]) for k_ in range(4)] + [w13[nl].cpu(), w13s[nl].cpu(), w2[nl].cpu(),
                                                                 w2s[nl].cpu()]
            dt, ref_out = cpu_sample(rows, w_cpu, x_h, logits_h, bias_h, remap)
            err = O.rel_frobenius(full_out[rows.to(dev)].cpu(), ref_out)
            sample = (f"{rows.numel()} rows spread over the step's batch of {tokens} tokens, taken from the output "
                      f"of the full-batch step, all {hit.numel()} experts they hit, through oracle/moe_oracle.py")
            cpu_base = {"value": rows.numel() / dt, "unit": "tokens/s", "cores": torch.get_num_threads(),
                        "kind": "port", "sample": sample, "rel_frobenius_vs_gpu": err}
            parity = {"rel_frobenius_vs_oracle": err, "rows": int(rows.numel()), "routing_ids_equal": True,
                      "tolerance": 2e-2}
    if world > 1:
        dist.barrier()
    if rank == 0:
        total_tokens = tokens * world
        tps = total_tokens * args.steps / (ms * 1e-3)
        tps_e2e = total_tokens * args.steps / (ms_e2e * 1e-3)
        tflops = layer_flops(total_tokens) * args.steps / (ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu": tokens, "hidden": H, "intermediate": INTER,
                       "experts": E, "top_k": TOPK, "shared_experts": 1, "routing": "grouped 8/4 sigmoid+bias",
                       "parallelism": f"ep{world}",
                       "l2": "inputs larger than L2: every step streams this rank's expert weights "
                             f"({(layer.e_local + 1) * 3 * H * INTER / 1e9:.2f} GB) from HBM"},
            "tflops": tflops,
            "fp8_peak_frac": tflops / (2.0 * load_peaks()["bf16_tflops_sustained" if ms > 1000.0 else "bf16_tflops"]
                                       * world),
            "fp8_peak_note": "layer TFLOP/s over 2 x the measured bf16 figure (sustained for a timed region longer "
                             "than 1 s, else burst)",
            "e2e": {"value": tps_e2e, "unit": "tokens/s", "h2d_bytes_per_step": tokens * H * 2 + tokens * E * 4,
                    "d2h_bytes_per_step": tokens * H * 2, "ms_per_step": ms_e2e / args.steps,
                    "host_copy_ceiling_ms": ms_copy,
                    "host_copy_note": "the same copies (pinned host <-> device, both directions at once, every rank "
                                      "at the same time) with no kernel running: the floor of an end-to-end step on "
                                      "this box"},
            "gpu_launches": launches, "clocks": clocks, "roofline": roof,
        }
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
            line["parity"] = parity
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_profile(args):
    """Small stand-alone case of one kernel for `ncu` (a few GB on the device, a handful of
    launches): `--profile gemm1|gemm2|dense` with `--tokens` and `--experts` scaled down so that
    rows per expert (tokens * 8 / experts) stay at the full workload's 256."""
    from dlblas_b200 import _C, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    e, t = args.experts, args.tokens
    g = torch.Generator().manual_seed(7)
    if args.profile == "dense":
        m, n, k = t, 2 * INTER, H
        a = (torch.randn(m, k, generator=g)).to(FP8).to(dev)
        b = (torch.randn(n, k, generator=g)).to(FP8).to(dev)
        a_s = torch.rand(m, k // 128, generator=g).to(dev)
        b_s = torch.rand(n // 128, k // 128, generator=g).to(dev)
        for _ in range(args.steps):
            ops.fp8_gemm(a, b, a_s, b_s, torch.bfloat16)
        torch.cuda.synchronize()
        _C.check_status(dev)
        return
    if args.profile == "gemm16":
        # 16-bit grouped GEMM (whole K accumulated in TMEM, pairs of CTAs): `experts` groups of `tokens` rows in all
        from dlblas_b200.kernels.grouped_gemm.BF16 import m_grouped_gemm
        gd = torch.Generator(device=dev).manual_seed(7)
        a = torch.randn(t, H, generator=gd, device=dev, dtype=torch.bfloat16)
        b = torch.randn(e, 2 * INTER, H, generator=gd, device=dev, dtype=torch.bfloat16) * 0.05
        sizes = torch.full((e,), t // e, device=dev, dtype=torch.int64)
        for _ in range(args.steps):
            m_grouped_gemm(a, b, sizes, trans_b=True)
        torch.cuda.synchronize()
        _C.check_status(dev)
        return
    if args.profile == "kgrouped":
        # k_grouped_gemm at the shapes of the reference's benchmark (benchmarks/grouped_gemm/BF16/k_grouped_gemm.py:
        # bf16, (m, n) in four pairs, random group sizes averaging 5120 rows): `experts` groups, CUDA events around
        # whole calls, the torch loop of one matmul per group beside it.  `--steps 2` is the case for ncu.
        import random
        from dlblas_b200.kernels.grouped_gemm.BF16 import k_grouped_gemm
        random.seed(0)
        raw = [random.randint(0, 2 * 5120) for _ in range(e)]
        sizes = torch.tensor(raw, dtype=torch.int64, device=dev)
        k_total = sum(raw)
        starts = [0]
        for r in raw:
            starts.append(starts[-1] + r)
        shapes = ((3072, 4096),) if args.steps <= 2 else ((1536, 2048), (2048, 768), (3072, 4096), (4096, 1536))
        print(f"| m | n | groups | K total | ms | TFLOP/s | of measured bf16 burst | torch per-group loop ms |\n|---|---|---|---|---|---|---|---|")
        for (m, n) in shapes:
            gd = torch.Generator(device=dev).manual_seed(7)
            a = torch.randn(k_total, m, generator=gd, device=dev, dtype=torch.bfloat16)
            b = torch.randn(k_total, n, generator=gd, device=dev, dtype=torch.bfloat16)
            out = None
            for _ in range(2):
                out = k_grouped_gemm(a, b, sizes)
            _C.check_status(dev)
            if args.steps <= 2:
                continue
            ref = torch.empty_like(out)

            def loop():
                for i in range(e):
                    torch.matmul(a[starts[i]:starts[i + 1]].t(), b[starts[i]:starts[i + 1]], out=ref[i])
            ms = _time_kernel(lambda: k_grouped_gemm(a, b, sizes), dev, iters=args.steps)
            ms_loop = _time_kernel(loop, dev, iters=max(3, args.steps // 4))
            assert torch.equal(out, ref), "k_grouped_gemm differs from the per-group matmul"
            tf = 2.0 * k_total * m * n / ms / 1e9
            print(f"| {m} | {n} | {e} | {k_total} | {ms:.3f} | {tf:.0f} | {tf / load_peaks()['bf16_tflops']:.2f} | {ms_loop:.3f} |",
                  flush=True)
            del a, b, out, ref
        torch.cuda.synchronize()
        return
    w13, w13s, w2, w2s = make_weights(e, 1, dev)
    x = torch.randn(t, H, generator=g).to(torch.bfloat16).to(dev)
    ids = torch.stack([torch.randperm(e, generator=g)[:TOPK] for _ in range(t)]).to(dev)
    wts = torch.rand(t, TOPK, generator=g).to(dev)
    s_rows = t * TOPK
    sidx, st, en, pos = ops.sort_by_expert(ids, e, want_pos=True)
    mt = ops.max_tiles_for(s_rows, e)
    tiles = ops.build_tiles(st, en, 0, e, mt)
    a1, a1s = ops.quant_fp8(x, 128, _C.QUANT_RECIP_MUL, 0.0, False, pos, TOPK, s_rows)
    hq = torch.empty(s_rows, INTER, dtype=FP8, device=dev)
    hs = torch.empty(s_rows, INTER // 128, dtype=torch.float32, device=dev)
    y = torch.empty(s_rows, H, dtype=torch.bfloat16, device=dev)
    for _ in range(args.steps):
        if args.profile == "gemm1":
            ops.grouped_gemm(a1, a1s, w13, w13s, tiles, mt, _C.EPI_SWIGLU_QUANT, hq, q_scale=hs,
                             round_dtype=torch.bfloat16)
        else:
            if _ == 0:
                ops.grouped_gemm(a1, a1s, w13, w13s, tiles, mt, _C.EPI_SWIGLU_QUANT, hq, q_scale=hs,
                                 round_dtype=torch.bfloat16)
            ops.grouped_gemm(hq, hs, w2, w2s, tiles, mt, _C.EPI_SCATTER_WEIGHT, y, sorted_idx=sidx, weights=wts)
    torch.cuda.synchronize()
    _C.check_status(dev)


def _time_kernel(fn, dev, iters=20, flush=None):
    """Average CUDA-event time of one launch in ms; `flush` (a buffer larger than L2) is rewritten between
    launches so that every launch starts from a cold L2."""
    for _ in range(3):
        fn()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize(dev)
        total += a.elapsed_time(b)
    return total / iters


def run_profile_bandwidth(args):
    """`--profile bandwidth`: every HBM-bound kernel of the step alone at the step's sizes, CUDA events around
    each launch, L2 flushed in between; prints a markdown table of algorithmic bytes, time, GB/s and the fraction
    of the measured copy bandwidth."""
    from dlblas_b200 import _C, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak = load_peaks()["hbm_gbs"]
    t, k = args.tokens, TOPK + 1
    x_h, logits_h, bias_h = make_tokens(t, 100)
    x, logits, bias = x_h.to(dev), logits_h.to(dev), bias_h.to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    w, ids = ops.route_grouped_topk(logits, bias, TOPK, True, GROUPS, TOPK_GROUP)
    ids9 = torch.cat([ids.long(), torch.full((t, 1), E, dtype=torch.int64, device=dev)], dim=1)
    s_rows = t * k
    sidx, st, en, pos = ops.sort_by_expert(ids9, E + 1, want_pos=True)
    y = torch.randn(s_rows, H, device=dev).to(torch.bfloat16)
    gu = torch.randn(s_rows // 4, 2 * INTER, device=dev).to(torch.bfloat16)
    rows = []

    def add(name, fn, nbytes):
        ms = _time_kernel(fn, dev, 20, flush)
        gbs = nbytes / ms / 1e6
        rows.append(f"| {name} | {nbytes / 1e6:.1f} | {ms * 1e3:.1f} | {gbs:.0f} | {gbs / peak:.2f} |")

    add("grouped_topk (8192 x 256 fp32 logits -> ids, weights)", lambda: ops.route_grouped_topk(
        logits, bias, TOPK, True, GROUPS, TOPK_GROUP), 4.0 * t * E + 8.0 * t * TOPK)
    add("sort_by_expert (73 728 slots, 257 experts; 4 kernels)", lambda: ops.sort_by_expert(
        ids9, E + 1, want_pos=True), 8.0 * s_rows * 2 + 12.0 * s_rows + 16.0 * (E + 1))
    add("quant_fp8, fan-out 9 (x bf16 -> a1 e4m3 + scales in expert order)", lambda: ops.quant_fp8(
        x, 128, _C.QUANT_RECIP_MUL, 0.0, False, pos, k, s_rows), 2.0 * t * H + k * t * H * (1 + 4 / 128))
    add("quant_fp8, no fan-out", lambda: ops.quant_fp8(x, 128, _C.QUANT_RECIP_MUL, 0.0),
        2.0 * t * H + t * H * (1 + 4 / 128))
    add("silu_mul_quant (18 432 x 4096 bf16 -> e4m3 + scales)", lambda: ops.silu_mul_quant(
        gu, _C.QUANT_RECIP_MUL, 0.0), 4.0 * gu.shape[0] * INTER + gu.shape[0] * INTER * (1 + 4 / 128))
    add("sum_topk (73 728 x 7168 bf16 -> 8192 x 7168)", lambda: ops.sum_topk(y, t, k, ids9, 0, E + 1),
        2.0 * s_rows * H + 2.0 * t * H)
    print(f"HBM copy bandwidth measured on this pool: {peak:.0f} GB/s\n")
    print("| kernel | algorithmic MB | us / launch | GB/s | of measured |\n|---|---|---|---|---|")
    print("\n".join(rows))


def run_profile_timeline(args):
    """`--profile timeline` (under torchrun for more than one GPU): the benchmarked step on `--tokens` tokens per rank
    under torch.profiler, CUDA activities only; rank 0 prints the kernels of the last of four profiled steps in launch
    order with their start (ms from the step's first kernel) and duration.  Times under the profiler run a few percent
    above the bench's; the table is for shares and for what runs alone."""
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    layer = Layer(world, rank, dev, group)
    x, logits, bias = [t.to(dev) for t in make_tokens(args.tokens, 100 + rank)]
    for _ in range(5):
        layer.step(x, logits, bias)
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    _print_step_timeline(lambda: layer.step(x, logits, bias), dev, rank, f"{world} GPU(s), {args.tokens} tokens per rank")
    if world > 1:
        dist.destroy_process_group()


def _print_step_timeline(step, dev, rank, label, steps=4):
    """Runs `step` `steps` times under torch.profiler (CUDA activities) and prints, on rank 0, the kernels of the last
    one in launch order."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            step()
        torch.cuda.synchronize(dev)
    if rank != 0:
        return
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    t_end = evs[-1].time_range.end
    span = (t_end - evs[0].time_range.start) / steps
    last = [e for e in evs if e.time_range.start >= t_end - span]
    t0 = last[0].time_range.start
    print("| start (ms) | duration (ms) | kernel |\n|---|---|---|")
    for e in last:
        print(f"| {(e.time_range.start - t0) / 1e3:.3f} | {(e.time_range.end - e.time_range.start) / 1e3:.3f} | "
              f"`{e.name[:100]}` |")
    print(f"\nstep under the profiler: {span / 1e3:.3f} ms, {label}")


def run_profile_sweep(args):
    """`--profile sweep`: the stand-alone block-scaled GEMM over the 12 shapes of the benchmark set, and the two
    grouped GEMMs of the Mixtral-shaped layer; CUDA events, L2 flushed between launches."""
    from dlblas_b200 import _C, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(3)
    print(f"divisor: 2 x {peaks['source']} cuBLAS bf16 burst figure = {fp8_peak:.0f} TFLOP/s\n")
    print("| M | N | K | us / launch | TFLOP/s | of 2 x bf16 burst |\n|---|---|---|---|---|---|")
    for m in (128, 1024, 4096, 8192):
        for n, k in ((24576, 1536), (7168, 2048), (4096, 7168)):
            a = torch.randn(m, k, generator=g, device=dev).to(FP8)
            b = torch.randn(n, k, generator=g, device=dev).to(FP8)
            a_s = torch.rand(m, k // 128, generator=g, device=dev)
            b_s = torch.rand(n // 128, k // 128, generator=g, device=dev)
            ms = _time_kernel(lambda: ops.fp8_gemm(a, b, a_s, b_s, torch.bfloat16), dev, 10, flush)
            tf = 2.0 * m * n * k / ms / 1e9
            print(f"| {m} | {n} | {k} | {ms * 1e3:.1f} | {tf:.0f} | {tf / fp8_peak:.2f} |")
    # Mixtral-shaped layer: 4096 tokens, top-2 of 8 experts, hidden 4096, intermediate 14336
    t, h, inter, e, k = 4096, 4096, 14336, 8, 2
    ws = []
    for shape in ((e, 2 * inter, h), (e, h, inter)):
        wq = torch.empty(shape, dtype=FP8, device=dev)
        wsc = torch.empty(shape[0], shape[1] // 128, shape[2] // 128, device=dev)
        for i in range(e):
            q, sc = quantize_blocks_gpu(torch.randn(1, shape[1], shape[2], generator=g, device=dev) * 0.02)
            wq[i], wsc[i] = q[0], sc[0]
        ws += [wq, wsc]
    x = torch.randn(t, h, generator=g, device=dev).to(torch.bfloat16)
    wt, ids = ops.route_softmax_topk(torch.randn(t, e, generator=g, device=dev), k, True)
    sidx, st, en, pos = ops.sort_by_expert(ids, e, want_pos=True)
    mt = ops.max_tiles_for(t * k, e)
    tiles = ops.build_tiles(st, en, 0, e, mt)
    a1, a1s = ops.quant_fp8(x, 128, _C.QUANT_RECIP_MUL, 0.0, False, pos, k, t * k)
    hq = torch.empty(t * k, inter, dtype=FP8, device=dev)
    hs = torch.empty(t * k, inter // 128, dtype=torch.float32, device=dev)
    y = torch.empty(t * k, h, dtype=torch.bfloat16, device=dev)
    ms1 = _time_kernel(lambda: ops.grouped_gemm(a1, a1s, ws[0], ws[1], tiles, mt, _C.EPI_SWIGLU_QUANT, hq, q_scale=hs,
                                                round_dtype=torch.bfloat16), dev, 10, flush)
    ms2 = _time_kernel(lambda: ops.grouped_gemm(hq, hs, ws[2], ws[3], tiles, mt, _C.EPI_SCATTER_WEIGHT, y,
                                                sorted_idx=sidx, weights=wt.flatten()), dev, 10, flush)
    f1, f2 = 2.0 * t * k * 2 * inter * h, 2.0 * t * k * inter * h
    print("\nMixtral-shaped layer (4096 tokens, 8 experts top-2, hidden 4096, intermediate 14336), grouped GEMMs:\n")
    print("| GEMM | us / launch | TFLOP/s | of 2 x bf16 burst |\n|---|---|---|---|")
    print(f"| w13 + silu*up + quantise | {ms1 * 1e3:.1f} | {f1 / ms1 / 1e9:.0f} | {f1 / ms1 / 1e9 / fp8_peak:.2f} |")
    print(f"| w2 + routed weight, scattered | {ms2 * 1e3:.1f} | {f2 / ms2 / 1e9:.0f} | {f2 / ms2 / 1e9 / fp8_peak:.2f} |")
    _C.check_status(dev)


def run_decode(args):
    """Optional second workload (not the headline line): the decode-shaped case of the benchmark set, 128
    tokens per GPU with Zipf-skewed routing (alpha 1.2) through the low-latency (masked layout) layer and the
    shared expert.  Prints per-step latency percentiles measured with one pair of CUDA events per step."""
    import torch.distributed as dist

    from dlblas_b200 import _C, ops
    from dlblas_b200.layers.moe.ep_moe import FusedMoELowLatency
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    tokens = 128
    nl = E // world
    w13, w13s, w2, w2s = make_weights(nl + 1, 1000 + rank, dev)
    layer = FusedMoELowLatency(world, group, E, H, layer_index=0)
    g = torch.Generator().manual_seed(200 + rank)
    x = torch.randn(tokens, H, generator=g).to(torch.bfloat16).to(dev)
    pop = torch.randperm(E, generator=torch.Generator().manual_seed(77)).float() + 1.0
    logits = (torch.randn(tokens, E, generator=g) + torch.log(pop ** -1.2 / (pop ** -1.2).sum())).to(dev)

    side = torch.cuda.Stream(dev)
    overlap_shared = os.environ.get("DLBLAS_BENCH_DECODE_OVERLAP", "1") == "1"

    def shared_expert():
        xq, xs = ops.quant_fp8(x, 128, _C.QUANT_RECIP_MUL, 0.0)
        c1 = ops.fp8_gemm(xq, w13[nl], xs, w13s[nl], torch.bfloat16)
        hq, hs = ops.silu_mul_quant(c1, _C.QUANT_RECIP_MUL)
        return ops.fp8_gemm(hq, w2[nl], hs, w2s[nl], torch.bfloat16)

    def step():
        # the shared expert's four small kernels run on a second stream beside the routed experts' weight streaming
        cur = torch.cuda.current_stream(dev)
        if overlap_shared:
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                shared = shared_expert()
        w, ids = ops.route_softmax_topk(logits, TOPK, True)
        routed = layer.forward(x, w, ids, w13[:nl], w13s[:nl], w2[:nl], w2s[:nl])
        if overlap_shared:
            cur.wait_stream(side)
        else:
            shared = shared_expert()
        return routed + shared

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize(dev)
    if args.profile == "timeline":                # `--workload decode --profile timeline`: the eager step, kernel by kernel
        if world > 1:
            dist.barrier()
        _print_step_timeline(step, dev, rank, f"{world} GPU(s), decode shape, eager launches")
        if world > 1:
            dist.destroy_process_group()
        return
    # The layer has no host round trip (one GPU: device-side plan; several ranks: peer-to-peer stores and the
    # extension's own barrier kernel), so the whole step (about 40 short kernels) replays as one CUDA graph on
    # every rank.  With DLBLAS_EP_BACKEND=nccl the all-to-all needs its split sizes on the host and the step runs
    # eagerly.
    run, graphed = step, False
    host_free = world == 1 or type(layer.token_dispatcher).__name__ == "TokenDispatcherLowLatencyP2P"
    if host_free:
        try:
            warm = torch.cuda.Stream(dev)
            warm.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(warm):
                step()
            torch.cuda.current_stream(dev).wait_stream(warm)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_out = step()                                # noqa: F841  (kept alive with the graph)
            run, graphed = graph.replay, True
        except Exception as exc:                                  # capture not possible: measure the eager step
            print(f"# CUDA graph capture failed ({type(exc).__name__}: {exc}); timing the eager step", file=sys.stderr)
            run, graphed = step, False
        torch.cuda.synchronize(dev)
        if world > 1:
            # every rank replays, or none does: the barriers inside the step need all ranks in the same mode
            flag = torch.tensor([1 if graphed else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag[0]) == 0:
                run, graphed = step, False
        for _ in range(3):
            run()
        torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in evs:
        a.record()
        run()
        b.record()
    torch.cuda.synchronize(dev)
    _C.check_status(dev)
    lat = torch.tensor([a.elapsed_time(b) for a, b in evs], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(lat, op=dist.ReduceOp.MAX)            # a step ends when its slowest rank ends
    lat = lat.cpu().sort().values
    # experts that received at least one row on this rank: their weights (and the shared expert's) are what a step
    # streams from HBM
    _, _, _, masked_m, _ = layer.token_dispatcher.dispatch(x, ops.route_softmax_topk(logits, TOPK, True)[1], None, E)
    if hasattr(layer.token_dispatcher, "barrier"):
        layer.token_dispatcher.barrier(1)          # the combine's barrier, so that all ranks stay in step
    e_hit = torch.tensor([float((masked_m > 0).sum())], device=dev)
    if world > 1:
        dist.all_reduce(e_hit, op=dist.ReduceOp.MAX)
    torch.cuda.synchronize(dev)
    _C.check_status(dev)
    if rank == 0:
        p50 = float(lat[len(lat) // 2])
        p99 = float(lat[min(len(lat) - 1, int(len(lat) * 0.99))])
        streamed = (float(e_hit[0]) + 1.0) * 3.0 * H * INTER      # e4m3 bytes of w13 + w2 per expert hit, + shared
        hbm = load_peaks()["hbm_gbs"]
        print(json.dumps({"metric": "moe_decode_layer_latency_ms", "value": p50, "unit": "ms", "p50_ms": p50, "p99_ms": p99,
                          "experts_hit_max_over_ranks": int(e_hit[0]), "weight_bytes_streamed": streamed,
                          "hbm_frac_of_measured": streamed / (p50 * 1e-3) / (hbm * 1e9),
                          "tokens_per_s": tokens * world / (p50 * 1e-3), "n_gpus": world, "steps": args.steps,
                          "higher_is_better": False, "dtype": "fp8_e4m3", "data": "synthetic",
                          "config": {"workload": "deepseek_v3_moe_decode", "tokens_per_gpu": tokens, "experts": E,
                                     "top_k": TOPK, "routing": "softmax top-8, Zipf(1.2) expert popularity",
                                     "parallelism": f"ep{world}",
                                     "exchange": "peer-to-peer stores, masked layout" if (host_free and world > 1)
                                     else ("none (one rank)" if world == 1 else "nccl all-to-all, masked layout"),
                                     "cuda_graph": graphed}}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile", default="", choices=["", "gemm1", "gemm2", "dense", "gemm16", "kgrouped", "bandwidth", "sweep", "timeline"],
                    help="run only one kernel on a small case (for ncu) and exit")
    ap.add_argument("--experts", type=int, default=32, help="experts of the --profile case")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=T_PER_GPU, help="tokens per GPU per step")
    ap.add_argument("--cpu-tokens", type=int, default=32, help="tokens of the CPU baseline sample")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--workload", default="prefill", choices=["prefill", "decode"],
                    help="prefill = the headline benchmark; decode = 128 tokens per GPU, latency percentiles")
    args = ap.parse_args()
    if args.profile == "bandwidth":
        run_profile_bandwidth(args)
    elif args.profile == "sweep":
        run_profile_sweep(args)
    elif args.profile == "timeline" and args.workload == "decode":
        run_decode(args)
    elif args.profile == "timeline":
        run_profile_timeline(args)
    elif args.profile:
        run_profile(args)
    elif args.workload == "decode" and args.impl == "b200":
        run_decode(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
