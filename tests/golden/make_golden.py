"""Generate the golden fixtures under tests/golden/ by running the reference's own code.

Run once, in a container that has the reference checkout, with
    python tests/golden/make_golden.py --reference <path-to-reference-checkout>
The fixtures it writes (``*.pt``) are committed; tests never need the checkout.

How the reference runs without a GPU: its Triton kernels execute under the Triton
interpreter (TRITON_INTERPRET=1).  The package cannot be imported as a whole on a
CPU-only box (its ``__init__`` probes the GPU and imports every kernel), so empty
parent packages are pre-seeded in ``sys.modules`` with ``__path__`` pointing into
the checkout and sub-modules are then imported by file.  The interpreter rounds
fp32->bf16 / fp32->fp8 casts differently from GPUs, so only cast-free results are
stored: integer outputs, fp32 outputs and fp32 scales.
"""
import argparse
import ast
import contextlib
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def install_shim(ref: str):
    pkg_root = os.path.join(ref, "dlblas")

    def mk(name, path):
        m = types.ModuleType(name)
        m.__path__ = [path]
        sys.modules[name] = m
        return m

    mk("dlblas", pkg_root)
    mk("dlblas.kernels", os.path.join(pkg_root, "kernels"))
    mk("dlblas.layers", os.path.join(pkg_root, "layers"))
    mk("dlblas.layers.moe", os.path.join(pkg_root, "layers", "moe"))
    mk("dlblas.layers.moe.kernels", os.path.join(pkg_root, "layers", "moe", "kernels"))

    dev = types.ModuleType("dlblas.utils.device_utils")
    dev.get_device_props = lambda idx=0: {"multi_processor_count": 8, "warps_per_sm": 8}
    dev.infer_device = lambda: "cpu"
    dev.is_npu = dev.is_cuda = dev.is_tma_supported = dev.is_muxi = dev.is_mlu = lambda: False
    dev.NUM_CORES = 8
    dev.DEVICE = "cpu"
    sys.modules["dlblas.utils.device_utils"] = dev

    # keep only the first autotune config, the interpreter cannot benchmark
    real_autotune = triton.autotune

    def one_config_autotune(configs, key, **kw):
        kw.pop("warmup", None)
        kw.pop("rep", None)
        return real_autotune(configs=configs[:1], key=key, **kw)

    triton.autotune = one_config_autotune
    torch.cuda.device = lambda d: contextlib.nullcontext()


@triton.jit
def _exp(x):
    return tl.exp(x)


def gold_sort(ref, out):
    from dlblas.layers.moe.kernels.fused_moe import _dlblas_get_sorted_idx
    # inputs and expected vectors hard-coded in the reference's own test file
    src = open(os.path.join(ref, "tests", "test_dlblas_get_sorted_idx.py")).read()
    tree = ast.parse(src)
    cases = []
    for fn in [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name.startswith("test_")]:
        vals = {}
        for node in ast.walk(fn):
            if isinstance(node, ast.Assign) and isinstance(node.targets[0], ast.Name):
                name = node.targets[0].id
                v = node.value
                if isinstance(v, ast.Call) and getattr(v.func, "attr", "") == "tensor":
                    vals[name] = ast.literal_eval(v.args[0])
                elif isinstance(v, ast.Constant) and name == "num_experts":
                    vals[name] = v.value
        ids = torch.tensor(vals["topk_ids"], dtype=torch.int64)
        s_idx, s, e = _dlblas_get_sorted_idx(ids, vals["num_experts"])
        cases.append(dict(name=fn.name, topk_ids=ids, num_experts=vals["num_experts"],
                          test_sorted_idx=torch.tensor(vals["expected_sorted_idx"]),
                          test_exp_start=torch.tensor(vals["expected_exp_start"]),
                          test_exp_end=torch.tensor(vals["expected_exp_end"]),
                          run_sorted_idx=s_idx.clone(), run_exp_start=s.clone(), run_exp_end=e.clone()))
    g = torch.Generator().manual_seed(1)
    for (t, k, e) in [(64, 2, 8), (257, 8, 256), (33, 4, 16)]:
        ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)])
        if e == 16:
            ids[ids < 4] = -1
        s_idx, s, en = _dlblas_get_sorted_idx(ids, e)
        cases.append(dict(name=f"random_{t}x{k}_E{e}", topk_ids=ids, num_experts=e,
                          run_sorted_idx=s_idx.clone(), run_exp_start=s.clone(), run_exp_end=en.clone()))
    torch.save(cases, os.path.join(out, "sort.pt"))
    print("sort:", len(cases), "cases")


def gold_quant(ref, out):
    from dlblas.kernels.fp8 import per_token_group_quant_fp8
    from dlblas.kernels.moe import quant_fp8
    g = torch.Generator().manual_seed(2)
    x = torch.randn(48, 512, generator=g).to(torch.bfloat16)
    x[3, 128:256] *= 100.0
    x[5, :128] *= 1e-4
    _, s_moe = quant_fp8(x, 128)
    _, s_grp = per_token_group_quant_fp8(x, 128)
    _, s_col = per_token_group_quant_fp8(x, 128, column_major_scales=True)
    torch.save(dict(x=x, scale_quant_fp8=s_moe.clone(), scale_per_token_group=s_grp.clone(),
                    scale_colmajor=s_col.clone().contiguous(), colmajor_stride=tuple(s_col.stride())),
               os.path.join(out, "quant.pt"))
    print("quant: ok")


def gold_gemm(ref, out):
    from dlblas.kernels.fp8_gemm import fp8_gemm
    g = torch.Generator().manual_seed(3)
    m, n, k = 192, 256, 384
    a = torch.randn(m, k, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, generator=g).to(torch.float8_e4m3fn)
    a_s = torch.randn(m, k // 128, generator=g)
    b_s = torch.randn(n // 128, k // 128, generator=g)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.float32)
    c = fp8_gemm(a, b, a_s, b_s)
    torch.set_default_dtype(old)
    torch.save(dict(a=a, b=b, a_s=a_s, b_s=b_s, c_fp32=c.clone()), os.path.join(out, "fp8_gemm.pt"))
    print("fp8_gemm: ok")


def gold_grouped(ref, out):
    from dlblas.layers.moe.kernels.blocked_fp8_fused_moe import fused_moe_blocked_fp8_kernel_launcher
    from dlblas.layers.moe.kernels.fused_moe import _dlblas_get_sorted_idx
    g = torch.Generator().manual_seed(4)
    t, h, n, e, k = 40, 256, 384, 6, 2
    xq = torch.randn(t, h, generator=g).to(torch.float8_e4m3fn)
    xs = torch.rand(t, h // 128, generator=g) + 0.5
    w = torch.randn(e, n, h, generator=g).to(torch.float8_e4m3fn)
    ws = torch.rand(e, n // 128, h // 128, generator=g) + 0.5
    ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)])
    wts = torch.rand(t, k, generator=g)
    sidx, st, en = _dlblas_get_sorted_idx(ids, e)
    c1 = torch.zeros(t * k, n, dtype=torch.float32)
    fused_moe_blocked_fp8_kernel_launcher(xq, xs, w, ws, c1, sidx, st, en, wts, enable_weights=False,
                                          top_k=k, num_tokens=t, reindex_a=True, reindex_c=False)
    aq = torch.randn(t * k, h, generator=g).to(torch.float8_e4m3fn)
    as_ = torch.rand(t * k, h // 128, generator=g) + 0.5
    c2 = torch.zeros(t * k, n, dtype=torch.float32)
    fused_moe_blocked_fp8_kernel_launcher(aq, as_, w, ws, c2, sidx, st, en, wts, enable_weights=True,
                                          top_k=1, num_tokens=t, reindex_a=False, reindex_c=True)
    torch.save(dict(xq=xq, xs=xs, w=w, ws=ws, ids=ids, wts=wts, sorted_idx=sidx.clone(), exp_start=st.clone(),
                    exp_end=en.clone(), c1_fp32=c1, aq=aq, as_=as_, c2_fp32=c2, top_k=k),
               os.path.join(out, "grouped_gemm.pt"))
    print("grouped: ok")


def gold_activation(ref, out):
    import dlblas.layers.moe.kernels.activation as act
    act.fast_expf = _exp
    g = torch.Generator().manual_seed(5)
    gu = torch.randn(24, 512, generator=g) * 3
    o = act.silu_and_mul(gu)
    torch.save(dict(gate_up=gu, out_fp32=o.clone()), os.path.join(out, "silu_and_mul.pt"))
    print("silu_and_mul: ok")


def gold_grouped_topk(ref, out):
    from dlblas.kernels.moe import biased_grouped_topk
    cases = []
    g = torch.Generator().manual_seed(6)
    for (e, ng, tg, tk, t) in [(128, 4, 2, 4, 64), (256, 8, 4, 8, 512), (512, 16, 8, 16, 33)]:
        logits = torch.randn(t, e, generator=g)
        bias = torch.randn(e, generator=g) * 0.01
        w, ids = biased_grouped_topk(logits, logits, bias, tk, True, ng, tg)
        cases.append(dict(logits=logits, bias=bias, topk=tk, num_expert_group=ng, topk_group=tg,
                          weights=w.clone(), ids=ids.clone()))
    torch.save(cases, os.path.join(out, "grouped_topk.pt"))
    print("grouped_topk:", len(cases), "cases")


def gold_topk_gating(ref, out):
    import dlblas.kernels.topk_gating_fwd_part1 as p1
    import dlblas.kernels.topk_gating_fwd_part2 as p2
    p1.tl_exp = _exp
    p2.logits = types.SimpleNamespace(device="cpu")
    from dlblas.kernels.topk_gating import call
    cases = []
    g = torch.Generator().manual_seed(7)
    for (t, e, k, cf, mc, hp) in [(64, 8, 2, 1.0, 2, False), (64, 8, 2, 1.0, 2, True), (96, 16, 4, 0.5, 2, False)]:
        logits = torch.randn(t, e, generator=g)
        l_aux, ec, w, sel = call(logits, k, cf, mc, hp)
        cases.append(dict(logits=logits, k=k, capacity_factor=cf, min_capacity=mc, higher_precision=hp,
                          l_aux=l_aux.clone(), ec_idx=ec.clone(), weights=w.clone(), select=sel.clone()))
    torch.save(cases, os.path.join(out, "topk_gating.pt"))
    print("topk_gating:", len(cases), "cases")


def gold_topk_gating_bwd(ref, out):
    """Gradient of the gating's auxiliary loss with respect to the logits: the reference's default backward
    (dlblas/kernels/topk_gating.py:270-276 -> topk_gating_bwd.py:50-68), and the two kernels of its
    higher-precision backward (topk_gating.py:186-242) fed with the gradient of the token weights."""
    import dlblas.kernels.topk_gating_fwd_part1 as p1
    import dlblas.kernels.topk_gating_fwd_part2 as p2
    p1.tl_exp = _exp
    p2.logits = types.SimpleNamespace(device="cpu")
    from dlblas.kernels.topk_gating import TopKGatingFunc, topk_bwd_triton, topk_fwd_triton
    from dlblas.kernels.topk_gating import _capacity
    from dlblas.kernels.topk_gating_fwd_part1 import call as part1
    from dlblas.kernels.topk_gating_fwd_part2 import call as part2
    cases = []
    g = torch.Generator().manual_seed(9)
    for (t, e, k, cf) in [(64, 8, 2, 1.0), (96, 16, 4, 0.5)]:
        logits = torch.randn(t, e, generator=g).requires_grad_(True)
        l_aux, ec, w, sel = TopKGatingFunc.apply(logits, k, cf, 2, False)
        gl = torch.tensor(0.7)
        l_aux.backward(gl)
        case = dict(logits=logits.detach().clone(), k=k, capacity_factor=cf, min_capacity=2, grad_l_aux=gl,
                    grad_logits_default=logits.grad.clone())
        # higher-precision pieces, called directly (the autograd wrapper of the reference indexes the wrong
        # output gradient, so it cannot be driven through .backward())
        capacity = _capacity(logits.detach(), torch.tensor(cf * k), torch.tensor(2)).item()
        gates, masks = part1(logits.detach(), k)
        locations, res, ce = part2(gates, masks, k)
        ec2, w2, sel2, for_bwd = topk_fwd_triton(gates, masks, locations, capacity)
        gw = torch.randn(k * t, generator=g)
        try:
            grad = topk_bwd_triton(gates, ce, masks, *for_bwd, gl, gw.view(k, t))
            case.update(grad_weights=gw, grad_logits_hp_reference=grad.clone(), weights_hp=w2.clone(),
                        gate_ks=for_bwd[0].clone(), denom=for_bwd[2].clone())
        except Exception as exc:
            case["hp_error"] = repr(exc)[:300]
        cases.append(case)
    torch.save(cases, os.path.join(out, "topk_gating_bwd.pt"))
    print("topk_gating_bwd:", len(cases), "cases", [c.get("hp_error", "hp ok") for c in cases])


def gold_permute(ref, out):
    """Training-side permutation (dlblas/kernels/permute/moe_triton_kernels.py): permute / un-permute forward
    and backward on fp32 data (no low-precision casts, which the interpreter rounds differently)."""
    sys.modules.setdefault("dlblas.kernels.permute", types.ModuleType("dlblas.kernels.permute")).__path__ = [
        os.path.join(ref, "dlblas", "kernels", "permute")]
    import dlblas.kernels.permute.moe_triton_kernels as P
    cases = []
    g = torch.Generator().manual_seed(31)
    for (t, k, e, h, neg) in [(37, 2, 8, 64, False), (50, 4, 16, 128, True)]:
        x = torch.randn(t, h, generator=g)
        ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32)
        if neg:
            ids[torch.rand(t, k, generator=g) < 0.2] = -1
        n_neg = int((ids == -1).sum())
        n_out = t * k - n_neg
        permuted = torch.zeros(n_out, h)
        row_id_map = torch.full((t * k,), -1, dtype=torch.int32)   # the reference leaves unrouted entries unwritten
        ws = []
        perm, rmap, sorted_ids, ws = P.moe_permute_topk_op_triton(x, ids, n_out, ws, t * k, n_neg, permuted, row_id_map)
        probs = torch.rand(t, k, generator=g)
        y = torch.randn(n_out, h, generator=g)
        un = P.moe_recover_topk_op_triton(y, rmap, probs, t, k)
        un_noprob = P.moe_recover_topk_op_triton(y, rmap, None, t, k)
        go = torch.randn(t, h, generator=g)
        act_grad, prob_grad = P.moe_recover_topk_bwd_op_triton(go, y, rmap, probs)
        gperm = torch.randn(n_out, h, generator=g)
        case = dict(x=x, ids=ids, permuted=perm.clone(), row_id_map=rmap.clone(), sorted_row_id=sorted_ids.clone(),
                    probs=probs, y=y, unpermuted=un.clone(), unpermuted_noprob=un_noprob.clone(), grad_out=go,
                    act_grad=act_grad.clone(), prob_grad=prob_grad.clone(), grad_permuted=gperm)
        if not neg:
            case["permute_bwd"] = P.moe_permute_topk_bwd_op(gperm, sorted_ids, (t, h), k).clone()
        cases.append(case)
    torch.save(cases, os.path.join(out, "permute.pt"))
    print("permute:", len(cases), "cases")


def gold_align(ref, out):
    """moe_align_block_size (dlblas/kernels/moe_align_block_size.py:138-210) under the interpreter."""
    from dlblas.kernels.moe_align_block_size import moe_align_block_size
    cases = []
    # the worked example of the function's own docstring (:160-176), shifted to 0-based expert ids
    ids = torch.tensor([[1, 2, 3], [0, 1, 3], [0, 2, 3], [0, 1, 2]], dtype=torch.int32)
    todo = [(ids, 4, 4, False)]
    g = torch.Generator().manual_seed(41)
    for (t, k, e, bs, pad) in [(40, 2, 8, 16, False), (65, 4, 16, 64, True), (9, 8, 32, 128, False)]:
        todo.append((torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32), bs, e, pad))
    for (ids, bs, e, pad) in todo:
        s_ids, e_ids, n_post = moe_align_block_size(ids.clone(), bs, e, e, None, pad)
        cases.append(dict(topk_ids=ids, block_size=bs, num_experts=e, pad_sorted_ids=pad, sorted_ids=s_ids.clone(),
                          expert_ids=e_ids.clone(), num_tokens_post_pad=n_post.clone()))
    torch.save(cases, os.path.join(out, "align_block.pt"))
    print("align_block:", len(cases), "cases; docstring example ->", cases[0]["sorted_ids"].tolist())


def gold_scatter_gather(ref, out):
    from dlblas.kernels.fused_moe_v3 import ep_gather, ep_scatter
    g = torch.Generator().manual_seed(8)
    e, t, k, h = 3, 13, 2, 1024
    topk = torch.full((t, k), -1, dtype=torch.int32)
    for i in range(t):
        sel = torch.randperm(e, generator=g)[:k]
        keep = torch.rand(k, generator=g) > 0.3
        topk[i] = torch.where(keep, sel.to(torch.int32), torch.full((k,), -1, dtype=torch.int32))
    real_counts = torch.bincount(topk[topk >= 0].to(torch.int64), minlength=e).to(torch.int32)
    counts = (real_counts + 127) // 128 * 128          # the dispatcher aligns every expert to 128 rows
    total = int(counts.sum())
    x = torch.randn(t, h, generator=g).to(torch.float8_e4m3fn)
    xs = torch.randn(t, h // 128, generator=g)
    out_x = torch.zeros(total, h, dtype=torch.float8_e4m3fn)
    out_s = torch.zeros(total, h // 128)
    m_idx = torch.zeros(total, dtype=torch.int32)
    out_index = torch.zeros_like(topk)
    start = torch.zeros_like(counts)
    ep_scatter(x, xs, topk, counts, start, out_x, out_s, m_idx, out_index)
    y = torch.randn(total, h, generator=g).to(torch.bfloat16)
    wt = torch.rand(t, k, generator=g)
    gat = torch.zeros(t, h, dtype=torch.float32)
    ep_gather(y, topk, wt, out_index, gat)
    torch.save(dict(x=x, xs=xs, topk=topk, counts=counts, real_counts=real_counts, out_x=out_x, out_s=out_s, m_indices=m_idx,
                    output_index=out_index, y=y, wt=wt, gather_fp32=gat), os.path.join(out, "scatter_gather.pt"))
    print("scatter_gather: ok")


def gold_eplb(ref, out):
    """Expert-parallel load balancer: the hash replica choice (Triton kernel under the interpreter and the
    reference test's own golden model) and the re-balancing tables of dlblas/layers/moe/eplb.py."""
    import importlib.util
    from dlblas.kernels.moe import map_logic_to_physical_idx_hash_random
    spec = importlib.util.spec_from_file_location("ref_test_eplb", os.path.join(ref, "tests", "kernels", "test_eplb.py"))
    tmod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tmod)
    golden_model = tmod.reference_map_logic_to_physical_idx_hash_random
    cases = []
    # the known-answer inputs of tests/kernels/test_eplb.py:94-103
    topk = torch.tensor([[1, 2], [2, 2], [0, 1], [1, 3]], dtype=torch.int32)
    log2phy = torch.tensor([[10, 11], [12, 13], [14, -1], [15, 16]], dtype=torch.int32)
    logcnt = torch.tensor([2, 2, 1, 2], dtype=torch.int32)
    cases.append(dict(name="reference_test", topk_idx=topk, log2phy=log2phy, logcnt=logcnt, seed=99999))
    g = torch.Generator().manual_seed(21)
    for (t, k, e, r, seed) in [(70, 8, 32, 3, 12345), (300, 4, 16, 4, 7), (66000, 2, 8, 2, 99999)]:
        logcnt = torch.randint(0, r + 1, (e,), generator=g, dtype=torch.int32)
        log2phy = torch.full((e, r), -1, dtype=torch.int32)
        nxt = 0
        for i in range(e):
            for j in range(int(logcnt[i])):
                log2phy[i, j] = nxt
                nxt += 1
        topk = torch.randint(-1, e, (t, k), generator=g, dtype=torch.int32)
        cases.append(dict(name=f"random_{t}x{k}", topk_idx=topk, log2phy=log2phy, logcnt=logcnt, seed=seed))
    for c in cases:
        small = c["topk_idx"].shape[0] <= 300
        name = c["name"]
        if small:
            try:
                c["kernel_out"] = map_logic_to_physical_idx_hash_random(c["topk_idx"], c["log2phy"], c["logcnt"],
                                                                        seed=c["seed"]).clone()
            except Exception as exc:   # the interpreter rejects the kernel's 0xFFFFFFFF literal as an int32 scalar
                c["kernel_out"] = None
                c["kernel_error"] = repr(exc)[:200]
            c["model_out"] = golden_model(c["topk_idx"], c["log2phy"], c["logcnt"], seed=c["seed"])
        else:
            # the interpreter needs minutes for 66000 tokens: only the rows whose (t << 16) leaves 32 bits
            sel = torch.arange(65530, 65560)
            full = golden_model(c["topk_idx"][:65560], c["log2phy"], c["logcnt"], seed=c["seed"])
            c["rows"] = sel
            c["model_out_rows"] = full[sel]
            c["num_tokens"] = c["topk_idx"].shape[0]
            c["topk_rows"] = c["topk_idx"][sel].clone()      # tests rebuild the batch: these rows, -1 elsewhere
            del c["topk_idx"]
        print("eplb hash", name, "kernel == model:",
              bool(torch.equal(c["kernel_out"], c["model_out"])) if small and c["kernel_out"] is not None else "n/a")

    # ---- re-balancing tables (host code; the reference calls .cuda() on an index tensor) ----
    torch.Tensor.cuda = lambda self, *a, **k: self
    import dlblas.layers.moe.eplb as E
    tables = []
    g = torch.Generator().manual_seed(22)
    for (layers, experts, replicas, groups, nodes, gpus) in [(2, 16, 24, 4, 1, 4), (3, 32, 40, 8, 2, 8),
                                                             (2, 16, 20, 3, 2, 4), (1, 256, 288, 8, 1, 8),
                                                             (2, 8, 8, 4, 1, 4)]:
        w = (torch.rand(layers, experts, generator=g) * 1000).float()
        phy2log, log2phy, logcnt = E.rebalance_experts(w, replicas, groups, nodes, gpus)
        disp = E.compute_logical_to_rank_dispatch_physical_map(log2phy, gpus, replicas, seed=42)
        tables.append(dict(weight=w, num_replicas=replicas, num_groups=groups, num_nodes=nodes, num_gpus=gpus,
                           phy2log=phy2log, log2phy=log2phy, logcnt=logcnt, dispatch=disp))
    # the default statistic of EPLBMetadata.init (descending integers: ties between load / replica quotients)
    w = torch.arange(64, dtype=torch.int32).flip(dims=(0,)).expand(2, -1)
    phy2log, log2phy, logcnt = E.rebalance_experts(w, 64 + 16, 4, 1, 8)
    tables.append(dict(weight=w.clone(), num_replicas=80, num_groups=4, num_nodes=1, num_gpus=8, phy2log=phy2log,
                       log2phy=log2phy, logcnt=logcnt,
                       dispatch=E.compute_logical_to_rank_dispatch_physical_map(log2phy, 8, 80, seed=42)))
    torch.save(dict(hash=cases, tables=tables), os.path.join(out, "eplb.pt"))
    print("eplb:", len(cases), "hash cases,", len(tables), "tables")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    install_shim(a.reference)
    todo = [gold_sort, gold_quant, gold_gemm, gold_grouped, gold_activation, gold_grouped_topk,
            gold_topk_gating, gold_topk_gating_bwd, gold_scatter_gather, gold_eplb, gold_permute, gold_align]
    for fn in todo:
        if a.only and a.only not in fn.__name__:
            continue
        fn(a.reference, a.out)


if __name__ == "__main__":
    main()
