"""CPU oracle for the FP8 MoE expert path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch on the CPU, the arithmetic of the
reference's MoE expert path with round-to-nearest-even casts at exactly the
points where the reference rounds.  Only tests, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it; the
product package never does.

Parity status: pinned.  Every function below is checked (tests/test_oracle.py)
against fixtures under tests/golden/ that were produced by running the
reference's own Python/Triton sources under the Triton interpreter
(tests/golden/make_golden.py) and against the hard-coded vectors of the
reference's tests.  The Triton interpreter rounds fp32->bf16 and fp32->fp8
casts differently from real GPUs (truncation / wrong carry), so fixtures are
taken only from cast-free quantities (integer outputs, fp32 outputs, scales).

Each function cites the reference source it follows (path inside the
reference project : lines).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def _clamp_fp8(v: torch.Tensor) -> torch.Tensor:
    """`tl.clamp(v, -448, 448)` as the compiled reference kernels evaluate it (dlblas/kernels/moe.py:413,
    dlblas/kernels/fp8.py:48): min(max(v, -448), 448) with the GPU's non-propagating min / max, which return
    the non-NaN operand, so NaN (0 / 0 of an all-zero group with scale 0) becomes -448.  torch.clamp and the
    Triton interpreter propagate NaN instead; the compiled kernel is the one restated here."""
    return torch.where(torch.isnan(v), torch.full_like(v, -FP8_MAX), v.clamp(-FP8_MAX, FP8_MAX))


# --------------------------------------------------------------------------- #
# quantisation
# --------------------------------------------------------------------------- #
def quant_fp8(a: torch.Tensor, group_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """dlblas/kernels/moe.py:377-421 (`_quant_fp8_kernel`) and :466-474.

    scale = absmax * (1/448) (fp32 multiply, no epsilon), q = clamp(a / scale).
    An all-zero group gives scale 0; its 0 / 0 quotients clamp to -448 (see `_clamp_fp8`), so the
    payload is finite and the group contributes payload * 0 = 0 to any product.
    """
    assert a.dim() == 2 and a.shape[1] % group_size == 0
    m, k = a.shape
    g = a.to(torch.float32).reshape(m, k // group_size, group_size)
    rmax = torch.tensor(1.0 / FP8_MAX, dtype=torch.float32)
    scale = g.abs().amax(-1) * rmax
    q = _clamp_fp8(g / scale[..., None])
    return q.reshape(m, k).to(FP8), scale


def per_token_group_quant_fp8(x: torch.Tensor, group_size: int, eps: float = 1e-10,
                              column_major_scales: bool = False):
    """dlblas/kernels/fp8.py:9-51, 55-105, 108-182.

    scale = max(absmax, eps) / 448 (true division), q = clamp(x / scale).
    With column_major_scales the scale tensor has shape [M, G] and strides (1, M).
    """
    assert x.shape[-1] % group_size == 0
    shp = x.shape
    g = x.to(torch.float32).reshape(-1, shp[-1] // group_size, group_size)
    absmax = torch.maximum(g.abs().amax(-1), torch.tensor(eps, dtype=torch.float32))
    scale = absmax / torch.tensor(FP8_MAX, dtype=torch.float32)
    q = _clamp_fp8(g / scale[..., None]).reshape(shp).to(FP8)
    scale = scale.reshape(shp[:-1] + (shp[-1] // group_size,))
    if column_major_scales:
        assert x.dim() == 2
        scale = scale.t().contiguous().t()
    return q, scale


def tma_align_input_scale(scale: torch.Tensor) -> torch.Tensor:
    """dlblas/kernels/quant_dequant.py:22-83: [M, G] row-major -> view [M, G] of a
    [G, pad4(M)] buffer (column-major, M padded to a multiple of 16 bytes)."""
    m, g = scale.shape
    pad_m = (m + 3) // 4 * 4
    out = torch.zeros(g, pad_m, dtype=scale.dtype)
    out[:, :m] = scale.t()
    return out.t()[:m]


# --------------------------------------------------------------------------- #
# activation
# --------------------------------------------------------------------------- #
def silu_and_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """dlblas/layers/moe/kernels/activation.py:17-58: fp32 silu(gate) * up,
    stored in the input dtype; gate = columns [0, N), up = columns [N, 2N)."""
    n = gate_up.shape[-1] // 2
    g = gate_up[..., :n].to(torch.float32)
    u = gate_up[..., n:].to(torch.float32)
    return ((g / (1.0 + torch.exp(-g))) * u).to(gate_up.dtype)


def silu_and_mul_masked_post_quant(inp: torch.Tensor, masked_m: torch.Tensor, group_size: int = 128):
    """dlblas/kernels/moe.py:204-269: for rows < masked_m[e]:
    g = in_dtype(silu_fp32(gate)); p = up * g (in the input dtype);
    scale = max(absmax(p), 1e-10) / 448; q = clamp(p / scale).  Rows at or beyond
    masked_m[e] are left untouched (returned as zeros here, with scale 0)."""
    e, m, n2 = inp.shape
    n = n2 // 2
    out = torch.zeros(e, m, n, dtype=torch.float32)
    out_s = torch.zeros(e, m, n // group_size, dtype=torch.float32)
    for i in range(e):
        r = int(masked_m[i])
        if r == 0:
            continue
        gate = inp[i, :r, :n].to(torch.float32)
        up = inp[i, :r, n:]
        gate = (gate / (1.0 + torch.exp(-gate))).to(inp.dtype)
        p = (up * gate).to(torch.float32).reshape(r, n // group_size, group_size)
        absmax = torch.maximum(p.abs().amax(-1), torch.tensor(1e-10, dtype=torch.float32))
        s = absmax / torch.tensor(FP8_MAX, dtype=torch.float32)
        out[i, :r] = _clamp_fp8(p / s[..., None]).reshape(r, n)
        out_s[i, :r] = s
    return out.to(FP8), out_s


# --------------------------------------------------------------------------- #
# GEMMs
# --------------------------------------------------------------------------- #
def fp8_gemm(a: torch.Tensor, b: torch.Tensor, a_s: torch.Tensor, b_s: torch.Tensor,
             out_dtype: torch.dtype = torch.bfloat16, block: int = 128) -> torch.Tensor:
    """dlblas/kernels/fp8_gemm.py:17-89 and the blockwise ground truth of
    tests/kernels/test_fp8_gemm.py:34-68.

    C[m, n] = sum_kb (sum_{j in kb} A[m, j] B[n, j]) * a_s[m, kb] * b_s[n // 128, kb],
    fp32 accumulation over kb in increasing order, cast to out_dtype at the end.
    """
    k = a.shape[-1]
    a2 = a.reshape(-1, k).to(torch.float32)
    m = a2.shape[0]
    n = b.shape[0]
    b2 = b.to(torch.float32)
    a_s2 = a_s.reshape(m, -1)
    kb_n = (k + block - 1) // block
    acc = torch.zeros(m, n, dtype=torch.float32)
    bs_rows = b_s.repeat_interleave(block, dim=0)[:n]          # [N, KB]
    for kb in range(kb_n):
        sl = slice(kb * block, min((kb + 1) * block, k))
        part = a2[:, sl] @ b2[:, sl].t()
        acc += part * a_s2[:, kb:kb + 1] * bs_rows[:, kb][None, :]
    return acc.to(out_dtype).reshape(*a.shape[:-1], n)


def stable_sort_by_expert(topk_ids: torch.Tensor, num_experts: int):
    """dlblas/layers/moe/kernels/fused_moe.py:27-51, 83-88.

    sorted_idx = argsort(ids.flatten()) with the canonical (stable) tie order:
    ascending flat index inside each expert segment, `-1` entries first.
    exp_start[e] = first sorted position holding e, exp_end = start + count; an
    expert without tokens gets start = end = 0 (the `exp_start *= 0` branch at :47-49).
    """
    flat = topk_ids.flatten().to(torch.int64)
    sorted_idx = torch.argsort(flat, stable=True)
    valid = flat[flat >= 0]
    cnt = torch.bincount(valid, minlength=num_experts)[:num_experts]
    n_neg = int((flat < 0).sum())
    end = torch.cumsum(cnt, 0) + n_neg
    start = end - cnt
    start = torch.where(cnt > 0, start, torch.zeros_like(start))
    end = torch.where(cnt > 0, end, torch.zeros_like(end))
    return sorted_idx, start, end


def grouped_gemm(a, a_s, b, b_s, sorted_idx, exp_start, exp_end, weights=None, *, top_k=1,
                 expert_offset=0, reindex_a=True, reindex_c=True, num_rows_c=None,
                 out_dtype=torch.bfloat16, zeros=True, block=128):
    """dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py:30-156 (+ launcher :159-242).

    For local expert e (global id e + expert_offset) and every sorted position p in
    [exp_start, exp_end): A row = sorted_idx[p] // top_k if reindex_a else p; the
    block-scaled product with B[e] is accumulated in fp32 over 128-wide K blocks,
    optionally multiplied by weights.flatten()[sorted_idx[p]] in fp32, cast to
    out_dtype and written to row sorted_idx[p] if reindex_c else p.
    """
    e_local, n, k = b.shape
    if num_rows_c is None:
        num_rows_c = sorted_idx.numel()
    c = torch.zeros(num_rows_c, n, dtype=out_dtype)
    wflat = None if weights is None else weights.flatten().to(torch.float32)
    for e in range(e_local):
        s, t = int(exp_start[e + expert_offset]), int(exp_end[e + expert_offset])
        if t <= s:
            continue
        pos = torch.arange(s, t)
        sid = sorted_idx[pos]
        rows_a = sid // top_k if reindex_a else pos
        acc = fp8_gemm(a[rows_a], b[e], a_s[rows_a], b_s[e], out_dtype=torch.float32, block=block)
        if wflat is not None:
            acc = acc * wflat[sid][:, None]
        rows_c = sid if reindex_c else pos
        c[rows_c] = acc.to(out_dtype)
    return c


def fused_moe_blocked_fp8(x_q, x_s, w1, w1_s, w2, w2_s, topk_weights, topk_ids, topk,
                          out_dtype=torch.bfloat16, expert_offset=0, num_experts=None,
                          renormalize=False, ep_size=1, group_size=128):
    """dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py:261-338, with the rounding
    points of the GPU path: GEMM1 -> out_dtype, silu*up -> out_dtype, quant_fp8,
    GEMM2 (x routed weight in fp32) -> out_dtype, sum over k in out_dtype.
    Does not mutate topk_ids (the reference adds expert_offset in place, :288)."""
    e_local = w1.shape[0]
    if num_experts is None:
        num_experts = e_local * (ep_size if ep_size > 1 else 1)
    if renormalize:
        topk_weights = topk_weights / topk_weights.sum(dim=-1, keepdim=True)
    ids = topk_ids.clone().to(torch.int64)
    ids[ids != -1] += expert_offset
    sorted_idx, exp_start, exp_end = stable_sort_by_expert(ids, num_experts)
    m = x_q.shape[0]
    c1 = grouped_gemm(x_q, x_s, w1, w1_s, sorted_idx, exp_start, exp_end, None, top_k=topk,
                      expert_offset=expert_offset, reindex_a=True, reindex_c=False,
                      num_rows_c=m * topk, out_dtype=out_dtype)
    h = silu_and_mul(c1)
    # rows that belong to no local expert are zero: 0/0 would poison the scale, the
    # reference never reads those rows in GEMM2 either.
    h_q, h_s = quant_fp8(h, group_size)
    c2 = grouped_gemm(h_q, h_s, w2, w2_s, sorted_idx, exp_start, exp_end, topk_weights, top_k=1,
                      expert_offset=expert_offset, reindex_a=False, reindex_c=True,
                      num_rows_c=m * topk, out_dtype=out_dtype)
    return c2.reshape(m, topk, -1).sum(dim=1)


def moe_layer(x, topk_weights, topk_ids, w13, w13_s, w2, w2_s, top_k, renormalize=False,
              expert_offset=0, num_experts=None, ep_size=1, group_size=128):
    """dlblas/layers/moe/ep_moe.py:444-484 (`DlblasTritonFusedMoEBlockedF8Impl.forward`)."""
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    x_q, x_s = quant_fp8(x2, group_size)
    out = fused_moe_blocked_fp8(x_q, x_s, w13, w13_s, w2, w2_s, topk_weights, topk_ids, top_k,
                                out_dtype=x.dtype, expert_offset=expert_offset, num_experts=num_experts,
                                renormalize=renormalize, ep_size=ep_size, group_size=group_size)
    return out.reshape(shp)


def dense_swiglu_mlp(x, w13, w13_s, w2, w2_s, group_size=128):
    """Shared expert of the DeepSeek-V3-shaped configuration: one dense SwiGLU MLP with
    the same quantisation and rounding points as one routed expert with weight 1."""
    x_q, x_s = quant_fp8(x, group_size)
    c1 = fp8_gemm(x_q, w13, x_s, w13_s, out_dtype=x.dtype)
    h_q, h_s = quant_fp8(silu_and_mul(c1), group_size)
    return fp8_gemm(h_q, w2, h_s, w2_s, out_dtype=x.dtype)


# --------------------------------------------------------------------------- #
# routing
# --------------------------------------------------------------------------- #
def _first_max_topk(scores: torch.Tensor, k: int):
    """k rounds of argmax, lowest index on ties (the canonical tie-break)."""
    s = scores.clone().to(torch.float32)
    t, e = s.shape
    ids = torch.empty(t, k, dtype=torch.int64)
    vals = torch.empty(t, k, dtype=torch.float32)
    ar = torch.arange(e)
    for j in range(k):
        mx = s.max(dim=1, keepdim=True).values
        first = torch.where(s == mx, ar[None, :], torch.full((1, 1), e)).min(dim=1).values
        ids[:, j] = first
        vals[:, j] = mx[:, 0]
        s[torch.arange(t), first] = -float("inf")
    return vals, ids


def softmax_topk(logits: torch.Tensor, k: int, renormalize: bool = False):
    """Routing used by the reference's callers and tests
    (tests/kernels/test_fused_moe_v2.py:100-102, tests/kernels/test_fused_moe.py:213-215):
    topk(softmax(logits, fp32), k) then optional w / sum(w)
    (dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py:245-250)."""
    p = torch.softmax(logits.to(torch.float32), dim=-1)
    w, ids = _first_max_topk(p, k)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, ids


_EXP_TAYLOR = [1.6059043836821613e-10, 2.08767569878681e-09, 2.505210838544172e-08, 2.755731922398589e-07,
               2.7557319223985893e-06, 2.48015873015873e-05, 0.0001984126984126984, 0.001388888888888889,
               0.008333333333333333, 0.041666666666666664, 0.16666666666666666, 0.5, 1.0, 1.0]


def sigmoid_exact(x: torch.Tensor) -> torch.Tensor:
    """Canonical sigmoid of the routing scores (`scores = gating_output.sigmoid()`, dlblas/kernels/moe.py:490).

    torch's fp32 sigmoid goes through a library exponential whose last bit differs between CPUs and GPUs, so
    "the reference's score" is only defined up to one fp32 ulp.  The canonical value used by this oracle and
    by the CUDA kernel is the fp64 evaluation below, made of individually rounded IEEE multiplies, adds and
    one divide (every torch call here is one such operation), rounded once to fp32: any IEEE machine
    reproduces it bit for bit.  It is within one fp32 ulp of torch.sigmoid, so routing decisions differ
    from a reference run only where two candidates are within an ulp or two of each other."""
    z = (-x.to(torch.float64)).clamp(-750.0, 750.0)
    n = torch.round(z * 1.4426950408889634)
    r = z - n * 0.6931471803691238
    r = r - n * 1.9082149292705877e-10
    p = torch.full_like(r, _EXP_TAYLOR[0])
    for c in _EXP_TAYLOR[1:]:
        p = p * r + c                       # two roundings: torch does not fuse them
    ni = n.to(torch.int64)
    n1 = torch.div(ni, 2, rounding_mode="trunc")
    n2 = ni - n1

    def pow2(k):
        return ((k + 1023) << 52).view(torch.float64)

    e = (p * pow2(n1)) * pow2(n2)
    return (1.0 / (1.0 + e)).to(torch.float32)


def biased_grouped_topk(gating_output, correction_bias, topk, renormalize, num_expert_group,
                        topk_group, routed_scaling_factor=None):
    """dlblas/kernels/moe.py:477-521 with canonical tie-breaks: group score = sum of the
    two largest (sigmoid + bias) in the group; keep the topk_group best groups (lowest
    group index on ties); top-k of the biased scores inside kept groups (lowest expert
    index on ties, slots in descending biased score); weights = unbiased sigmoid at the
    chosen experts, divided by their sum when renormalize.  Returns fp32 weights and
    int32 ids.  The reference's `topk(sorted=False)` leaves the slot order open, so ids
    are compared with the reference as per-row sets."""
    scores = sigmoid_exact(gating_output.to(torch.float32))
    t, e = scores.shape
    choice = scores + correction_bias.to(torch.float32)[None, :]
    grp = choice.view(t, num_expert_group, -1)
    top2, _ = _first_max_topk(grp.reshape(t * num_expert_group, -1), 2)
    gscore = top2.sum(-1).view(t, num_expert_group)
    _, gidx = _first_max_topk(gscore, topk_group)
    gmask = torch.zeros(t, num_expert_group, dtype=torch.bool)
    gmask.scatter_(1, gidx, True)
    emask = gmask[:, :, None].expand(t, num_expert_group, e // num_expert_group).reshape(t, e)
    masked = choice.masked_fill(~emask, -float("inf"))
    _, ids = _first_max_topk(masked, topk)
    w = scores.gather(1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.to(torch.float32), ids.to(torch.int32)


def topk_gating(logits: torch.Tensor, k: int, capacity_factor: float = 1.0, min_capacity: int = 2):
    """dlblas/kernels/topk_gating.py:15-24, 245-268 with part1 (topk_gating_fwd_part1.py:16-52),
    part2 (topk_gating_fwd_part2.py:11-42) and part3 (topk_gating_fwd_part3.py:9-61, 123-155);
    same results as the torch restatement in benchmarks/topk_gating.py:130-196.

    Canonical choices where the reference leaves the order open: argmax ties go to the
    lowest expert index; `torch.topk(..., dim=0)` over the int mask is taken as a stable
    descending sort (lowest token index first among equal values).
    Returns (l_aux, token_rearranged_ec_idx int32 [k*T], token_exp_weights [k*T],
    expert_select_token_idx int64 [E*capacity]).
    """
    t, e = logits.shape
    lg = logits.to(torch.float32)
    ex = torch.exp(lg)                                   # part1: no max subtraction
    gates = ex / ex.sum(dim=1, keepdim=True)
    # float32 product, as `(T / E) * torch.tensor(capacity_factor * k)` evaluates (topk_gating.py:15-24, 254)
    capacity = int(torch.ceil((t / e) * torch.tensor(capacity_factor * k)).to(torch.int64))
    capacity = max(capacity, int(min_capacity))
    _, ids = _first_max_topk(gates, k)                   # [T, k]
    ids_ks = ids.t().contiguous()                        # [k, T]
    masks = torch.nn.functional.one_hot(ids_ks.reshape(-1), num_classes=e)   # [k*T, E]
    locations = torch.cumsum(masks, dim=0) - 1
    masks = masks.reshape(k, t, e)
    locations = locations.reshape(k, t, e)
    me = gates.mean(dim=0)
    ce = masks[0].to(torch.float32).mean(dim=0)
    l_aux = torch.mean(me * ce * e * e)
    masks = masks * (locations < capacity)
    locations_s = (locations * masks).sum(dim=2)         # [k, T]
    gate_s, indices_s = torch.max(gates[None] * masks.to(torch.float32), dim=2)
    # torch.max returns an unspecified index for an all-zero row; the kernel's
    # tl.max(return_indices=True) on zeros gives index 0.
    indices_s = torch.where(masks.sum(dim=2) > 0, indices_s, torch.zeros_like(indices_s))
    denom = gate_s.sum(dim=0)
    denom = torch.clamp(denom, min=torch.finfo(torch.float32).eps)
    gate_s = gate_s / denom
    ec_idx = (indices_s.to(torch.int32) * capacity + locations_s.to(torch.int32)).reshape(-1)
    sel = (masks * torch.arange(k, 0, -1).reshape(k, 1, 1)).sum(dim=0)       # [T, E]
    order = torch.argsort(sel, dim=0, descending=True, stable=True)[:capacity]  # [C, E]
    expert_select = order.t().reshape(e * capacity)
    return l_aux.to(logits.dtype), ec_idx, gate_s.reshape(-1).to(logits.dtype), expert_select.to(torch.int64)


# --------------------------------------------------------------------------- #
# permute / combine of the contiguous (DeepGEMM-style) layout
# --------------------------------------------------------------------------- #
def ep_scatter(recv_x, recv_x_scale, recv_topk, num_recv_tokens_per_expert):
    """dlblas/kernels/fused_moe_v3.py:19-155.  The reference allocates slots with
    atomics, so the order inside one expert is open; the canonical order is token-major,
    then slot-major (what a sequential run of the kernel produces).
    Returns (out_x, out_scale, m_indices, output_index, expert_start_loc)."""
    counts = num_recv_tokens_per_expert.to(torch.int64)
    total = int(counts.sum())
    start = torch.cumsum(counts, 0) - counts
    out_x = torch.zeros(total, recv_x.shape[1], dtype=recv_x.dtype)
    out_s = torch.zeros(total, recv_x_scale.shape[1], dtype=recv_x_scale.dtype)
    m_indices = torch.repeat_interleave(torch.arange(counts.numel()), counts).to(torch.int32)
    output_index = torch.zeros_like(recv_topk)
    cur = start.clone()
    for t in range(recv_topk.shape[0]):
        for j in range(recv_topk.shape[1]):
            ex = int(recv_topk[t, j])
            if ex >= 0:
                d = int(cur[ex])
                cur[ex] += 1
                output_index[t, j] = d
                out_x[d] = recv_x[t]
                out_s[d] = recv_x_scale[t]
    return out_x, out_s, m_indices, output_index, start


def ep_gather(inp, recv_topk_ids, recv_topk_weight, input_index, out_dtype=torch.bfloat16):
    """dlblas/kernels/fused_moe_v3.py:159-233: out[t] = sum_k w[t,k] * in[idx[t,k]] over
    slots with id >= 0, fp32 accumulation in slot order, cast to out_dtype."""
    t, k = recv_topk_ids.shape
    acc = torch.zeros(t, inp.shape[1], dtype=torch.float32)
    for j in range(k):
        ok = recv_topk_ids[:, j] >= 0
        rows = input_index[:, j].to(torch.int64).clamp(min=0)
        contrib = inp[rows].to(torch.float32) * recv_topk_weight[:, j:j + 1].to(torch.float32)
        acc = torch.where(ok[:, None], acc + contrib, acc)
    return acc.to(out_dtype)


# --------------------------------------------------------------------------- #
# synthetic inputs of the benchmark configurations
# --------------------------------------------------------------------------- #
def quantize_weight_blocks(w: torch.Tensor, block: int = 128):
    """Weights ~N(0, 0.02^2) are quantised per 128x128 block: scale = absmax / 448,
    q = RNE_e4m3(w / scale); scales fp32 [E, N/128, K/128]."""
    e, n, k = w.shape
    blk = w.reshape(e, n // block, block, k // block, block)
    s = blk.abs().amax(dim=(2, 4), keepdim=True) / FP8_MAX
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = (blk / s).clamp(-FP8_MAX, FP8_MAX).reshape(e, n, k).to(FP8)
    return q, s.reshape(e, n // block, k // block).to(torch.float32)


def make_layer_inputs(t, h, i, e, seed=0, w_std=0.02):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g)
    w13 = torch.randn(e, 2 * i, h, generator=g) * w_std
    w2 = torch.randn(e, h, i, generator=g) * w_std
    w13_q, w13_s = quantize_weight_blocks(w13)
    w2_q, w2_s = quantize_weight_blocks(w2)
    return x, logits, w13_q, w13_s, w2_q, w2_s


def rel_frobenius(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.to(torch.float64)
    b = b.to(torch.float64)
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def eplb_hash_map(topk_idx: torch.Tensor, log2phy: torch.Tensor, logcnt: torch.Tensor, seed: int = 12345) -> torch.Tensor:
    """dlblas/kernels/moe.py:524-556 and the golden model tests/kernels/test_eplb.py:60-90: replica
    hash32((t << 16) ^ (k << 8) ^ seed) & 0x7fffffff mod logcnt[e], all arithmetic modulo 2^32."""
    import numpy as np
    t, k = topk_idx.shape
    ids = topk_idx.cpu().numpy().astype(np.int64)
    l2p = log2phy.cpu().numpy().astype(np.int64)
    cnt = logcnt.cpu().numpy().astype(np.int64)
    tt = np.arange(t, dtype=np.uint64)[:, None]
    kk = np.arange(k, dtype=np.uint64)[None, :]
    mask = np.uint64(0xFFFFFFFF)
    x = ((tt << np.uint64(16)) ^ (kk << np.uint64(8)) ^ np.uint64(seed & 0xFFFFFFFF)) & mask
    for _ in range(2):
        x = (((x >> np.uint64(16)) ^ x) * np.uint64(0x45d9f3b)) & mask
    x = ((x >> np.uint64(16)) ^ x) & np.uint64(0x7FFFFFFF)
    safe_ids = np.clip(ids, 0, len(cnt) - 1)
    c = cnt[safe_ids]
    ok = (ids >= 0) & (c > 0)
    replica = (x.astype(np.int64) % np.maximum(c, 1))
    out = np.where(ok, l2p[safe_ids, np.minimum(replica, l2p.shape[1] - 1)], -1)
    return torch.from_numpy(out.astype(np.int32))


def topk_gating_grad(logits: torch.Tensor, k: int, capacity_factor: float, min_capacity: int, grad_l_aux,
                     grad_weights=None) -> torch.Tensor:
    """Gradient of (l_aux, token_exp_weights) with respect to the logits by automatic differentiation of
    `topk_gating` above (indices, masks and capacity drops are constants; clamp passes the gradient where
    the denominator is not clamped).  With grad_weights=None this is the reference's default backward,
    dlblas/kernels/topk_gating_bwd.py:13-68 (only the auxiliary loss is differentiated)."""
    x = logits.detach().to(torch.float32).clone().requires_grad_(True)
    l_aux, _, w, _ = topk_gating(x, k, capacity_factor, min_capacity)
    loss = l_aux * torch.as_tensor(grad_l_aux, dtype=torch.float32)
    if grad_weights is not None:
        loss = loss + (w * grad_weights.to(torch.float32).reshape(-1)).sum()
    loss.backward()
    return x.grad


def topk_gating_bwd_reference_hp(logits: torch.Tensor, k: int, capacity_factor: float, min_capacity: int, grad_l_aux,
                                 grad_weights: torch.Tensor) -> torch.Tensor:
    """The two kernels of the reference's higher-precision backward exactly as written
    (dlblas/kernels/topk_gating.py:139-183): they divide the saved, already normalised weights by the
    denominator twice, so the coupling term is 1/denominator too small compared with the true gradient."""
    t, e = logits.shape
    lg = logits.to(torch.float32)
    ex = torch.exp(lg)
    gates = ex / ex.sum(dim=1, keepdim=True)
    capacity = max(int(math.ceil((t / e) * (capacity_factor * k))), int(min_capacity))
    _, ids = _first_max_topk(gates, k)
    ids_ks = ids.t().contiguous()
    masks = torch.nn.functional.one_hot(ids_ks.reshape(-1), num_classes=e)
    locations = (torch.cumsum(masks, dim=0) - 1).reshape(k, t, e)
    masks = masks.reshape(k, t, e)
    ce = masks[0].to(torch.float32).mean(dim=0)
    masks = masks * (locations < capacity)
    gate_s, indices_s = torch.max(gates[None] * masks.to(torch.float32), dim=2)
    indices_s = torch.where(masks.sum(dim=2) > 0, indices_s, torch.zeros_like(indices_s))
    eps = torch.finfo(torch.float32).eps
    denom = gate_s.sum(dim=0)
    cd = torch.clamp(denom, min=eps)
    w = gate_s / cd
    gw = grad_weights.to(torch.float32).reshape(k, t)
    coupling = torch.where(denom >= eps, (-gw * (w / cd / cd)).sum(dim=0), torch.zeros_like(denom))
    add_1 = gw / cd + coupling
    scat = torch.zeros(k, t, e).scatter_(2, indices_s.unsqueeze(-1), add_1.unsqueeze(-1))
    add_2 = (scat * masks).sum(dim=0) + ce * torch.as_tensor(grad_l_aux, dtype=torch.float32) * e / t
    dx = gates * add_2
    return dx - gates * dx.sum(dim=1, keepdim=True)


def permute_topk(tokens: torch.Tensor, indices: torch.Tensor):
    """dlblas/kernels/permute/moe_triton_kernels.py:17-137 (the torch model is permute_torch of
    tests/kernels/permute/permute_triton.py:23-38): rows in stable expert order, slots routed to -1 dropped.
    Returns (permuted [routed, H], row_id_map int32 [k*T] k-major with -1 for dropped slots, sorted slot ids)."""
    t, k = indices.shape
    flat = indices.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    dropped = int((flat < 0).sum())
    kept = order[dropped:]
    permuted = tokens.index_select(0, kept // k)
    rmap = torch.full((k * t,), -1, dtype=torch.int32)
    rmap[(kept % k) * t + kept // k] = torch.arange(kept.numel(), dtype=torch.int32)
    return permuted, rmap, order


def unpermute_topk(permuted: torch.Tensor, row_id_map: torch.Tensor, probs, tokens: int, top_k: int) -> torch.Tensor:
    """gather_kernel (:229-271): accumulate in the tensor dtype, rounding after every product and add."""
    dt = permuted.dtype
    out = torch.zeros(tokens, permuted.shape[1], dtype=dt)
    rmap = row_id_map.view(top_k, tokens).to(torch.int64)
    for j in range(top_k):
        rows = rmap[j]
        ok = rows >= 0
        frag = permuted[rows.clamp(min=0)]
        if probs is not None:
            frag = (frag * probs[:, j:j + 1].to(dt)).to(dt)
        frag = torch.where(ok[:, None], frag, torch.zeros_like(frag))
        out = frag if j == 0 else (out + frag).to(dt)
    return out


def unpermute_topk_bwd(grad_out: torch.Tensor, fwd_in: torch.Tensor, row_id_map: torch.Tensor, probs: torch.Tensor):
    """scatter_bwd_kernel_optimized (:427-478): act_grad fp32 = dtype(grad_out * dtype(prob)) scattered to the
    permuted rows; prob_grad[t, k] = fp32 sum of dtype(grad_out[t] * fwd_in[row])."""
    t, k = probs.shape
    dt = grad_out.dtype
    rmap = row_id_map.view(k, t).to(torch.int64)
    act = torch.zeros(fwd_in.shape, dtype=torch.float32)
    pg = torch.zeros(t, k, dtype=torch.float32)
    for j in range(k):
        rows = rmap[j]
        ok = rows >= 0
        act[rows[ok]] = (grad_out[ok] * probs[ok, j:j + 1].to(dt)).to(dt).to(torch.float32)
        pg[ok, j] = (grad_out[ok] * fwd_in[rows[ok]]).to(dt).to(torch.float32).sum(dim=1)
    return act, pg


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int, pad_sorted_ids: bool = False):
    """dlblas/kernels/moe_align_block_size.py:138-210 (docstring example :160-176): per expert, the flat
    slot indices in ascending order, padded with `numel` to a multiple of block_size; expert id per block
    (0 past the end); total padded length."""
    flat = topk_ids.reshape(-1).to(torch.int64)
    numel = flat.numel()
    max_padded = numel + num_experts * (block_size - 1)
    if pad_sorted_ids:
        max_padded = (max_padded + block_size - 1) // block_size * block_size
    sorted_ids = torch.full((max_padded,), numel, dtype=torch.int32)
    expert_ids = torch.zeros(((max_padded + block_size - 1) // block_size,), dtype=torch.int32)
    off = 0
    for e in range(num_experts):
        slots = torch.nonzero(flat == e).flatten()
        n = int(slots.numel())
        sorted_ids[off:off + n] = slots.to(torch.int32)
        blocks = (n + block_size - 1) // block_size
        expert_ids[off // block_size: off // block_size + blocks] = e
        off += blocks * block_size
    return sorted_ids, expert_ids, torch.tensor([off], dtype=torch.int32)


def fused_moe_v2(x, w1, w1_s, w2, w2_s, topk_weights, topk_ids, group_size: int = 128, out_dtype=torch.bfloat16):
    """dlblas/kernels/fused_moe_v2.py:323-471 for block-quantised FP8: the same pipeline as
    fused_moe_blocked_fp8 with the `max(absmax, 1e-10) / 448` activation scales of
    per_token_group_quant_fp8 (moe_kernel_prepare_input, :214-225)."""
    t, k = topk_ids.shape
    x_q, x_s = per_token_group_quant_fp8(x, group_size)
    sorted_idx, exp_start, exp_end = stable_sort_by_expert(topk_ids, w1.shape[0])
    c1 = grouped_gemm(x_q, x_s, w1, w1_s, sorted_idx, exp_start, exp_end, top_k=k, reindex_a=True, reindex_c=False,
                      num_rows_c=t * k, out_dtype=out_dtype)
    h_q, h_s = per_token_group_quant_fp8(silu_and_mul(c1), group_size)
    y = grouped_gemm(h_q, h_s, w2, w2_s, sorted_idx, exp_start, exp_end, topk_weights.reshape(-1).to(torch.float32),
                     top_k=1, reindex_a=False, reindex_c=True, num_rows_c=t * k, out_dtype=out_dtype)
    return y.view(t, k, -1).sum(dim=1)


def m_grouped_gemm(a: torch.Tensor, b: torch.Tensor, size_per_group: torch.Tensor, trans_b: bool = False) -> torch.Tensor:
    """dlblas/kernels/grouped_gemm/BF16/m_grouped_gemm.py:235-352 against its ground truth `gmm`
    (utils.py:77-86): per group, fp32 accumulation of 16-bit operands, one rounding to the operand type."""
    out, start = [], 0
    for i, size in enumerate(size_per_group.tolist()):
        rhs = b[i].t() if trans_b else b[i]
        out.append((a[start:start + size].to(torch.float32) @ rhs.to(torch.float32)).to(a.dtype))
        start += size
    return torch.cat(out) if out else a.new_empty(0, b.shape[1] if trans_b else b.shape[2])


def fused_moe_16bit(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                    topk_ids: torch.Tensor) -> torch.Tensor:
    """The unquantised mode of dlblas/kernels/fused_moe_v2.py:375-466 (the vLLM-style `fused_experts`): per (token,
    slot) with a valid expert id, `c1 = x W1[e]^T` rounded to the 16-bit type, `silu(gate) * up` in fp32 rounded to that
    type (:413-423 via silu_and_mul), `y = act W2[e]^T` rounded; the token's output is the fp32 sum of
    `weight * y` over its slots, rounded once.  (The reference multiplies by the routing weight inside the second GEMM
    before rounding `y` and then sums the rounded rows; the two differ by one bf16 rounding per slot, far inside the
    test tolerance of tests/kernels/test_fused_moe_v2.py:136, atol = 0.07.)"""
    m, h = x.shape
    out = torch.zeros(m, h, dtype=torch.float32)
    for t in range(m):
        for j in range(topk_ids.shape[1]):
            e = int(topk_ids[t, j])
            if e < 0 or e >= w1.shape[0]:
                continue
            c1 = (x[t].float() @ w1[e].float().t()).to(x.dtype).float()
            n = c1.numel() // 2
            act = ((c1[:n] / (1.0 + torch.exp(-c1[:n]))) * c1[n:]).to(x.dtype).float()
            y = (act @ w2[e].float().t()).to(x.dtype).float()
            out[t] += float(topk_weights[t, j]) * y
    return out.to(x.dtype)


def k_grouped_gemm(a: torch.Tensor, b: torch.Tensor, size_per_group: torch.Tensor) -> torch.Tensor:
    """dlblas/kernels/grouped_gemm/BF16/k_grouped_gemm.py:126-176 against its ground truth `gmm_dw`
    (tests/kernels/grouped_gemm/BF16/test_k_grouped_gemm.py:10-28): c[g] = a_g^T b_g over row groups of the shared
    leading dimension, fp32 accumulation of 16-bit operands, one rounding to the operand type; zeros for an empty
    group."""
    out = a.new_zeros(size_per_group.numel(), a.shape[1], b.shape[1])
    start = 0
    for g, size in enumerate(size_per_group.tolist()):
        out[g] = (a[start:start + size].to(torch.float32).t() @ b[start:start + size].to(torch.float32)).to(a.dtype)
        start += size
    return out
