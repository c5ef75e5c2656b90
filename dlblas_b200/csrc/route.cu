// Routing kernels: one warp per token row, scores in registers, warp-shuffle arg-max with
// a deterministic tie-break (lowest expert index wins).
#include "common.cuh"
#include "sort.cuh"

namespace dlb {
namespace {

constexpr int WARPS = 8;
constexpr int MAX_VPT = 32;  // up to 1024 experts

struct ArgMax {
  float v;
  int i;
};
// larger value wins; equal values: smaller index wins
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ ArgMax warp_argmax(ArgMax a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  return a;
}

constexpr float NEG_INF = -__builtin_huge_valf();

// Element e of a row lives in lane e % 32, register e / 32 (coalesced loads).
template <typename T, int VPT>
__device__ __forceinline__ void load_row(const T* row, int experts, int lane, float (&x)[VPT]) {
#pragma unroll
  for (int s = 0; s < VPT; ++s) {
    const int e = s * 32 + lane;
    x[s] = e < experts ? to_f32<T>(row[e]) : NEG_INF;
  }
}

template <int VPT>
__device__ __forceinline__ ArgMax row_argmax(const float (&x)[VPT], int lane) {
  ArgMax a = {NEG_INF, 0x7fffffff};
#pragma unroll
  for (int s = 0; s < VPT; ++s) a = better(a, ArgMax{x[s], s * 32 + lane});
  return warp_argmax(a);
}

template <int VPT>
__device__ __forceinline__ void knock_out(float (&x)[VPT], int idx, int lane) {
#pragma unroll
  for (int s = 0; s < VPT; ++s)
    if (s * 32 + lane == idx) x[s] = NEG_INF;
}

// topk(softmax(logits)) : selection on the logits themselves (softmax is monotone), weights
// = exp(x - max) / sum.
template <typename T, int VPT, typename IdT>
__global__ void __launch_bounds__(WARPS * 32) softmax_topk_kernel(const T* __restrict__ logits, long long tokens,
                                                                  int experts, int top_k, int renorm,
                                                                  float* __restrict__ weights, IdT* __restrict__ ids) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (t >= tokens) return;
  float x[VPT];
  load_row<T, VPT>(logits + t * experts, experts, lane, x);
  float mx = NEG_INF;
#pragma unroll
  for (int s = 0; s < VPT; ++s) mx = fmaxf(mx, x[s]);
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int s = 0; s < VPT; ++s) sum += (s * 32 + lane < experts) ? expf(x[s] - mx) : 0.f;
  sum = warp_sum(sum);
  float my_w = 0.f;
  int my_id = 0;
  float wsum = 0.f;
  for (int j = 0; j < top_k; ++j) {   // top_k <= 32: lane j keeps slot j
    const ArgMax a = row_argmax<VPT>(x, lane);
    const float w = expf(a.v - mx) / sum;
    wsum += w;
    if (lane == j) {
      my_w = w;
      my_id = a.i;
    }
    knock_out<VPT>(x, a.i, lane);
  }
  if (lane < top_k) {
    weights[t * top_k + lane] = renorm ? my_w / wsum : my_w;
    ids[t * top_k + lane] = (IdT)my_id;
  }
}

// Logistic function whose result does not depend on any library's exponential: evaluated in fp64 with
// individually rounded IEEE operations only (no fused multiply-add, no transcendental call) and rounded
// once to fp32, so that a restatement with the same sequence of operations on any IEEE machine gives the
// same bits.  exp(z), z = -x: n = rint(z * log2(e)), r = z - n * ln2 (two-part constant),
// degree-13 Taylor polynomial in r (|r| <= 0.35: truncation below 1e-17), scaled by 2^n in two exact steps.
// The score differs from a correctly rounded fp32 sigmoid in well under one input in a million, and from
// torch's fp32 sigmoid by at most one unit in the last place.
__device__ __forceinline__ double pow2_exact(int n) { return __longlong_as_double((long long)(n + 1023) << 52); }

__device__ __forceinline__ float sigmoid_exact(float x) {
  double z = -(double)x;
  z = fmin(fmax(z, -750.0), 750.0);
  const double n = rint(__dmul_rn(z, 1.4426950408889634));
  double r = __dsub_rn(z, __dmul_rn(n, 0.6931471803691238));
  r = __dsub_rn(r, __dmul_rn(n, 1.9082149292705877e-10));
  double p = 1.6059043836821613e-10;
  p = __dadd_rn(__dmul_rn(p, r), 2.08767569878681e-09);
  p = __dadd_rn(__dmul_rn(p, r), 2.505210838544172e-08);
  p = __dadd_rn(__dmul_rn(p, r), 2.755731922398589e-07);
  p = __dadd_rn(__dmul_rn(p, r), 2.7557319223985893e-06);
  p = __dadd_rn(__dmul_rn(p, r), 2.48015873015873e-05);
  p = __dadd_rn(__dmul_rn(p, r), 0.0001984126984126984);
  p = __dadd_rn(__dmul_rn(p, r), 0.001388888888888889);
  p = __dadd_rn(__dmul_rn(p, r), 0.008333333333333333);
  p = __dadd_rn(__dmul_rn(p, r), 0.041666666666666664);
  p = __dadd_rn(__dmul_rn(p, r), 0.16666666666666666);
  p = __dadd_rn(__dmul_rn(p, r), 0.5);
  p = __dadd_rn(__dmul_rn(p, r), 1.0);
  p = __dadd_rn(__dmul_rn(p, r), 1.0);
  const int ni = (int)n;              // |n| <= 1083
  const int n1 = ni / 2, n2 = ni - n1;  // both powers of two are normal numbers
  const double e = __dmul_rn(__dmul_rn(p, pow2_exact(n1)), pow2_exact(n2));
  return __double2float_rn(__ddiv_rn(1.0, __dadd_rn(1.0, e)));
}

// DeepSeek-V3 style grouped routing (dlblas/kernels/moe.py:477-521).
template <typename T, int VPT>
__global__ void __launch_bounds__(WARPS * 32) grouped_topk_kernel(const T* __restrict__ logits,
                                                                  const float* __restrict__ bias, long long tokens,
                                                                  int experts, int num_groups, int topk_group, int top_k,
                                                                  int renorm, float* __restrict__ weights,
                                                                  int* __restrict__ ids) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int per_group = experts / num_groups;
  float sc[VPT];   // unbiased sigmoid scores
  float ch[VPT];   // biased scores used for the choice
  {
    float x[VPT];
    load_row<T, VPT>(logits + t * experts, experts, lane, x);
#pragma unroll
    for (int s = 0; s < VPT; ++s) {
      const int e = s * 32 + lane;
      if (e < experts) {
        sc[s] = sigmoid_exact(x[s]);
        ch[s] = sc[s] + __ldg(bias + e);
      } else {
        sc[s] = 0.f;
        ch[s] = NEG_INF;
      }
    }
  }
  // group score = sum of the two largest biased scores of the group; lane g keeps group g's score
  float gscore = NEG_INF;
  for (int g = 0; g < num_groups; ++g) {
    const int lo = g * per_group, hi = lo + per_group;
    ArgMax a = {NEG_INF, 0x7fffffff};
#pragma unroll
    for (int s = 0; s < VPT; ++s) {
      const int e = s * 32 + lane;
      if (e >= lo && e < hi) a = better(a, ArgMax{ch[s], e});
    }
    a = warp_argmax(a);
    ArgMax b = {NEG_INF, 0x7fffffff};
#pragma unroll
    for (int s = 0; s < VPT; ++s) {
      const int e = s * 32 + lane;
      if (e >= lo && e < hi && e != a.i) b = better(b, ArgMax{ch[s], e});
    }
    b = warp_argmax(b);
    if (lane == g) gscore = a.v + b.v;
  }
  // keep the topk_group best groups (bit mask, same in every lane)
  unsigned keep = 0;
  for (int j = 0; j < topk_group; ++j) {
    ArgMax a = {gscore, lane};
    if (lane >= num_groups) a = ArgMax{NEG_INF, 0x7fffffff};
    a = warp_argmax(a);
    keep |= 1u << a.i;
    if (lane == a.i) gscore = NEG_INF;
  }
#pragma unroll
  for (int s = 0; s < VPT; ++s) {
    const int e = s * 32 + lane;
    if (e < experts && !((keep >> (e / per_group)) & 1u)) ch[s] = NEG_INF;
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < top_k; ++j) {
    const ArgMax a = row_argmax<VPT>(ch, lane);
    // owner lane broadcasts the unbiased score of the chosen expert
    float w = 0.f;
#pragma unroll
    for (int s = 0; s < VPT; ++s)
      if (s * 32 + lane == a.i) w = sc[s];
    w = __shfl_sync(0xffffffffu, w, a.i & 31);
    wsum += w;
    if (lane == j) {
      my_w = w;
      my_id = a.i;
    }
    knock_out<VPT>(ch, a.i, lane);
  }
  if (lane < top_k) {
    weights[t * top_k + lane] = renorm ? my_w / wsum : my_w;
    ids[t * top_k + lane] = my_id;
  }
}

// ---- capacity-limited gating (dlblas.topk_gating) -----------------------------------
// part 1: gates = exp(x) / sum(exp(x)) (no max subtraction, topk_gating_fwd_part1.py:38-41),
// k rounds of arg-max on the gates; ids and chosen gates are written k-major.
template <typename T, int VPT>
__global__ void __launch_bounds__(WARPS * 32) gating_part1_kernel(const T* __restrict__ logits, long long tokens,
                                                                  int experts, int top_k, float* __restrict__ gates,
                                                                  int* __restrict__ ids_km, float* __restrict__ gate_km) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (t >= tokens) return;
  float x[VPT];
  load_row<T, VPT>(logits + t * experts, experts, lane, x);
  float sum = 0.f;
#pragma unroll
  for (int s = 0; s < VPT; ++s) {
    x[s] = (s * 32 + lane < experts) ? expf(x[s]) : NEG_INF;
    sum += (s * 32 + lane < experts) ? x[s] : 0.f;
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int s = 0; s < VPT; ++s) {
    const int e = s * 32 + lane;
    if (e < experts) {
      x[s] = x[s] / sum;
      gates[t * experts + e] = x[s];
    }
  }
  for (int j = 0; j < top_k; ++j) {
    const ArgMax a = row_argmax<VPT>(x, lane);
    if (lane == 0) {
      ids_km[(long long)j * tokens + t] = a.i;
      gate_km[(long long)j * tokens + t] = a.v;
    }
    knock_out<VPT>(x, a.i, lane);
  }
}

// part 2: per expert, me = mean of gates, ce = share of tokens whose first choice it is
// (topk_gating_fwd_part2.py:31-36); fixed summation order, no atomics.
__global__ void __launch_bounds__(256) gating_colsum_kernel(const float* __restrict__ gates,
                                                            const int* __restrict__ ids_km, long long tokens,
                                                            int experts, float* __restrict__ res,
                                                            float* __restrict__ ce_out) {
  __shared__ float s_sum[8][33];
  __shared__ int s_cnt[8][33];
  const int ex = threadIdx.x & 31, y = threadIdx.x >> 5;
  const int e = blockIdx.x * 32 + ex;
  float sum = 0.f;
  int cnt = 0;
  if (e < experts) {
    for (long long t = y; t < tokens; t += 8) {
      sum += gates[t * experts + e];
      cnt += (ids_km[t] == e) ? 1 : 0;
    }
  }
  s_sum[y][ex] = sum;
  s_cnt[y][ex] = cnt;
  __syncthreads();
  if (y == 0 && e < experts) {
    float tot = 0.f;
    int c = 0;
    for (int i = 0; i < 8; ++i) {
      tot += s_sum[i][ex];
      c += s_cnt[i][ex];
    }
    const float me = tot / (float)tokens;
    const float ce = (float)c / (float)tokens;
    res[e] = me * ce * (float)experts * (float)experts;
    ce_out[e] = ce;                                     // kept for the backward pass
  }
}

// part 3: drop entries beyond the capacity, renormalise the kept gates, emit the indices
// (topk_gating_fwd_part3.py:9-61) and the kept part of expert_select_token_idx.
template <typename T>
__global__ void __launch_bounds__(256) gating_part3_kernel(const int* __restrict__ ids_km,
                                                           const float* __restrict__ gate_km,
                                                           const int* __restrict__ rank, const float* __restrict__ res,
                                                           long long tokens, int experts, int top_k, long long capacity,
                                                           T* __restrict__ l_aux, int* __restrict__ ec_idx,
                                                           T* __restrict__ out_w, long long* __restrict__ select) {
  const long long t = (long long)blockIdx.x * 256 + threadIdx.x;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    float s = 0.f;
    for (int e = 0; e < experts; ++e) s += res[e];
    *l_aux = from_f32<T>(s / (float)experts);
  }
  if (t >= tokens) return;
  float denom = 0.f;
  for (int j = 0; j < top_k; ++j) {
    const long long f = (long long)j * tokens + t;
    if (rank[f] < capacity) denom += gate_km[f];
  }
  const float eps = sizeof(T) == 2 ? 9.765625e-4f : 1.1920929e-7f;   // torch.finfo(dtype).eps
  denom = denom < eps ? eps : denom;
  for (int j = 0; j < top_k; ++j) {
    const long long f = (long long)j * tokens + t;
    const int loc = rank[f];
    const bool kept = loc < capacity;
    out_w[f] = from_f32<T>(kept ? gate_km[f] / denom : 0.f);
    ec_idx[f] = kept ? (int)((long long)ids_km[f] * capacity + loc) : 0;
    if (kept) select[(long long)ids_km[f] * capacity + loc] = t;
  }
}

// Experts with fewer than `capacity` tokens: the remaining slots of expert_select_token_idx
// take the tokens that did not choose the expert, in ascending order (what a stable
// descending sort of the reference's int mask gives).  One warp per expert.
__global__ void __launch_bounds__(WARPS * 32) gating_fill_kernel(const int* __restrict__ ids_km,
                                                                 const int* __restrict__ counts, long long tokens,
                                                                 int experts, int top_k, long long capacity,
                                                                 long long* __restrict__ select) {
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (e >= experts) return;
  long long filled = counts[e];
  if (filled >= capacity) return;
  for (long long t0 = 0; t0 < tokens && filled < capacity; t0 += 32) {
    const long long t = t0 + lane;
    bool free_tok = t < tokens;
    if (free_tok)
      for (int j = 0; j < top_k; ++j) free_tok = free_tok && (ids_km[(long long)j * tokens + t] != e);
    const unsigned m = __ballot_sync(0xffffffffu, free_tok);
    const long long pos = filled + __popc(m & ((1u << lane) - 1u));
    if (free_tok && pos < capacity) select[(long long)e * capacity + pos] = t;
    filled += __popc(m);
  }
}

template <template <int> class Launcher, typename... Args>
int dispatch_vpt(int experts, Args... args) {
  if (experts <= 32) return Launcher<1>::run(args...);
  if (experts <= 64) return Launcher<2>::run(args...);
  if (experts <= 128) return Launcher<4>::run(args...);
  if (experts <= 256) return Launcher<8>::run(args...);
  if (experts <= 512) return Launcher<16>::run(args...);
  return Launcher<32>::run(args...);
}

struct SoftmaxArgs {
  const void* logits;
  int dtype;
  long long tokens;
  int experts, top_k, renorm;
  float* weights;
  void* ids;
  int ids_dtype;
  cudaStream_t st;
};
template <int VPT> struct SoftmaxLauncher {
  template <typename T> static void go(const SoftmaxArgs& a) {
    const int grid = (int)ceil_div(a.tokens, WARPS);
    if (a.ids_dtype == DLB_I32)
      softmax_topk_kernel<T, VPT, int><<<grid, WARPS * 32, 0, a.st>>>(reinterpret_cast<const T*>(a.logits), a.tokens,
                                                                     a.experts, a.top_k, a.renorm, a.weights,
                                                                     reinterpret_cast<int*>(a.ids));
    else
      softmax_topk_kernel<T, VPT, long long><<<grid, WARPS * 32, 0, a.st>>>(reinterpret_cast<const T*>(a.logits),
                                                                           a.tokens, a.experts, a.top_k, a.renorm,
                                                                           a.weights, reinterpret_cast<long long*>(a.ids));
  }
  static int run(SoftmaxArgs a) {
    if (a.dtype == DLB_F32) go<float>(a);
    else if (a.dtype == DLB_BF16) go<__nv_bfloat16>(a);
    else go<__half>(a);
    count_launch();
    DLB_CHECK_LAUNCH("softmax_topk_kernel");
    return DLB_OK;
  }
};

struct GroupedArgs {
  const void* logits;
  int dtype;
  const float* bias;
  long long tokens;
  int experts, num_groups, topk_group, top_k, renorm;
  float* weights;
  int* ids;
  cudaStream_t st;
};
template <int VPT> struct GroupedLauncher {
  template <typename T> static void go(const GroupedArgs& a) {
    grouped_topk_kernel<T, VPT><<<(int)ceil_div(a.tokens, WARPS), WARPS * 32, 0, a.st>>>(
        reinterpret_cast<const T*>(a.logits), a.bias, a.tokens, a.experts, a.num_groups, a.topk_group, a.top_k, a.renorm,
        a.weights, a.ids);
  }
  static int run(GroupedArgs a) {
    if (a.dtype == DLB_F32) go<float>(a);
    else if (a.dtype == DLB_BF16) go<__nv_bfloat16>(a);
    else go<__half>(a);
    count_launch();
    DLB_CHECK_LAUNCH("grouped_topk_kernel");
    return DLB_OK;
  }
};

struct GatingArgs {
  const void* logits;
  int dtype;
  long long tokens;
  int experts, top_k;
  float* gates;
  int* ids_km;
  float* gate_km;
  cudaStream_t st;
};
template <int VPT> struct GatingLauncher {
  static int run(GatingArgs a) {
    const int grid = (int)ceil_div(a.tokens, WARPS);
    if (a.dtype == DLB_F32)
      gating_part1_kernel<float, VPT><<<grid, WARPS * 32, 0, a.st>>>(reinterpret_cast<const float*>(a.logits), a.tokens,
                                                                    a.experts, a.top_k, a.gates, a.ids_km, a.gate_km);
    else
      gating_part1_kernel<__half, VPT><<<grid, WARPS * 32, 0, a.st>>>(reinterpret_cast<const __half*>(a.logits), a.tokens,
                                                                     a.experts, a.top_k, a.gates, a.ids_km, a.gate_km);
    count_launch();
    DLB_CHECK_LAUNCH("gating_part1_kernel");
    return DLB_OK;
  }
};

// Backward of the gating: d(l_aux)/d(logits) and, on request, d(token_exp_weights)/d(logits).
//   add[e]  = ce[e] * grad_l_aux * E / T                                  (dlblas/kernels/topk_gating_bwd.py:31-33)
//           + sum over kept slots j with ids[j] == e of
//             ( gw[j] / D + [D not clamped] * sum_i(-gw[i] * g[i] / D^2) )   (w[j] = g[j] / D, D = sum of kept gates)
//   grad[e] = gates[e] * (add[e] - sum_i gates[i] * add[i])                (softmax backward, :40-44)
// One warp per token; reads what the forward left in its workspace.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32) gating_bwd_kernel(const float* __restrict__ gates,
                                                                const float* __restrict__ ce,
                                                                const int* __restrict__ ids_km,
                                                                const float* __restrict__ gate_km,
                                                                const int* __restrict__ rank, long long tokens,
                                                                int experts, int top_k, long long capacity,
                                                                const T* __restrict__ grad_l_aux,
                                                                const T* __restrict__ grad_w, T* __restrict__ grad_logits) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const float gl = to_f32<T>(*grad_l_aux) * (float)experts / (float)tokens;
  const float eps = sizeof(T) == 2 ? 9.765625e-4f : 1.1920929e-7f;   // torch.finfo(dtype).eps
  float denom = 0.f, coupling = 0.f;
  if (grad_w != nullptr) {
    for (int j = 0; j < top_k; ++j) {
      const long long f = (long long)j * tokens + t;
      if (rank[f] < capacity) denom += gate_km[f];
    }
    const bool clamped = denom < eps;
    const float cd = clamped ? eps : denom;
    if (!clamped) {
      for (int j = 0; j < top_k; ++j) {
        const long long f = (long long)j * tokens + t;
        if (rank[f] < capacity) coupling -= to_f32<T>(grad_w[f]) * gate_km[f] / (cd * cd);
      }
    }
    denom = cd;
  }
  const float* g_row = gates + t * experts;
  float dot = 0.f;
  for (int e = lane; e < experts; e += 32) {
    float add = ce[e] * gl;
    if (grad_w != nullptr) {
      for (int j = 0; j < top_k; ++j) {
        const long long f = (long long)j * tokens + t;
        if (ids_km[f] == e && rank[f] < capacity) add += to_f32<T>(grad_w[f]) / denom + coupling;
      }
    }
    dot += g_row[e] * add;
  }
  dot = warp_sum(dot);
  for (int e = lane; e < experts; e += 32) {
    float add = ce[e] * gl;
    if (grad_w != nullptr) {
      for (int j = 0; j < top_k; ++j) {
        const long long f = (long long)j * tokens + t;
        if (ids_km[f] == e && rank[f] < capacity) add += to_f32<T>(grad_w[f]) / denom + coupling;
      }
    }
    grad_logits[t * experts + e] = from_f32<T>(g_row[e] * (add - dot));
  }
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

struct GatingWs {
  size_t gates, ids_km, gate_km, rank, res, ce, counts, sort, bytes;
};
GatingWs gating_ws(long long tokens, int experts, int top_k) {
  GatingWs w;
  size_t off = 0;
  w.gates = off; off += align256((size_t)tokens * experts * 4);
  w.ids_km = off; off += align256((size_t)tokens * top_k * 4);
  w.gate_km = off; off += align256((size_t)tokens * top_k * 4);
  w.rank = off; off += align256((size_t)tokens * top_k * 4);
  w.res = off; off += align256((size_t)experts * 4);
  w.ce = off; off += align256((size_t)experts * 4);
  w.counts = off; off += align256((size_t)experts * 4);
  w.sort = off; off += sort_workspace_size(tokens * top_k, experts);
  w.bytes = off;
  return w;
}

// Logical -> physical expert ids for replicated experts: slot (t, k) of a token picks replica
// hash32((t << 16) ^ (k << 8) ^ seed) & 0x7fffffff mod logcnt[e] of its logical expert e
// (dlblas/kernels/moe.py:524-556; all arithmetic in 32 bits, as in the golden model of
// tests/kernels/test_eplb.py:60-90).  Negative ids and experts without a replica give -1.
constexpr int EPLB_THREADS = 256;
template <typename IdT>
__global__ void __launch_bounds__(EPLB_THREADS) eplb_map_hash_kernel(const IdT* __restrict__ topk_idx,
                                                                const int* __restrict__ log2phy,
                                                                const int* __restrict__ logcnt, long long slots,
                                                                int top_k, int num_logical, int max_replica,
                                                                uint32_t seed, int* __restrict__ out) {
  for (long long i = (long long)blockIdx.x * EPLB_THREADS + threadIdx.x; i < slots; i += (long long)gridDim.x * EPLB_THREADS) {
    const long long e = (long long)topk_idx[i];
    int phy = -1;
    if (e >= 0 && e < num_logical) {
      const int cnt = __ldg(logcnt + e);
      if (cnt > 0) {
        const uint32_t t = (uint32_t)(i / top_k);
        const uint32_t k = (uint32_t)(i - (long long)t * top_k);
        uint32_t x = (t << 16) ^ (k << 8) ^ seed;
        x = ((x >> 16) ^ x) * 0x45d9f3bu;
        x = ((x >> 16) ^ x) * 0x45d9f3bu;
        x = (x >> 16) ^ x;
        const uint32_t replica = (x & 0x7fffffffu) % (uint32_t)cnt;
        phy = __ldg(log2phy + e * max_replica + replica);
      }
    }
    out[i] = phy;
  }
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" int dlb_eplb_map_hash(const void* topk_idx, int ids_dtype, const int32_t* log2phy, const int32_t* logcnt,
                                 int64_t tokens, int top_k, int num_logical, int max_replica, uint32_t seed,
                                 int32_t* physical_idx, void* stream) {
  DLB_REQUIRE(tokens >= 0 && top_k > 0 && num_logical > 0 && max_replica > 0, DLB_ERR_INVALID,
              "eplb_map_hash: bad sizes tokens=%lld top_k=%d experts=%d replicas=%d", (long long)tokens, top_k,
              num_logical, max_replica);
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(topk_idx && log2phy && logcnt && physical_idx, DLB_ERR_INVALID, "eplb_map_hash: null pointer");
  const long long slots = tokens * top_k;
  const int grid = (int)std::min<long long>(ceil_div(slots, (long long)EPLB_THREADS), (long long)sm_count() * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (ids_dtype == DLB_I32) {
    eplb_map_hash_kernel<int><<<grid, EPLB_THREADS, 0, st>>>(reinterpret_cast<const int*>(topk_idx), log2phy, logcnt, slots,
                                                        top_k, num_logical, max_replica, seed, physical_idx);
  } else if (ids_dtype == DLB_I64) {
    eplb_map_hash_kernel<long long><<<grid, EPLB_THREADS, 0, st>>>(reinterpret_cast<const long long*>(topk_idx), log2phy,
                                                              logcnt, slots, top_k, num_logical, max_replica, seed,
                                                              physical_idx);
  } else {
    return fail(DLB_ERR_INVALID, "eplb_map_hash: ids must be int32 or int64 (got %d)", ids_dtype);
  }
  count_launch();
  DLB_CHECK_LAUNCH("eplb_map_hash_kernel");
  return DLB_OK;
}

extern "C" int dlb_route_softmax_topk(const void* logits, int dtype, int64_t tokens, int experts, int top_k,
                                      int renormalize, float* weights, void* ids, int ids_dtype, void* stream) {
  DLB_REQUIRE(tokens >= 0 && experts > 0 && experts <= 32 * MAX_VPT, DLB_ERR_INVALID,
              "route_softmax_topk: experts=%d must be in [1, 1024]", experts);
  DLB_REQUIRE(top_k > 0 && top_k <= experts && top_k <= 32, DLB_ERR_INVALID,
              "route_softmax_topk: top_k=%d must be in [1, min(experts, 32)]", top_k);
  DLB_REQUIRE(dtype == DLB_F32 || dtype == DLB_BF16 || dtype == DLB_F16, DLB_ERR_INVALID,
              "route_softmax_topk: unsupported logits dtype %d", dtype);
  DLB_REQUIRE(ids_dtype == DLB_I32 || ids_dtype == DLB_I64, DLB_ERR_INVALID, "route_softmax_topk: ids must be int32/int64");
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(logits && weights && ids, DLB_ERR_INVALID, "route_softmax_topk: null pointer");
  SoftmaxArgs a = {logits, dtype, tokens, experts, top_k, renormalize, weights, ids, ids_dtype, (cudaStream_t)stream};
  return dispatch_vpt<SoftmaxLauncher>(experts, a);
}

extern "C" int dlb_route_grouped_topk(const void* logits, int dtype, const float* bias, int64_t tokens, int experts,
                                      int num_groups, int topk_group, int top_k, int renormalize, float* weights,
                                      int32_t* ids, void* stream) {
  DLB_REQUIRE(tokens >= 0 && experts > 0 && experts <= 32 * MAX_VPT, DLB_ERR_INVALID,
              "route_grouped_topk: experts=%d must be in [1, 1024]", experts);
  DLB_REQUIRE(num_groups > 0 && num_groups <= 32 && experts % num_groups == 0 && experts / num_groups >= 2,
              DLB_ERR_INVALID, "route_grouped_topk: num_groups=%d must divide experts, be <= 32, with >= 2 experts each",
              num_groups);
  DLB_REQUIRE(topk_group > 0 && topk_group <= num_groups, DLB_ERR_INVALID, "route_grouped_topk: bad topk_group %d",
              topk_group);
  DLB_REQUIRE(top_k > 0 && top_k <= 32 && top_k <= topk_group * (experts / num_groups), DLB_ERR_INVALID,
              "route_grouped_topk: top_k=%d out of range", top_k);
  DLB_REQUIRE(dtype == DLB_F32 || dtype == DLB_BF16 || dtype == DLB_F16, DLB_ERR_INVALID,
              "route_grouped_topk: unsupported logits dtype %d", dtype);
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(logits && bias && weights && ids, DLB_ERR_INVALID, "route_grouped_topk: null pointer");
  GroupedArgs a = {logits, dtype, bias, tokens, experts, num_groups, topk_group, top_k, renormalize, weights, ids,
                   (cudaStream_t)stream};
  return dispatch_vpt<GroupedLauncher>(experts, a);
}

extern "C" size_t dlb_topk_gating_workspace_size(int64_t tokens, int experts, int top_k) {
  if (tokens <= 0 || experts <= 0 || top_k <= 0) return 0;
  return gating_ws(tokens, experts, top_k).bytes;
}

extern "C" int dlb_topk_gating(const void* logits, int dtype, int64_t tokens, int experts, int top_k, int64_t capacity,
                               void* l_aux, int32_t* ec_idx, void* gate_weights, int64_t* select, void* workspace,
                               size_t workspace_bytes, void* stream) {
  DLB_REQUIRE(tokens > 0 && experts > 0 && experts <= 32 * MAX_VPT, DLB_ERR_INVALID,
              "topk_gating: experts=%d must be in [1, 1024] and tokens positive", experts);
  DLB_REQUIRE(top_k > 0 && top_k <= experts, DLB_ERR_INVALID, "topk_gating: top_k=%d out of range", top_k);
  DLB_REQUIRE(capacity > 0 && capacity <= tokens, DLB_ERR_INVALID,
              "topk_gating: capacity=%lld must be in [1, tokens=%lld]", (long long)capacity, (long long)tokens);
  DLB_REQUIRE(dtype == DLB_F32 || dtype == DLB_F16, DLB_ERR_INVALID, "topk_gating: logits must be fp32 or fp16");
  DLB_REQUIRE(logits && l_aux && ec_idx && gate_weights && select, DLB_ERR_INVALID, "topk_gating: null pointer");
  const GatingWs w = gating_ws(tokens, experts, top_k);
  DLB_REQUIRE(workspace != nullptr && workspace_bytes >= w.bytes, DLB_ERR_WORKSPACE,
              "topk_gating: workspace of %zu bytes needed, %zu given", w.bytes, workspace_bytes);
  char* ws = reinterpret_cast<char*>(workspace);
  float* gates = reinterpret_cast<float*>(ws + w.gates);
  int* ids_km = reinterpret_cast<int*>(ws + w.ids_km);
  float* gate_km = reinterpret_cast<float*>(ws + w.gate_km);
  int* rank = reinterpret_cast<int*>(ws + w.rank);
  float* res = reinterpret_cast<float*>(ws + w.res);
  int* counts = reinterpret_cast<int*>(ws + w.counts);
  cudaStream_t st = (cudaStream_t)stream;
  GatingArgs a = {logits, dtype, tokens, experts, top_k, gates, ids_km, gate_km, st};
  int rc = dispatch_vpt<GatingLauncher>(experts, a);
  if (rc != DLB_OK) return rc;
  gating_colsum_kernel<<<(int)ceil_div(experts, 32), 256, 0, st>>>(gates, ids_km, tokens, experts, res,
                                                                   reinterpret_cast<float*>(ws + w.ce));
  count_launch();
  DLB_CHECK_LAUNCH("gating_colsum_kernel");
  // position of every (slot, token) entry inside its expert, in k-major / token-minor order:
  // the cumulative sum of the one-hot masks of the reference (topk_gating_fwd_part2.py:31)
  rc = sort_by_expert(ids_km, DLB_I32, tokens * top_k, experts, nullptr, nullptr, nullptr, nullptr, rank, counts,
                      ws + w.sort, workspace_bytes - w.sort, st);
  if (rc != DLB_OK) return rc;
  const int grid3 = (int)ceil_div(tokens, 256);
  if (dtype == DLB_F32)
    gating_part3_kernel<float><<<grid3, 256, 0, st>>>(ids_km, gate_km, rank, res, tokens, experts, top_k, capacity,
                                                     reinterpret_cast<float*>(l_aux), ec_idx,
                                                     reinterpret_cast<float*>(gate_weights),
                                                     reinterpret_cast<long long*>(select));
  else
    gating_part3_kernel<__half><<<grid3, 256, 0, st>>>(ids_km, gate_km, rank, res, tokens, experts, top_k, capacity,
                                                      reinterpret_cast<__half*>(l_aux), ec_idx,
                                                      reinterpret_cast<__half*>(gate_weights),
                                                      reinterpret_cast<long long*>(select));
  count_launch();
  DLB_CHECK_LAUNCH("gating_part3_kernel");
  gating_fill_kernel<<<(int)ceil_div(experts, WARPS), WARPS * 32, 0, st>>>(ids_km, counts, tokens, experts, top_k,
                                                                          capacity, reinterpret_cast<long long*>(select));
  count_launch();
  DLB_CHECK_LAUNCH("gating_fill_kernel");
  return DLB_OK;
}

extern "C" int dlb_topk_gating_bwd(const void* workspace, size_t workspace_bytes, int dtype, int64_t tokens, int experts,
                                   int top_k, int64_t capacity, const void* grad_l_aux, const void* grad_weights,
                                   void* grad_logits, void* stream) {
  DLB_REQUIRE(tokens > 0 && experts > 0 && experts <= 32 * MAX_VPT && top_k > 0 && top_k <= experts, DLB_ERR_INVALID,
              "topk_gating_bwd: bad sizes tokens=%lld experts=%d top_k=%d", (long long)tokens, experts, top_k);
  DLB_REQUIRE(dtype == DLB_F32 || dtype == DLB_F16, DLB_ERR_INVALID, "topk_gating_bwd: dtype must be fp32 or fp16");
  DLB_REQUIRE(workspace && grad_l_aux && grad_logits, DLB_ERR_INVALID, "topk_gating_bwd: null pointer");
  const GatingWs w = gating_ws(tokens, experts, top_k);
  DLB_REQUIRE(workspace_bytes >= w.bytes, DLB_ERR_WORKSPACE,
              "topk_gating_bwd: the forward's workspace has %zu bytes, %zu given", w.bytes, workspace_bytes);
  const char* ws = reinterpret_cast<const char*>(workspace);
  const float* gates = reinterpret_cast<const float*>(ws + w.gates);
  const float* ce = reinterpret_cast<const float*>(ws + w.ce);
  const int* ids_km = reinterpret_cast<const int*>(ws + w.ids_km);
  const float* gate_km = reinterpret_cast<const float*>(ws + w.gate_km);
  const int* rank = reinterpret_cast<const int*>(ws + w.rank);
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = (int)ceil_div(tokens, WARPS);
  if (dtype == DLB_F32)
    gating_bwd_kernel<float><<<grid, WARPS * 32, 0, st>>>(gates, ce, ids_km, gate_km, rank, tokens, experts, top_k,
                                                          capacity, reinterpret_cast<const float*>(grad_l_aux),
                                                          reinterpret_cast<const float*>(grad_weights),
                                                          reinterpret_cast<float*>(grad_logits));
  else
    gating_bwd_kernel<__half><<<grid, WARPS * 32, 0, st>>>(gates, ce, ids_km, gate_km, rank, tokens, experts, top_k,
                                                           capacity, reinterpret_cast<const __half*>(grad_l_aux),
                                                           reinterpret_cast<const __half*>(grad_weights),
                                                           reinterpret_cast<__half*>(grad_logits));
  count_launch();
  DLB_CHECK_LAUNCH("gating_bwd_kernel");
  return DLB_OK;
}
