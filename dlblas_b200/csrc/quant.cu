// HBM-bound kernels of the MoE expert path: 1xG FP8 quantisation (optionally fused with
// the token-by-expert permutation), row permutation, silu*up (+ quantisation), and the
// weighted / unweighted combine.  Every thread moves 16-byte vectors; consecutive threads
// touch consecutive vectors of a row, so global accesses are fully coalesced.
#include "common.cuh"
#include "sort.cuh"

namespace dlb {
namespace {

constexpr int THREADS = 256;

template <typename T> struct Vec8 {
  // eight consecutive elements of type T
  static __device__ __forceinline__ void load(const T* p, float (&v)[8]);
  static __device__ __forceinline__ void store(T* p, const float (&v)[8]);
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
  }
};
template <> struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
  }
};

// absmax over the `lanes` (power of two, <= 32) consecutive lanes that share a group
__device__ __forceinline__ float group_max(float v, int lanes) {
  for (int o = lanes >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float quant_scale(float amax, int mode, float eps) {
  // DLB_QUANT_RECIP_MUL: dlblas/kernels/moe.py:396,410 ; DLB_QUANT_DIV_EPS: dlblas/kernels/fp8.py:46-47
  return mode == DLB_QUANT_RECIP_MUL ? amax * (1.0f / 448.0f) : fmaxf(amax, eps) / 448.0f;
}

__device__ __forceinline__ uint2 quant8(const float (&v)[8], float scale) {
  uint2 r;
  r.x = (uint32_t)f32x2_to_e4m3x2(v[0] / scale, v[1] / scale) |
        ((uint32_t)f32x2_to_e4m3x2(v[2] / scale, v[3] / scale) << 16);
  r.y = (uint32_t)f32x2_to_e4m3x2(v[4] / scale, v[5] / scale) |
        ((uint32_t)f32x2_to_e4m3x2(v[6] / scale, v[7] / scale) << 16);
  return r;
}

// One thread per 8 elements; a quantisation group of G elements spans G/8 lanes.
template <typename T>
__global__ void __launch_bounds__(THREADS) quant_fp8_kernel(const T* __restrict__ x, long long m, long long k,
                                                            long long ldx, int group, int mode, float eps,
                                                            uint8_t* __restrict__ q, float* __restrict__ scales,
                                                            long long s_rs, long long s_gs,
                                                            const int* __restrict__ dst_pos, int fanout) {
  const long long vec_per_row = k / 8;
  const long long total = m * vec_per_row;
  const int lanes = group / 8;
  for (long long u0 = (long long)blockIdx.x * THREADS; u0 < total; u0 += (long long)gridDim.x * THREADS) {
    const long long u = u0 + threadIdx.x;
    const bool active = u < total;
    const long long row = active ? u / vec_per_row : 0;
    const long long c = active ? (u - row * vec_per_row) * 8 : 0;
    float v[8];
    if (active) {
      Vec8<T>::load(x + row * ldx + c, v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = group_max(amax, lanes);
    const float scale = quant_scale(amax, mode, eps);
    if (!active) continue;
    const uint2 packed = quant8(v, scale);
    const bool first = ((c / 8) % lanes) == 0;
    const long long gidx = c / group;
    if (dst_pos == nullptr) {
      *reinterpret_cast<uint2*>(q + row * k + c) = packed;
      if (first) scales[row * s_rs + gidx * s_gs] = scale;
    } else {
      for (int j = 0; j < fanout; ++j) {
        const int d = __ldg(dst_pos + row * fanout + j);
        if (d < 0) continue;
        *reinterpret_cast<uint2*>(q + (long long)d * k + c) = packed;
        if (first) scales[(long long)d * s_rs + gidx * s_gs] = scale;
      }
    }
  }
}

// Row copies: one thread per 16 bytes of a row, plus the row's scales.
__global__ void __launch_bounds__(THREADS) permute_rows_kernel(const uint4* __restrict__ q, long long vec_per_row,
                                                               const float* __restrict__ scales, long long groups,
                                                               long long m, const int* __restrict__ dst_pos, int fanout,
                                                               uint4* __restrict__ out_q, float* __restrict__ out_s) {
  const long long total = m * vec_per_row;
  for (long long u = (long long)blockIdx.x * THREADS + threadIdx.x; u < total; u += (long long)gridDim.x * THREADS) {
    const long long row = u / vec_per_row;
    const long long c = u - row * vec_per_row;
    uint4 v = make_uint4(0, 0, 0, 0);
    float s = 0.f;
    bool loaded = false;               // rows without any destination are not read at all
    for (int j = 0; j < fanout; ++j) {
      const int d = __ldg(dst_pos + row * fanout + j);
      if (d < 0) continue;
      if (!loaded) {
        v = __ldg(q + u);
        if (scales != nullptr && c < groups) s = __ldg(scales + row * groups + c);
        loaded = true;
      }
      out_q[(long long)d * vec_per_row + c] = v;
      if (scales != nullptr && c < groups) out_s[(long long)d * groups + c] = s;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS) silu_and_mul_kernel(const T* __restrict__ in, long long rows, long long n,
                                                               long long ld_in, T* __restrict__ out, long long ld_out) {
  const long long vec_per_row = n / 8;
  const long long total = rows * vec_per_row;
  for (long long u = (long long)blockIdx.x * THREADS + threadIdx.x; u < total; u += (long long)gridDim.x * THREADS) {
    const long long row = u / vec_per_row;
    const long long c = (u - row * vec_per_row) * 8;
    float g[8], up[8], o[8];
    Vec8<T>::load(in + row * ld_in + c, g);
    Vec8<T>::load(in + row * ld_in + n + c, up);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (g[i] / (1.f + __expf(-g[i]))) * up[i];
    Vec8<T>::store(out + row * ld_out + c, o);
  }
}

// silu(gate) * up, rounded like the reference, then the 1x128 quantisation of the result.  With masked_m (masked
// layout, `experts` experts of rows_per_expert rows) only the valid rows are visited: a decode step holds a few
// hundred of them in a layout of tens of thousands.
template <typename T>
__global__ void __launch_bounds__(THREADS) silu_mul_quant_kernel(const T* __restrict__ in, long long rows, long long n,
                                                                 int mode, float eps, int round_silu,
                                                                 const int* __restrict__ masked_m, int experts,
                                                                 long long rows_per_expert, uint8_t* __restrict__ q,
                                                                 float* __restrict__ scales) {
  __shared__ int prefix[MASKED_MAX_EXPERTS + 1];
  const long long vec_per_row = n / 8;
  const long long groups = n / 128;
  long long my_rows = rows;
  if (masked_m != nullptr) {
    masked_prefix(masked_m, experts, (int)rows_per_expert, prefix);
    my_rows = prefix[experts];
  }
  const long long total = my_rows * vec_per_row;
  for (long long u0 = (long long)blockIdx.x * THREADS; u0 < total; u0 += (long long)gridDim.x * THREADS) {
    const long long u = u0 + threadIdx.x;
    const bool active = u < total;
    long long row = active ? u / vec_per_row : 0;
    const long long c = active ? (u % vec_per_row) * 8 : 0;
    if (masked_m != nullptr && active) {
      const int e = masked_find(prefix, experts, (int)row);
      row = (long long)e * rows_per_expert + (row - prefix[e]);
    }
    float h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = 0.f;
    if (active) {
      float g[8], up[8];
      Vec8<T>::load(in + row * 2 * n + c, g);
      Vec8<T>::load(in + row * 2 * n + n + c, up);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float s = silu_fast(g[i]);
        if (round_silu) s = to_f32<T>(from_f32<T>(s));
        h[i] = to_f32<T>(from_f32<T>(s * up[i]));
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(h[i]));
    amax = group_max(amax, 16);
    const float scale = quant_scale(amax, mode, eps);
    if (!active) continue;
    *reinterpret_cast<uint2*>(q + row * n + c) = quant8_rcp(h, 1.0f / scale);
    if (((c / 8) & 15) == 0) scales[row * groups + c / 128] = scale;
  }
}

// One warp per token: the slots' ids are read once per warp (lane j holds slot j), rows nobody routed to cost
// one load, and the lanes sweep the row's columns together (512 contiguous bytes per load instruction).
template <typename T, typename IdT>
__global__ void __launch_bounds__(THREADS) sum_topk_kernel(const T* __restrict__ y, long long tokens, int top_k,
                                                           long long h, const IdT* __restrict__ ids, long long id_lo,
                                                           long long id_hi, int skip_unrouted, T* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (THREADS / 32);
  for (long long t = (long long)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5); t < tokens; t += warps) {
    unsigned live = 0xffffffffu;                       // bit j: slot j contributes
    if (ids != nullptr) {
      bool in_range = false;
      if (lane < top_k) {                              // top_k <= 32 (checked by the caller)
        const long long id = (long long)ids[t * top_k + lane];
        in_range = id >= id_lo && id < id_hi;
      }
      live = __ballot_sync(0xffffffffu, in_range);
    }
    if (top_k < 32) live &= (1u << top_k) - 1u;
    if (live == 0u && skip_unrouted) continue;         // rows nobody routed to are left alone
    for (long long c = (long long)lane * 8; c < h; c += 256) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int j = 0; j < top_k; ++j) {
        if (!((live >> j) & 1u)) continue;
        float v[8];
        Vec8<T>::load(y + (t * top_k + j) * h + c, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[i];
      }
      Vec8<T>::store(out + t * h + c, acc);
    }
  }
}

template <typename T, typename IdxT>
__global__ void __launch_bounds__(THREADS) ep_gather_kernel(const T* __restrict__ in, long long h,
                                                            const IdxT* __restrict__ ids, const IdxT* __restrict__ index,
                                                            const float* __restrict__ weights, long long tokens,
                                                            int top_k, T* __restrict__ out) {
  const long long vec_per_row = h / 8;
  const long long total = tokens * vec_per_row;
  for (long long u = (long long)blockIdx.x * THREADS + threadIdx.x; u < total; u += (long long)gridDim.x * THREADS) {
    const long long t = u / vec_per_row;
    const long long c = (u - t * vec_per_row) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j = 0; j < top_k; ++j) {
      if ((long long)ids[t * top_k + j] < 0) continue;
      const long long src = (long long)index[t * top_k + j];
      const float w = __ldg(weights + t * top_k + j);
      float v[8];
      Vec8<T>::load(in + src * h + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i] * w;
    }
    Vec8<T>::store(out + t * h + c, acc);
  }
}

// ep_scatter bookkeeping: exclusive cumsum of the (aligned) per-expert counts and the
// expert id of every row of the contiguous layout.
__global__ void __launch_bounds__(1024) scatter_layout_kernel(const int* __restrict__ counts, int num_experts,
                                                              int* __restrict__ start_loc, int* __restrict__ m_indices,
                                                              long long m_indices_len) {
  extern __shared__ int s_start[];  // [num_experts + 1]
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < num_experts; ++e) {
      s_start[e] = run;
      run += counts[e];
    }
    s_start[num_experts] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) start_loc[e] = s_start[e];
  for (int e = 0; e < num_experts; ++e) {
    const int b = s_start[e], t = s_start[e + 1];
    for (long long r = b + threadIdx.x; r < t && r < m_indices_len; r += blockDim.x) m_indices[r] = e;
  }
}

template <typename IdxT>
__global__ void __launch_bounds__(THREADS) scatter_index_kernel(const IdxT* __restrict__ ids, const int* __restrict__ rank,
                                                                const int* __restrict__ start_loc, long long slots,
                                                                IdxT* __restrict__ output_index, int* __restrict__ dst_pos) {
  for (long long f = (long long)blockIdx.x * THREADS + threadIdx.x; f < slots; f += (long long)gridDim.x * THREADS) {
    const long long e = (long long)ids[f];
    int d = -1;
    if (e >= 0) {
      d = start_loc[e] + rank[f];
      output_index[f] = (IdxT)d;   // slots with id < 0 keep their previous content, as in the reference
    }
    dst_pos[f] = d;
  }
}

template <typename IdxT>
__global__ void __launch_bounds__(THREADS) dest_ranks_kernel(const IdxT* __restrict__ ids, long long tokens, int top_k,
                                                             int num_local, int world, int* __restrict__ dest) {
  const long long total = tokens * world;
  for (long long u = (long long)blockIdx.x * THREADS + threadIdx.x; u < total; u += (long long)gridDim.x * THREADS) {
    const long long t = u / world;
    const int r = (int)(u - t * world);
    bool hit = false;
    for (int j = 0; j < top_k; ++j) {
      const long long id = (long long)ids[t * top_k + j];
      hit = hit || (id >= 0 && id / num_local == r);
    }
    dest[u] = hit ? r : world;
  }
}

int grid_for(long long total_threads) {
  long long blocks = ceil_div(total_threads, THREADS);
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// ---- training-side un-permute (dlblas/kernels/permute/moe_triton_kernels.py) -----------------
// out[t] = sum over k of prob[t, k] * in[row_id_map[k * T + t]] (entries -1 skipped), accumulated in
// the tensor's own type with a rounding after every product and every add, as gather_kernel
// (:229-271) does.  Without probs it is the plain sum of permute's backward (:140-167).
template <typename T>
__global__ void __launch_bounds__(THREADS) unpermute_kernel(const T* __restrict__ in, const int* __restrict__ row_id_map,
                                                            const float* __restrict__ probs, long long tokens,
                                                            int top_k, long long h, T* __restrict__ out) {
  const long long vec_per_row = h / 8;
  const long long total = tokens * vec_per_row;
  for (long long u = (long long)blockIdx.x * THREADS + threadIdx.x; u < total; u += (long long)gridDim.x * THREADS) {
    const long long t = u / vec_per_row;
    const long long c = (u - t * vec_per_row) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    bool first = true;
    for (int j = 0; j < top_k; ++j) {
      const int row = __ldg(row_id_map + (long long)j * tokens + t);
      if (row < 0) {
        if (j == 0) first = false;      // the reference starts from zeros when slot 0 is unrouted
        continue;
      }
      float v[8];
      Vec8<T>::load(in + (long long)row * h + c, v);
      if (probs != nullptr) {
        const float p = to_f32<T>(from_f32<T>(__ldg(probs + t * top_k + j)));
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = to_f32<T>(from_f32<T>(v[i] * p));
      }
      if (j == 0 && first) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = v[i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = to_f32<T>(from_f32<T>(acc[i] + v[i]));
      }
    }
    Vec8<T>::store(out + t * h + c, acc);
  }
}

// Backward of the weighted un-permute (scatter_bwd_kernel_optimized, :427-478): one warp per token;
// act_grad[row] = grad_out[t] * prob[t, k] (product in the tensors' type, stored as fp32),
// prob_grad[t, k] = sum over columns of the type-rounded products grad_out[t] * fwd_in[row], in fp32.
template <typename T>
__global__ void __launch_bounds__(THREADS) unpermute_bwd_kernel(const T* __restrict__ grad_out,
                                                                const T* __restrict__ fwd_in,
                                                                const int* __restrict__ row_id_map,
                                                                const float* __restrict__ probs, long long tokens,
                                                                int top_k, long long h, float* __restrict__ act_grad,
                                                                float* __restrict__ prob_grad) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  for (int j = 0; j < top_k; ++j) {
    const int row = __ldg(row_id_map + (long long)j * tokens + t);
    float dot = 0.f;
    if (row >= 0) {
      const float p = to_f32<T>(from_f32<T>(__ldg(probs + t * top_k + j)));
      for (long long c = lane * 8; c < h; c += 256) {
        float go[8], fw[8];
        Vec8<T>::load(grad_out + t * h + c, go);
        Vec8<T>::load(fwd_in + (long long)row * h + c, fw);
        float ag[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          ag[i] = to_f32<T>(from_f32<T>(go[i] * p));
          dot += to_f32<T>(from_f32<T>(go[i] * fw[i]));
        }
        Vec8<float>::store(act_grad + (long long)row * h + c, ag);
      }
    }
    dot = warp_sum(dot);
    if (lane == 0) prob_grad[t * top_k + j] = dot;
  }
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" int dlb_quant_fp8(const void* x, int x_dtype, int64_t m, int64_t k, int64_t ldx, int group_size, int mode,
                             float eps, void* q, float* scales, int64_t scale_row_stride, int64_t scale_group_stride,
                             const int32_t* dst_pos, int fanout, void* stream) {
  DLB_REQUIRE(m >= 0 && k > 0, DLB_ERR_INVALID, "quant_fp8: bad sizes m=%lld k=%lld", (long long)m, (long long)k);
  DLB_REQUIRE(group_size == 32 || group_size == 64 || group_size == 128 || group_size == 256, DLB_ERR_INVALID,
              "quant_fp8: group_size %d not supported (32, 64, 128, 256)", group_size);
  DLB_REQUIRE(k % group_size == 0, DLB_ERR_INVALID, "quant_fp8: k=%lld is not a multiple of group_size=%d",
              (long long)k, group_size);
  DLB_REQUIRE(mode == DLB_QUANT_RECIP_MUL || mode == DLB_QUANT_DIV_EPS, DLB_ERR_INVALID, "quant_fp8: bad mode %d", mode);
  DLB_REQUIRE(dst_pos == nullptr || fanout > 0, DLB_ERR_INVALID, "quant_fp8: fanout must be positive with dst_pos");
  if (m == 0) return DLB_OK;
  DLB_REQUIRE(x && q && scales, DLB_ERR_INVALID, "quant_fp8: null pointer");
  const int esz = x_dtype == DLB_F32 ? 4 : 2;
  DLB_REQUIRE((uintptr_t)x % 16 == 0 && (ldx * esz) % 16 == 0 && (uintptr_t)q % 8 == 0, DLB_ERR_INVALID,
              "quant_fp8: x rows must be 16-byte aligned and q 8-byte aligned");
  const int grid = grid_for(m * (k / 8));
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* qq = reinterpret_cast<uint8_t*>(q);
  if (x_dtype == DLB_BF16)
    quant_fp8_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), m, k, ldx,
                                                             group_size, mode, eps, qq, scales, scale_row_stride,
                                                             scale_group_stride, dst_pos, fanout);
  else if (x_dtype == DLB_F16)
    quant_fp8_kernel<__half><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __half*>(x), m, k, ldx, group_size, mode,
                                                      eps, qq, scales, scale_row_stride, scale_group_stride, dst_pos,
                                                      fanout);
  else if (x_dtype == DLB_F32)
    quant_fp8_kernel<float><<<grid, THREADS, 0, st>>>(reinterpret_cast<const float*>(x), m, k, ldx, group_size, mode,
                                                     eps, qq, scales, scale_row_stride, scale_group_stride, dst_pos,
                                                     fanout);
  else
    return fail(DLB_ERR_INVALID, "quant_fp8: unsupported input dtype %d", x_dtype);
  count_launch();
  DLB_CHECK_LAUNCH("quant_fp8_kernel");
  return DLB_OK;
}

extern "C" int dlb_permute_rows(const void* q, int64_t row_bytes, const float* scales, int64_t groups, int64_t m,
                                const int32_t* dst_pos, int fanout, void* out_q, float* out_scales, void* stream) {
  DLB_REQUIRE(m >= 0 && row_bytes > 0 && row_bytes % 16 == 0, DLB_ERR_INVALID,
              "permute_rows: row_bytes=%lld must be a positive multiple of 16", (long long)row_bytes);
  DLB_REQUIRE(groups >= 0 && groups <= row_bytes / 16, DLB_ERR_INVALID, "permute_rows: too many scale groups per row");
  DLB_REQUIRE(fanout > 0, DLB_ERR_INVALID, "permute_rows: fanout must be positive");
  if (m == 0) return DLB_OK;
  DLB_REQUIRE(q && dst_pos && out_q && (scales == nullptr || out_scales != nullptr), DLB_ERR_INVALID,
              "permute_rows: null pointer");
  DLB_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)out_q % 16 == 0, DLB_ERR_INVALID,
              "permute_rows: q and out_q must be 16-byte aligned");
  const long long vpr = row_bytes / 16;
  permute_rows_kernel<<<grid_for(m * vpr), THREADS, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(q), vpr, scales, groups, m, dst_pos, fanout, reinterpret_cast<uint4*>(out_q),
      out_scales);
  count_launch();
  DLB_CHECK_LAUNCH("permute_rows_kernel");
  return DLB_OK;
}

extern "C" int dlb_silu_and_mul(const void* gate_up, int dtype, int64_t rows, int64_t n, int64_t ld_in, void* out,
                                int64_t ld_out, void* stream) {
  DLB_REQUIRE(rows >= 0 && n > 0 && n % 8 == 0, DLB_ERR_INVALID, "silu_and_mul: n=%lld must be a positive multiple of 8",
              (long long)n);
  if (rows == 0) return DLB_OK;
  DLB_REQUIRE(gate_up && out, DLB_ERR_INVALID, "silu_and_mul: null pointer");
  const int esz = dtype == DLB_F32 ? 4 : 2;
  DLB_REQUIRE((uintptr_t)gate_up % 16 == 0 && (uintptr_t)out % 16 == 0 && (ld_in * esz) % 16 == 0 &&
                  (ld_out * esz) % 16 == 0 && (n * esz) % 16 == 0,
              DLB_ERR_INVALID, "silu_and_mul: rows must be 16-byte aligned");
  const int grid = grid_for(rows * (n / 8));
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == DLB_BF16)
    silu_and_mul_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(gate_up), rows,
                                                                n, ld_in, reinterpret_cast<__nv_bfloat16*>(out), ld_out);
  else if (dtype == DLB_F16)
    silu_and_mul_kernel<__half><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __half*>(gate_up), rows, n, ld_in,
                                                         reinterpret_cast<__half*>(out), ld_out);
  else if (dtype == DLB_F32)
    silu_and_mul_kernel<float><<<grid, THREADS, 0, st>>>(reinterpret_cast<const float*>(gate_up), rows, n, ld_in,
                                                        reinterpret_cast<float*>(out), ld_out);
  else
    return fail(DLB_ERR_INVALID, "silu_and_mul: unsupported dtype %d", dtype);
  count_launch();
  DLB_CHECK_LAUNCH("silu_and_mul_kernel");
  return DLB_OK;
}

extern "C" int dlb_silu_mul_quant(const void* gate_up, int dtype, int64_t rows, int64_t n, int quant_mode, float eps,
                                  int round_silu, const int32_t* masked_m, int64_t rows_per_expert, void* q,
                                  float* scales, void* stream) {
  DLB_REQUIRE(rows >= 0 && n > 0 && n % 128 == 0, DLB_ERR_INVALID,
              "silu_mul_quant: n=%lld must be a positive multiple of 128", (long long)n);
  DLB_REQUIRE(quant_mode == DLB_QUANT_RECIP_MUL || quant_mode == DLB_QUANT_DIV_EPS, DLB_ERR_INVALID,
              "silu_mul_quant: bad mode %d", quant_mode);
  DLB_REQUIRE(masked_m == nullptr || rows_per_expert > 0, DLB_ERR_INVALID, "silu_mul_quant: rows_per_expert needed");
  if (rows == 0) return DLB_OK;
  DLB_REQUIRE(gate_up && q && scales, DLB_ERR_INVALID, "silu_mul_quant: null pointer");
  DLB_REQUIRE((uintptr_t)gate_up % 16 == 0 && (uintptr_t)q % 8 == 0, DLB_ERR_INVALID, "silu_mul_quant: misaligned");
  int grid = grid_for(rows * (n / 8));
  int experts = 0;
  if (masked_m != nullptr) {
    DLB_REQUIRE(rows % rows_per_expert == 0 && rows / rows_per_expert <= MASKED_MAX_EXPERTS, DLB_ERR_INVALID,
                "silu_mul_quant: rows=%lld must be a whole number (at most %d) of experts of %lld rows", (long long)rows,
                MASKED_MAX_EXPERTS, (long long)rows_per_expert);
    experts = (int)(rows / rows_per_expert);
    grid = min(grid, 4 * sm_count());   // the valid rows are few; every block pays for the running sums
  }
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* qq = reinterpret_cast<uint8_t*>(q);
  if (dtype == DLB_BF16)
    silu_mul_quant_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(gate_up), rows,
                                                                  n, quant_mode, eps, round_silu, masked_m,
                                                                  experts, rows_per_expert, qq, scales);
  else if (dtype == DLB_F16)
    silu_mul_quant_kernel<__half><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __half*>(gate_up), rows, n, quant_mode,
                                                           eps, round_silu, masked_m, experts, rows_per_expert, qq, scales);
  else
    return fail(DLB_ERR_INVALID, "silu_mul_quant: unsupported dtype %d (bf16 / fp16)", dtype);
  count_launch();
  DLB_CHECK_LAUNCH("silu_mul_quant_kernel");
  return DLB_OK;
}

namespace {
template <typename T>
int launch_sum_topk(const void* y, int64_t tokens, int top_k, int64_t h, const void* ids, int ids_dtype, int64_t lo,
                    int64_t hi, int skip, void* out, cudaStream_t st) {
  const int grid = grid_for(tokens * 32);          // one warp per token
  if (ids != nullptr && ids_dtype == DLB_I32)
    sum_topk_kernel<T, int><<<grid, THREADS, 0, st>>>(reinterpret_cast<const T*>(y), tokens, top_k, h,
                                                     reinterpret_cast<const int*>(ids), lo, hi, skip,
                                                     reinterpret_cast<T*>(out));
  else
    sum_topk_kernel<T, long long><<<grid, THREADS, 0, st>>>(reinterpret_cast<const T*>(y), tokens, top_k, h,
                                                           reinterpret_cast<const long long*>(ids), lo, hi, skip,
                                                           reinterpret_cast<T*>(out));
  count_launch();
  DLB_CHECK_LAUNCH("sum_topk_kernel");
  return DLB_OK;
}
}  // namespace

extern "C" int dlb_moe_sum_topk(const void* y, int dtype, int64_t tokens, int top_k, int64_t h, const void* ids,
                                int ids_dtype, int64_t id_lo, int64_t id_hi, int skip_unrouted_rows, void* out,
                                void* stream) {
  DLB_REQUIRE(tokens >= 0 && top_k > 0 && top_k <= 32 && h > 0 && h % 8 == 0, DLB_ERR_INVALID,
              "sum_topk: h=%lld must be a positive multiple of 8 and top_k=%d at most 32", (long long)h, top_k);
  DLB_REQUIRE(ids == nullptr || ids_dtype == DLB_I32 || ids_dtype == DLB_I64, DLB_ERR_INVALID,
              "sum_topk: ids must be int32/int64");
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(y && out, DLB_ERR_INVALID, "sum_topk: null pointer");
  DLB_REQUIRE((uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0, DLB_ERR_INVALID, "sum_topk: misaligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int skip = (ids != nullptr && skip_unrouted_rows) ? 1 : 0;
  if (dtype == DLB_BF16)
    return launch_sum_topk<__nv_bfloat16>(y, tokens, top_k, h, ids, ids_dtype, id_lo, id_hi, skip, out, st);
  if (dtype == DLB_F16) return launch_sum_topk<__half>(y, tokens, top_k, h, ids, ids_dtype, id_lo, id_hi, skip, out, st);
  if (dtype == DLB_F32) return launch_sum_topk<float>(y, tokens, top_k, h, ids, ids_dtype, id_lo, id_hi, skip, out, st);
  return fail(DLB_ERR_INVALID, "sum_topk: unsupported dtype %d", dtype);
}

namespace {
template <typename T>
int launch_gather(const void* in, int64_t h, const void* ids, const void* index, int idx_dtype, const float* weights,
                  int64_t tokens, int top_k, void* out, cudaStream_t st) {
  const int grid = grid_for(tokens * (h / 8));
  if (idx_dtype == DLB_I32)
    ep_gather_kernel<T, int><<<grid, THREADS, 0, st>>>(reinterpret_cast<const T*>(in), h,
                                                      reinterpret_cast<const int*>(ids),
                                                      reinterpret_cast<const int*>(index), weights, tokens, top_k,
                                                      reinterpret_cast<T*>(out));
  else
    ep_gather_kernel<T, long long><<<grid, THREADS, 0, st>>>(reinterpret_cast<const T*>(in), h,
                                                            reinterpret_cast<const long long*>(ids),
                                                            reinterpret_cast<const long long*>(index), weights, tokens,
                                                            top_k, reinterpret_cast<T*>(out));
  count_launch();
  DLB_CHECK_LAUNCH("ep_gather_kernel");
  return DLB_OK;
}
}  // namespace

extern "C" int dlb_ep_gather(const void* in, int dtype, int64_t h, const void* ids, const void* index, int idx_dtype,
                             const float* weights, int64_t tokens, int top_k, void* out, void* stream) {
  DLB_REQUIRE(tokens >= 0 && top_k > 0 && h > 0 && h % 8 == 0, DLB_ERR_INVALID,
              "ep_gather: h=%lld must be a positive multiple of 8", (long long)h);
  DLB_REQUIRE(idx_dtype == DLB_I32 || idx_dtype == DLB_I64, DLB_ERR_INVALID, "ep_gather: ids must be int32/int64");
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(in && ids && index && weights && out, DLB_ERR_INVALID, "ep_gather: null pointer");
  DLB_REQUIRE((uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0, DLB_ERR_INVALID, "ep_gather: misaligned");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == DLB_BF16) return launch_gather<__nv_bfloat16>(in, h, ids, index, idx_dtype, weights, tokens, top_k, out, st);
  if (dtype == DLB_F16) return launch_gather<__half>(in, h, ids, index, idx_dtype, weights, tokens, top_k, out, st);
  if (dtype == DLB_F32) return launch_gather<float>(in, h, ids, index, idx_dtype, weights, tokens, top_k, out, st);
  return fail(DLB_ERR_INVALID, "ep_gather: unsupported dtype %d", dtype);
}

namespace {
size_t align256(size_t v) { return (v + 255) / 256 * 256; }
}

extern "C" size_t dlb_ep_scatter_workspace_size(int64_t tokens, int top_k, int num_experts) {
  if (tokens <= 0 || top_k <= 0 || num_experts <= 0) return 0;
  const long long slots = tokens * top_k;
  return align256((size_t)slots * 4) * 2 + sort_workspace_size(slots, num_experts);
}

extern "C" int dlb_ep_scatter(const void* x, int64_t row_bytes, const float* x_scale, int64_t groups, const void* ids,
                              int idx_dtype, int64_t tokens, int top_k, const int32_t* counts, int num_experts,
                              int32_t* expert_start_loc, void* out_x, float* out_scale, int32_t* m_indices,
                              int64_t m_indices_len, void* output_index, void* workspace, size_t workspace_bytes,
                              void* stream) {
  DLB_REQUIRE(tokens >= 0 && top_k > 0 && num_experts > 0 && num_experts <= 8192, DLB_ERR_INVALID,
              "ep_scatter: bad sizes");
  DLB_REQUIRE(idx_dtype == DLB_I32 || idx_dtype == DLB_I64, DLB_ERR_INVALID, "ep_scatter: ids must be int32/int64");
  DLB_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, DLB_ERR_INVALID, "ep_scatter: row_bytes must be a multiple of 16");
  DLB_REQUIRE(counts && expert_start_loc && m_indices, DLB_ERR_INVALID, "ep_scatter: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  scatter_layout_kernel<<<1, 1024, (size_t)(num_experts + 1) * 4, st>>>(counts, num_experts, expert_start_loc, m_indices,
                                                                        m_indices_len);
  count_launch();
  DLB_CHECK_LAUNCH("scatter_layout_kernel");
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(x && ids && out_x && output_index, DLB_ERR_INVALID, "ep_scatter: null pointer");
  const long long slots = tokens * top_k;
  const size_t need = dlb_ep_scatter_workspace_size(tokens, top_k, num_experts);
  DLB_REQUIRE(workspace != nullptr && workspace_bytes >= need, DLB_ERR_WORKSPACE,
              "ep_scatter: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  char* ws = reinterpret_cast<char*>(workspace);
  int* rank = reinterpret_cast<int*>(ws);
  int* dst_pos = reinterpret_cast<int*>(ws + align256((size_t)slots * 4));
  void* sort_ws = ws + 2 * align256((size_t)slots * 4);
  int rc = sort_by_expert(ids, idx_dtype, slots, num_experts, nullptr, nullptr, nullptr, nullptr, rank, nullptr, sort_ws,
                          workspace_bytes - 2 * align256((size_t)slots * 4), st);
  if (rc != DLB_OK) return rc;
  if (idx_dtype == DLB_I32)
    scatter_index_kernel<int><<<grid_for(slots), THREADS, 0, st>>>(reinterpret_cast<const int*>(ids), rank,
                                                                  expert_start_loc, slots,
                                                                  reinterpret_cast<int*>(output_index), dst_pos);
  else
    scatter_index_kernel<long long><<<grid_for(slots), THREADS, 0, st>>>(reinterpret_cast<const long long*>(ids), rank,
                                                                        expert_start_loc, slots,
                                                                        reinterpret_cast<long long*>(output_index),
                                                                        dst_pos);
  count_launch();
  DLB_CHECK_LAUNCH("scatter_index_kernel");
  return dlb_permute_rows(x, row_bytes, x_scale, groups, tokens, dst_pos, top_k, out_x, out_scale, stream);
}

extern "C" int dlb_ep_dest_ranks(const void* ids, int ids_dtype, int64_t tokens, int top_k, int num_local_experts,
                                 int world, int32_t* dest, void* stream) {
  DLB_REQUIRE(tokens >= 0 && top_k > 0 && num_local_experts > 0 && world > 0, DLB_ERR_INVALID, "ep_dest_ranks: bad sizes");
  DLB_REQUIRE(ids_dtype == DLB_I32 || ids_dtype == DLB_I64, DLB_ERR_INVALID, "ep_dest_ranks: ids must be int32/int64");
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(ids && dest, DLB_ERR_INVALID, "ep_dest_ranks: null pointer");
  const int grid = grid_for(tokens * world);
  cudaStream_t st = (cudaStream_t)stream;
  if (ids_dtype == DLB_I32)
    dest_ranks_kernel<int><<<grid, THREADS, 0, st>>>(reinterpret_cast<const int*>(ids), tokens, top_k, num_local_experts,
                                                    world, dest);
  else
    dest_ranks_kernel<long long><<<grid, THREADS, 0, st>>>(reinterpret_cast<const long long*>(ids), tokens, top_k,
                                                          num_local_experts, world, dest);
  count_launch();
  DLB_CHECK_LAUNCH("dest_ranks_kernel");
  return DLB_OK;
}

extern "C" int dlb_unpermute(const void* in, int dtype, const int32_t* row_id_map, const float* probs, int64_t tokens,
                             int top_k, int64_t h, void* out, void* stream) {
  DLB_REQUIRE(tokens >= 0 && top_k > 0 && h > 0 && h % 8 == 0, DLB_ERR_INVALID,
              "unpermute: bad sizes tokens=%lld top_k=%d h=%lld (h must be a multiple of 8)", (long long)tokens, top_k,
              (long long)h);
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(in && row_id_map && out, DLB_ERR_INVALID, "unpermute: null pointer");
  DLB_REQUIRE((uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0, DLB_ERR_INVALID, "unpermute: misaligned tensors");
  const long long total = tokens * (h / 8);
  const int grid = (int)std::min<long long>(ceil_div(total, (long long)THREADS), (long long)sm_count() * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == DLB_BF16)
    unpermute_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(in), row_id_map,
                                                             probs, tokens, top_k, h,
                                                             reinterpret_cast<__nv_bfloat16*>(out));
  else if (dtype == DLB_F16)
    unpermute_kernel<__half><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __half*>(in), row_id_map, probs, tokens,
                                                      top_k, h, reinterpret_cast<__half*>(out));
  else if (dtype == DLB_F32)
    unpermute_kernel<float><<<grid, THREADS, 0, st>>>(reinterpret_cast<const float*>(in), row_id_map, probs, tokens,
                                                     top_k, h, reinterpret_cast<float*>(out));
  else
    return fail(DLB_ERR_INVALID, "unpermute: unsupported dtype %d", dtype);
  count_launch();
  DLB_CHECK_LAUNCH("unpermute_kernel");
  return DLB_OK;
}

extern "C" int dlb_unpermute_bwd(const void* grad_out, const void* fwd_in, int dtype, const int32_t* row_id_map,
                                 const float* probs, int64_t tokens, int top_k, int64_t h, float* act_grad,
                                 float* prob_grad, void* stream) {
  DLB_REQUIRE(tokens >= 0 && top_k > 0 && h > 0 && h % 8 == 0, DLB_ERR_INVALID,
              "unpermute_bwd: bad sizes tokens=%lld top_k=%d h=%lld", (long long)tokens, top_k, (long long)h);
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(grad_out && fwd_in && row_id_map && probs && act_grad && prob_grad, DLB_ERR_INVALID,
              "unpermute_bwd: null pointer");
  DLB_REQUIRE((uintptr_t)grad_out % 16 == 0 && (uintptr_t)fwd_in % 16 == 0 && (uintptr_t)act_grad % 16 == 0,
              DLB_ERR_INVALID, "unpermute_bwd: misaligned tensors");
  const int grid = (int)ceil_div(tokens, (long long)(THREADS / 32));
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == DLB_BF16)
    unpermute_bwd_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(grad_out), reinterpret_cast<const __nv_bfloat16*>(fwd_in), row_id_map,
        probs, tokens, top_k, h, act_grad, prob_grad);
  else if (dtype == DLB_F16)
    unpermute_bwd_kernel<__half><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __half*>(grad_out),
                                                          reinterpret_cast<const __half*>(fwd_in), row_id_map, probs,
                                                          tokens, top_k, h, act_grad, prob_grad);
  else if (dtype == DLB_F32)
    unpermute_bwd_kernel<float><<<grid, THREADS, 0, st>>>(reinterpret_cast<const float*>(grad_out),
                                                         reinterpret_cast<const float*>(fwd_in), row_id_map, probs,
                                                         tokens, top_k, h, act_grad, prob_grad);
  else
    return fail(DLB_ERR_INVALID, "unpermute_bwd: unsupported dtype %d", dtype);
  count_launch();
  DLB_CHECK_LAUNCH("unpermute_bwd_kernel");
  return DLB_OK;
}
