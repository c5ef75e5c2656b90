// Shared helpers of the dlblas_b200 CUDA extension (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/dlblas_b200.h"

namespace dlb {

// Records the message returned by dlb_last_error_string() (thread local) and
// hands back the code so call sites can `return fail(...)`.
int fail(int code, const char* fmt, ...);

inline int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return DLB_OK;
  return fail(DLB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

int sm_count();  // multiprocessors of the current device (cached per device)
void count_launch();  // bumps the per-thread kernel launch counter read by dlb_launch_count()
// limit of one barrier wait in SM clock cycles: the value given to dlb_set_wait_policy(), else `fallback`
unsigned long long wait_limit_cycles(unsigned long long fallback);
bool withhold_loads();  // dlb_set_wait_policy(): the GEMMs' load role issues nothing (makes the waits run out)

#define DLB_CHECK_LAUNCH(name)                                  \
  do {                                                          \
    cudaError_t e__ = cudaGetLastError();                       \
    if (e__ != cudaSuccess) return dlb::check_cuda(e__, name);  \
  } while (0)

#define DLB_REQUIRE(cond, code, ...)                 \
  do {                                               \
    if (!(cond)) return dlb::fail(code, __VA_ARGS__); \
  } while (0)

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Masked layouts ([experts, rows_per_expert, ...] with only the first masked_m[e] rows of expert e in use) hold a few
// hundred valid rows among tens of thousands in a decode step.  These two helpers let a kernel walk the valid rows only:
// every block builds the running sums of min(masked_m[e], cap) in shared memory (prefix[experts] = their total; warp 0
// scans, all threads of the block must call), then item i of [0, total) is row i - prefix[e] of expert e.
constexpr int MASKED_MAX_EXPERTS = 1024;
#ifdef __CUDACC__
__device__ inline void masked_prefix(const int* __restrict__ masked_m, int experts, int cap, int* prefix) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int carry = 0;
    for (int e0 = 0; e0 < experts; e0 += 32) {
      const int e = e0 + lane;
      const int v = e < experts ? min(max(__ldg(masked_m + e), 0), cap) : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
      }
      if (e < experts) prefix[e] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) prefix[experts] = carry;
  }
  __syncthreads();
}
// the expert that holds item `item` (< prefix[experts]): the last e with prefix[e] <= item
__device__ inline int masked_find(const int* prefix, int experts, int item) {
  int lo = 0, hi = experts;   // invariant: prefix[lo] <= item < prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= item) lo = mid; else hi = mid;
  }
  return lo;
}
#endif

// ---- warp helpers -------------------------------------------------------- //
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- element conversion ---------------------------------------------------- //
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// The reference clamps before it casts (`tl.clamp(out, fp8_min, fp8_max)`, dlblas/kernels/moe.py:413,
// dlblas/kernels/fp8.py:48): min(max(x, -448), 448) with the non-propagating min / max of the GPU, so a NaN
// (0 / 0 of an all-zero group whose scale is 0) becomes -448 and never reaches the payload.  fmaxf / fminf
// return the non-NaN operand, which reproduces that.
__device__ __forceinline__ float clamp_e4m3(float x) { return fminf(fmaxf(x, -448.f), 448.f); }

// Two fp32 -> packed e4m3x2 (lo in bits 0-7): clamp to +-448, then round to nearest even.
__device__ __forceinline__ uint16_t f32x2_to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(clamp_e4m3(hi)), "f"(clamp_e4m3(lo)));
  return r;
}

// silu for the fused silu*up + quantise paths: fast exponential and a 2-ulp divide.  The result
// is multiplied by `up` and rounded to a 16-bit type straight away, so the extra fp32 error only
// shows where the product sits within 2 ulp of a 16-bit rounding boundary.
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.f + __expf(-g)); }

// Eight values times the reciprocal of their group's scale -> eight e4m3 bytes.  `inv` is the
// correctly rounded 1 / scale; v * inv is within one fp32 ulp of v / scale.
__device__ __forceinline__ uint2 quant8_rcp(const float (&v)[8], float inv) {
  uint2 r;
  r.x = (uint32_t)f32x2_to_e4m3x2(v[0] * inv, v[1] * inv) | ((uint32_t)f32x2_to_e4m3x2(v[2] * inv, v[3] * inv) << 16);
  r.y = (uint32_t)f32x2_to_e4m3x2(v[4] * inv, v[5] * inv) | ((uint32_t)f32x2_to_e4m3x2(v[6] * inv, v[7] * inv) << 16);
  return r;
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

}  // namespace dlb
