// Expert-parallel dispatch / combine by direct stores into the peers' memory (NVLink / NVSwitch).
//
// Every rank owns a receive buffer of W regions (one per source rank) of `region_rows` rows.
// The dispatch kernel quantises a token once and stores its FP8 row, scales and routing
// metadata straight into the region "my rank" of every destination rank that owns one of its
// experts: the all-to-all is fused with the quantiser and with the permutation, no staging
// buffer, no host-side split sizes.  The combine kernel pushes result rows back the same way.
// Cross-rank ordering (a barrier after each push phase) is done by the caller on the stream.
// Only plain 16-byte global stores through peer pointers are used.
#include "common.cuh"

namespace dlb {
namespace {

constexpr int THREADS = 256;
constexpr int MAX_WORLD = 16;

struct PeerPtrs {
  void* p[MAX_WORLD];
};

__device__ __forceinline__ void load8_bf16(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8_f16(const __half* p, float (&v)[8]) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// One thread per 8 elements of a token row (16 lanes per 128-wide group), as in the local
// quantiser; `within[t * world + r]` is the row of token t inside my region on rank r (< 0:
// rank r gets nothing from this token).
template <bool IS_BF16>
__global__ void __launch_bounds__(THREADS) quant_push_kernel(const void* __restrict__ x, long long tokens, long long k,
                                                             long long ldx, int mode, float eps,
                                                             const int* __restrict__ within, int world, int my_rank,
                                                             long long region_rows, PeerPtrs peer_q, PeerPtrs peer_s,
                                                             PeerPtrs peer_meta, const int* __restrict__ meta,
                                                             int meta_ints, PeerPtrs peer_counts,
                                                             const int* __restrict__ counts) {
  const long long vec_per_row = k / 8;
  const long long total = tokens * vec_per_row;
  const long long groups = k / 128;
  if (blockIdx.x == 0 && threadIdx.x < world)
    reinterpret_cast<int*>(peer_counts.p[threadIdx.x])[my_rank] = counts[threadIdx.x];
  for (long long u0 = (long long)blockIdx.x * THREADS; u0 < total; u0 += (long long)gridDim.x * THREADS) {
    const long long u = u0 + threadIdx.x;
    const bool active = u < total;
    const long long row = active ? u / vec_per_row : 0;
    const long long c = active ? (u - row * vec_per_row) * 8 : 0;
    float v[8];
    if (active) {
      if (IS_BF16) load8_bf16(reinterpret_cast<const __nv_bfloat16*>(x) + row * ldx + c, v);
      else load8_f16(reinterpret_cast<const __half*>(x) + row * ldx + c, v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = mode == DLB_QUANT_RECIP_MUL ? amax * (1.0f / 448.0f) : fmaxf(amax, eps) / 448.0f;
    if (!active) continue;
    uint2 packed;
    packed.x = (uint32_t)f32x2_to_e4m3x2(v[0] / scale, v[1] / scale) |
               ((uint32_t)f32x2_to_e4m3x2(v[2] / scale, v[3] / scale) << 16);
    packed.y = (uint32_t)f32x2_to_e4m3x2(v[4] / scale, v[5] / scale) |
               ((uint32_t)f32x2_to_e4m3x2(v[6] / scale, v[7] / scale) << 16);
    const bool first = ((c / 8) & 15) == 0;
    for (int r = 0; r < world; ++r) {
      const int j = __ldg(within + row * world + r);
      if (j < 0) continue;
      const long long drow = (long long)my_rank * region_rows + j;
      *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(peer_q.p[r]) + drow * k + c) = packed;
      if (first) reinterpret_cast<float*>(peer_s.p[r])[drow * groups + c / 128] = scale;
      if (c == 0) {
        int* dm = reinterpret_cast<int*>(peer_meta.p[r]) + drow * meta_ints;
        for (int i = 0; i < meta_ints; ++i) dm[i] = __ldg(meta + row * meta_ints + i);
      }
    }
  }
}

// Receiver side: turns the metadata rows into local expert ids (-1: not a local expert or an
// unused row of the region) and weights.
__global__ void __launch_bounds__(THREADS) unpack_meta_kernel(const int* __restrict__ meta, int meta_ints, int top_k,
                                                              int kp, const int* __restrict__ counts, int world,
                                                              long long region_rows, int expert_lo, int num_local,
                                                              long long* __restrict__ ids, float* __restrict__ weights) {
  const long long total = (long long)world * region_rows * top_k;
  for (long long u = (long long)blockIdx.x * THREADS + threadIdx.x; u < total; u += (long long)gridDim.x * THREADS) {
    const long long row = u / top_k;
    const int j = (int)(u - row * top_k);
    const int src = (int)(row / region_rows);
    const bool used = (row - (long long)src * region_rows) < counts[src];
    long long id = -1;
    float w = 0.f;
    if (used) {
      const int g = meta[row * meta_ints + j];
      if (g >= expert_lo && g < expert_lo + num_local) id = g - expert_lo;
      w = __int_as_float(meta[row * meta_ints + kp + j]);
    }
    ids[u] = id;
    weights[u] = w;
  }
}

// Pushes the used rows of each region back to the rank they came from: row j of region s goes to
// rank s, region "my rank", row j.
__global__ void __launch_bounds__(THREADS) push_rows_kernel(const uint4* __restrict__ src, long long vec_per_row,
                                                            const int* __restrict__ counts, int world, int my_rank,
                                                            long long region_rows, PeerPtrs peer_dst) {
  const long long total = (long long)world * region_rows * vec_per_row;
  for (long long u = (long long)blockIdx.x * THREADS + threadIdx.x; u < total; u += (long long)gridDim.x * THREADS) {
    const long long row = u / vec_per_row;
    const long long c = u - row * vec_per_row;
    const int s = (int)(row / region_rows);
    const long long j = row - (long long)s * region_rows;
    if (j >= counts[s]) continue;
    reinterpret_cast<uint4*>(peer_dst.p[s])[((long long)my_rank * region_rows + j) * vec_per_row + c] = __ldg(src + u);
  }
}

// Combine step of the expert side, fused with the push: for every received row (row j of region s, j < counts[s])
// the results of its slots on local experts are summed in fp32 in slot order, rounded to bf16 / fp16 and stored
// straight into the source rank's combine buffer (region "my rank", row j).  One warp per row; ids are the
// local expert ids of the row's slots (negative = another rank's expert).
template <typename T>
__global__ void __launch_bounds__(THREADS) sum_push_kernel(const T* __restrict__ y, const long long* __restrict__ ids,
                                                           int top_k, long long h, const int* __restrict__ counts,
                                                           int world, int my_rank, long long region_rows,
                                                           PeerPtrs peer_dst, long long col_begin, long long col_end) {
  const int lane = threadIdx.x & 31;
  const long long rows = (long long)world * region_rows;
  const long long warps = (long long)gridDim.x * (THREADS / 32);
  for (long long r = (long long)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
    const int s = (int)(r / region_rows);
    const long long j = r - (long long)s * region_rows;
    if (j >= counts[s]) continue;
    const bool mine = lane < top_k && ids[r * top_k + lane] >= 0;
    const unsigned live = __ballot_sync(0xffffffffu, mine);
    T* dst = reinterpret_cast<T*>(peer_dst.p[s]) + ((long long)my_rank * region_rows + j) * h;
    for (long long c = col_begin + (long long)lane * 8; c < col_end; c += 256) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int q = 0; q < top_k; ++q) {
        if (!((live >> q) & 1u)) continue;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(y + (r * top_k + q) * h + c));
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += to_f32<T>(v[i]);
      }
      uint4 out;
      T* o = reinterpret_cast<T*>(&out);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = from_f32<T>(acc[i]);
      *reinterpret_cast<uint4*>(dst + c) = out;
    }
  }
}

// Index arithmetic of the host-free low-latency exchange, one kernel instead of some thirty small tensor operations.
// counts [world, cnt_stride] (the all-gathered pair counts: source rank x global expert); ids [pairs] this rank's
// (token, slot) expert ids (negative: none); rank_in [pairs] the pair's rank among this rank's pairs of the same
// expert.  Rows of an expert's block on its owner are ordered by source rank and, inside a source, by that rank; a
// rank's return buffer is ordered by expert, then by that rank.
//   as a source, per pair: pair_rank / pair_row (owner and row of its [nle * rpe] layout; -1 = not sent: no expert or
//     the block is full), pair_pos (row of the own return buffer), ids32 (the id, -1 when not sent);
//   as an owner: masked_m [nle] and, per row of the layout, row_rank / row_pos (source and row of its return buffer,
//     -1 = unused).
// Every block first builds the counts and their running sums over the experts in shared memory (a few KB).
__global__ void __launch_bounds__(THREADS) ll_plan_kernel(const int* __restrict__ counts, int cnt_stride, int world,
                                                          int experts, int me, int nle, int rpe,
                                                          const long long* __restrict__ ids,
                                                          const int* __restrict__ rank_in, int pairs,
                                                          int* __restrict__ pair_rank, int* __restrict__ pair_row,
                                                          int* __restrict__ pair_pos, int* __restrict__ ids32,
                                                          int* __restrict__ masked_m, int* __restrict__ row_rank,
                                                          int* __restrict__ row_pos) {
  extern __shared__ int plan_smem[];
  int* cs = plan_smem;                       // [world][experts] counts
  int* before = plan_smem + world * experts; // [world][experts] the source's pairs of lower experts
  for (int i = threadIdx.x; i < world * experts; i += THREADS) {
    const int r = i / experts;
    cs[i] = __ldg(counts + (long long)r * cnt_stride + (i - r * experts));
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  for (int r = threadIdx.x >> 5; r < world; r += THREADS / 32) {   // one warp per source: scan over the experts
    int carry = 0;
    for (int e0 = 0; e0 < experts; e0 += 32) {
      const int e = e0 + lane;
      const int v = e < experts ? cs[r * experts + e] : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
      }
      if (e < experts) before[r * experts + e] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  const int lo = me * nle;
  const long long stride = (long long)gridDim.x * THREADS;
  const long long first = (long long)blockIdx.x * THREADS + threadIdx.x;
  for (long long p = first; p < pairs; p += stride) {
    const long long id = ids[p];
    int pr = -1, prow = -1, ppos = -1, kept = -1;
    if (id >= 0 && id < experts) {
      const int e = (int)id;
      int rows_before_me = 0;
      for (int r = 0; r < me; ++r) rows_before_me += cs[r * experts + e];
      const int row = rows_before_me + rank_in[p];
      if (row < rpe) {
        pr = e / nle;
        prow = (e - pr * nle) * rpe + row;
        ppos = before[me * experts + e] + rank_in[p];
        kept = e;
      }
    }
    pair_rank[p] = pr;
    pair_row[p] = prow;
    pair_pos[p] = ppos;
    ids32[p] = kept;
  }
  const long long layout_rows = (long long)nle * rpe;
  for (long long i = first; i < layout_rows; i += stride) {
    const int le = (int)(i / rpe), row = (int)(i - (long long)le * rpe);
    const int e = lo + le;
    int end = 0, src = -1, first_row = 0;
    for (int r = 0; r < world; ++r) {
      const int c = cs[r * experts + e];
      if (src < 0 && row < end + c) {
        src = r;
        first_row = end;
      }
      end += c;
    }
    row_rank[i] = src;
    row_pos[i] = src >= 0 ? before[src * experts + e] + (row - first_row) : -1;
    if (row == 0) masked_m[le] = min(end, rpe);
  }
}

// Barrier among the ranks of an expert-parallel group, one rank per GPU.  Rank i owns an array of one 32-bit
// word per peer; arriving means storing the barrier's number (a counter that every rank advances in step) into
// word "my rank" of every peer's array with release semantics at system scope, so that everything this rank
// stored into the peers' memory before, from earlier kernels of the stream included, is visible to a peer that
// has seen the number.  Then thread r waits until word r of the own array has reached the number.  The number is
// this rank's count of barriers on these words (kept in device memory and advanced by the kernel).  The wait is
// bounded: when `limit_ns` nanoseconds have passed the kernel records DLB_STATUS_TIMEOUT in the status word and
// returns; it never traps and never spins without a limit, so a rank that died or raised before its arrival
// costs its peers one time-out and an exception on the host, not a hung GPU.  Plain peer stores and loads only.
__global__ void __launch_bounds__(32) rank_barrier_kernel(PeerPtrs signals, int world, int my_rank,
                                                          uint32_t* __restrict__ counter, unsigned long long limit_ns,
                                                          int* __restrict__ status) {
  const int r = threadIdx.x;
  // the barrier's number lives on the device, so that a launch replayed from a CUDA graph still counts on
  uint32_t number = 0;
  if (r == 0) {
    number = *counter + 1u;
    *counter = number;
  }
  number = __shfl_sync(0xffffffffu, number, 0);
  if (r >= world) return;
  __threadfence_system();
  uint32_t* theirs = reinterpret_cast<uint32_t*>(signals.p[r]) + my_rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(number) : "memory");
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(signals.p[my_rank]) + r;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if ((int32_t)(seen - number) >= 0) break;
    if (globaltimer_ns() - t0 > limit_ns) {
      if (status != nullptr) atomicExch(status, DLB_STATUS_TIMEOUT);
      break;
    }
    __nanosleep(200);
  }
}

// ---- low-latency (masked layout) exchange ---------------------------------------------------------------------
// Copies this rank's small vector (`vecs` 16-byte words) into slot "my rank" of the same array on every peer: an
// all-gather by stores.
__global__ void __launch_bounds__(THREADS) all_gather_small_kernel(const uint4* __restrict__ src, int vecs, int world,
                                                                   int my_rank, PeerPtrs dst) {
  const int d = blockIdx.y;
  if (d >= world) return;
  uint4* out = reinterpret_cast<uint4*>(dst.p[d]) + (long long)my_rank * vecs;
  for (int i = blockIdx.x * THREADS + threadIdx.x; i < vecs; i += gridDim.x * THREADS) out[i] = __ldg(src + i);
}

// Quantises every token once and stores its row and scales for each of its routed slots straight into the masked
// layout of the rank that owns the slot's expert: slot f goes to rank pair_rank[f] (< 0: nowhere), row pair_row[f]
// of that rank's [E_local * rows_per_expert, k] buffer.
template <bool IS_BF16>
__global__ void __launch_bounds__(THREADS) ll_quant_push_kernel(const void* __restrict__ x, long long tokens, long long k,
                                                                long long ldx, int mode, float eps,
                                                                const int* __restrict__ pair_rank,
                                                                const int* __restrict__ pair_row, int top_k,
                                                                PeerPtrs peer_q, PeerPtrs peer_s) {
  const long long vec_per_row = k / 8;
  const long long total = tokens * vec_per_row;
  const long long groups = k / 128;
  for (long long u0 = (long long)blockIdx.x * THREADS; u0 < total; u0 += (long long)gridDim.x * THREADS) {
    const long long u = u0 + threadIdx.x;
    const bool active = u < total;
    const long long row = active ? u / vec_per_row : 0;
    const long long c = active ? (u - row * vec_per_row) * 8 : 0;
    float v[8];
    if (active) {
      if (IS_BF16) load8_bf16(reinterpret_cast<const __nv_bfloat16*>(x) + row * ldx + c, v);
      else load8_f16(reinterpret_cast<const __half*>(x) + row * ldx + c, v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = mode == DLB_QUANT_RECIP_MUL ? amax * (1.0f / 448.0f) : fmaxf(amax, eps) / 448.0f;
    if (!active) continue;
    uint2 packed;
    packed.x = (uint32_t)f32x2_to_e4m3x2(v[0] / scale, v[1] / scale) |
               ((uint32_t)f32x2_to_e4m3x2(v[2] / scale, v[3] / scale) << 16);
    packed.y = (uint32_t)f32x2_to_e4m3x2(v[4] / scale, v[5] / scale) |
               ((uint32_t)f32x2_to_e4m3x2(v[6] / scale, v[7] / scale) << 16);
    const bool first = ((c / 8) & 15) == 0;
    for (int j = 0; j < top_k; ++j) {
      const int r = __ldg(pair_rank + row * top_k + j);
      if (r < 0) continue;
      const long long drow = __ldg(pair_row + row * top_k + j);
      *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(peer_q.p[r]) + drow * k + c) = packed;
      if (first) reinterpret_cast<float*>(peer_s.p[r])[drow * groups + c / 128] = scale;
    }
  }
}

// Row i of `src` goes to rank row_rank[i] (< 0: nowhere), row row_pos[i] of that rank's buffer.
__global__ void __launch_bounds__(THREADS) push_rows_indexed_kernel(const uint4* __restrict__ src, long long vec_per_row,
                                                                    long long rows, const int* __restrict__ row_rank,
                                                                    const int* __restrict__ row_pos, PeerPtrs peer_dst) {
  const long long total = rows * vec_per_row;
  for (long long u = (long long)blockIdx.x * THREADS + threadIdx.x; u < total; u += (long long)gridDim.x * THREADS) {
    const long long row = u / vec_per_row;
    const int r = __ldg(row_rank + row);
    if (r < 0) continue;
    const long long c = u - row * vec_per_row;
    reinterpret_cast<uint4*>(peer_dst.p[r])[(long long)__ldg(row_pos + row) * vec_per_row + c] = __ldg(src + u);
  }
}

// The same over a masked layout [experts, rows_per_expert]: only the first masked_m[e] rows of every expert are looked
// at (one warp per valid row), not the whole layout.
__global__ void __launch_bounds__(THREADS) push_rows_masked_kernel(const uint4* __restrict__ src, long long vec_per_row,
                                                                   const int* __restrict__ masked_m, int experts,
                                                                   int rows_per_expert, const int* __restrict__ row_rank,
                                                                   const int* __restrict__ row_pos, PeerPtrs peer_dst) {
  __shared__ int prefix[MASKED_MAX_EXPERTS + 1];
  masked_prefix(masked_m, experts, rows_per_expert, prefix);
  const int total = prefix[experts];
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (THREADS / 32);
  for (int item = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5); item < total; item += warps) {
    const int e = masked_find(prefix, experts, item);
    const long long row = (long long)e * rows_per_expert + (item - prefix[e]);
    const int r = __ldg(row_rank + row);
    if (r < 0) continue;
    const uint4* from = src + row * vec_per_row;
    uint4* to = reinterpret_cast<uint4*>(peer_dst.p[r]) + (long long)__ldg(row_pos + row) * vec_per_row;
    for (long long c = lane; c < vec_per_row; c += 32) to[c] = __ldg(from + c);
  }
}

int grid_for(long long total_threads) {
  long long blocks = ceil_div(total_threads, THREADS);
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

int fill_peers(PeerPtrs& dst, const void* const* src, int world, const char* what) {
  for (int r = 0; r < world; ++r) {
    DLB_REQUIRE(src != nullptr && src[r] != nullptr, DLB_ERR_INVALID, "%s: null peer pointer for rank %d", what, r);
    DLB_REQUIRE((uintptr_t)src[r] % 16 == 0, DLB_ERR_INVALID, "%s: peer pointer of rank %d is not 16-byte aligned", what, r);
    dst.p[r] = const_cast<void*>(src[r]);
  }
  return DLB_OK;
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" int dlb_p2p_quant_push(const void* x, int x_dtype, int64_t tokens, int64_t k, int64_t ldx, int mode, float eps,
                                  const int32_t* within, int world, int my_rank, int64_t region_rows,
                                  const void* const* peer_q, const void* const* peer_scales,
                                  const void* const* peer_meta, const int32_t* meta, int meta_ints,
                                  const void* const* peer_counts, const int32_t* counts, void* stream) {
  DLB_REQUIRE(tokens >= 0 && k > 0 && k % 128 == 0, DLB_ERR_INVALID, "p2p_quant_push: k=%lld must be a multiple of 128",
              (long long)k);
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD && my_rank >= 0 && my_rank < world, DLB_ERR_INVALID,
              "p2p_quant_push: world=%d (max %d), rank=%d", world, MAX_WORLD, my_rank);
  DLB_REQUIRE(tokens <= region_rows, DLB_ERR_INVALID, "p2p_quant_push: %lld tokens exceed the region of %lld rows",
              (long long)tokens, (long long)region_rows);
  DLB_REQUIRE(x_dtype == DLB_BF16 || x_dtype == DLB_F16, DLB_ERR_INVALID, "p2p_quant_push: x must be bf16 or fp16");
  DLB_REQUIRE(mode == DLB_QUANT_RECIP_MUL || mode == DLB_QUANT_DIV_EPS, DLB_ERR_INVALID, "p2p_quant_push: bad mode");
  DLB_REQUIRE(meta_ints > 0 && meta_ints % 4 == 0, DLB_ERR_INVALID, "p2p_quant_push: meta_ints must be a multiple of 4");
  DLB_REQUIRE(within && meta && counts && (tokens == 0 || x), DLB_ERR_INVALID, "p2p_quant_push: null pointer");
  DLB_REQUIRE(tokens == 0 || ((uintptr_t)x % 16 == 0 && (ldx * 2) % 16 == 0), DLB_ERR_INVALID,
              "p2p_quant_push: x rows must be 16-byte aligned");
  PeerPtrs pq, ps, pm, pc;
  int rc;
  if ((rc = fill_peers(pq, peer_q, world, "p2p_quant_push(q)")) != DLB_OK) return rc;
  if ((rc = fill_peers(ps, peer_scales, world, "p2p_quant_push(scales)")) != DLB_OK) return rc;
  if ((rc = fill_peers(pm, peer_meta, world, "p2p_quant_push(meta)")) != DLB_OK) return rc;
  if ((rc = fill_peers(pc, peer_counts, world, "p2p_quant_push(counts)")) != DLB_OK) return rc;
  const int grid = grid_for(tokens * (k / 8));
  cudaStream_t st = (cudaStream_t)stream;
  if (x_dtype == DLB_BF16)
    quant_push_kernel<true><<<grid, THREADS, 0, st>>>(x, tokens, k, ldx, mode, eps, within, world, my_rank, region_rows, pq,
                                                     ps, pm, meta, meta_ints, pc, counts);
  else
    quant_push_kernel<false><<<grid, THREADS, 0, st>>>(x, tokens, k, ldx, mode, eps, within, world, my_rank, region_rows,
                                                      pq, ps, pm, meta, meta_ints, pc, counts);
  count_launch();
  DLB_CHECK_LAUNCH("quant_push_kernel");
  return DLB_OK;
}

extern "C" int dlb_p2p_unpack_meta(const int32_t* meta, int meta_ints, int top_k, const int32_t* counts, int world,
                                   int64_t region_rows, int expert_lo, int num_local_experts, int64_t* ids,
                                   float* weights, void* stream) {
  DLB_REQUIRE(meta && counts && ids && weights, DLB_ERR_INVALID, "p2p_unpack_meta: null pointer");
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD && region_rows > 0 && top_k > 0, DLB_ERR_INVALID,
              "p2p_unpack_meta: bad sizes");
  const int kp = meta_ints / 2;
  DLB_REQUIRE(meta_ints % 4 == 0 && kp >= top_k, DLB_ERR_INVALID, "p2p_unpack_meta: meta_ints=%d too small for top_k=%d",
              meta_ints, top_k);
  unpack_meta_kernel<<<grid_for((long long)world * region_rows * top_k), THREADS, 0, (cudaStream_t)stream>>>(
      meta, meta_ints, top_k, kp, counts, world, region_rows, expert_lo, num_local_experts,
      reinterpret_cast<long long*>(ids), weights);
  count_launch();
  DLB_CHECK_LAUNCH("unpack_meta_kernel");
  return DLB_OK;
}

extern "C" int dlb_p2p_push_rows(const void* src, int64_t row_bytes, const int32_t* counts, int world, int my_rank,
                                 int64_t region_rows, const void* const* peer_dst, void* stream) {
  DLB_REQUIRE(src && counts, DLB_ERR_INVALID, "p2p_push_rows: null pointer");
  DLB_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && (uintptr_t)src % 16 == 0, DLB_ERR_INVALID,
              "p2p_push_rows: rows must be multiples of 16 bytes and 16-byte aligned");
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD && my_rank >= 0 && my_rank < world && region_rows > 0, DLB_ERR_INVALID,
              "p2p_push_rows: bad sizes");
  PeerPtrs pd;
  int rc = fill_peers(pd, peer_dst, world, "p2p_push_rows");
  if (rc != DLB_OK) return rc;
  const long long vpr = row_bytes / 16;
  push_rows_kernel<<<grid_for((long long)world * region_rows * vpr), THREADS, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(src), vpr, counts, world, my_rank, region_rows, pd);
  count_launch();
  DLB_CHECK_LAUNCH("push_rows_kernel");
  return DLB_OK;
}

// col_begin, col_count: the columns of every row that this call sums and stores (multiples of 8; 0, h = all);
// max_blocks > 0 caps the grid, for a call that shares the GPU with a kernel of another stream.
static int p2p_sum_push(const void* y, int dtype, const int64_t* ids, int top_k, int64_t h, const int32_t* counts,
                        int world, int my_rank, int64_t region_rows, const void* const* peer_dst, void* stream,
                        int64_t col_begin, int64_t col_count, int max_blocks) {
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD && my_rank >= 0 && my_rank < world && region_rows > 0, DLB_ERR_INVALID,
              "p2p_sum_push: bad world / rank / region");
  DLB_REQUIRE(top_k > 0 && top_k <= 32 && h > 0 && h % 8 == 0, DLB_ERR_INVALID,
              "p2p_sum_push: top_k=%d must be in [1, 32] and h=%lld a multiple of 8", top_k, (long long)h);
  DLB_REQUIRE(col_begin >= 0 && col_count > 0 && col_begin + col_count <= h && col_begin % 8 == 0 && col_count % 8 == 0,
              DLB_ERR_INVALID, "p2p_sum_push: columns [%lld, +%lld) of h=%lld must be multiples of 8 inside the row",
              (long long)col_begin, (long long)col_count, (long long)h);
  DLB_REQUIRE(dtype == DLB_BF16 || dtype == DLB_F16, DLB_ERR_INVALID, "p2p_sum_push: dtype must be bf16 or fp16");
  DLB_REQUIRE(y && ids && counts, DLB_ERR_INVALID, "p2p_sum_push: null pointer");
  DLB_REQUIRE((uintptr_t)y % 16 == 0, DLB_ERR_INVALID, "p2p_sum_push: y must be 16-byte aligned");
  PeerPtrs pd;
  int rc = fill_peers(pd, peer_dst, world, "p2p_sum_push");
  if (rc != DLB_OK) return rc;
  int grid = grid_for((long long)world * region_rows * 32);
  if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == DLB_BF16)
    sum_push_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(y),
                                                            reinterpret_cast<const long long*>(ids), top_k, h, counts,
                                                            world, my_rank, region_rows, pd, col_begin,
                                                            col_begin + col_count);
  else
    sum_push_kernel<__half><<<grid, THREADS, 0, st>>>(reinterpret_cast<const __half*>(y),
                                                     reinterpret_cast<const long long*>(ids), top_k, h, counts, world,
                                                     my_rank, region_rows, pd, col_begin, col_begin + col_count);
  count_launch();
  DLB_CHECK_LAUNCH("sum_push_kernel");
  return DLB_OK;
}

extern "C" int dlb_p2p_sum_push(const void* y, int dtype, const int64_t* ids, int top_k, int64_t h, const int32_t* counts,
                                int world, int my_rank, int64_t region_rows, const void* const* peer_dst, void* stream) {
  return p2p_sum_push(y, dtype, ids, top_k, h, counts, world, my_rank, region_rows, peer_dst, stream, 0, h, 0);
}

extern "C" int dlb_p2p_sum_push_cols(const void* y, int dtype, const int64_t* ids, int top_k, int64_t h,
                                     const int32_t* counts, int world, int my_rank, int64_t region_rows,
                                     const void* const* peer_dst, void* stream, int64_t col_begin, int64_t col_count,
                                     int max_blocks) {
  return p2p_sum_push(y, dtype, ids, top_k, h, counts, world, my_rank, region_rows, peer_dst, stream, col_begin,
                      col_count, max_blocks);
}

extern "C" int dlb_p2p_push_rows_masked(const void* src, int64_t row_bytes, const int32_t* masked_m, int num_local_experts,
                                        int rows_per_expert, const int32_t* row_rank, const int32_t* row_pos, int world,
                                        const void* const* peer_dst, void* stream) {
  DLB_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, DLB_ERR_INVALID,
              "p2p_push_rows_masked: rows must be multiples of 16 bytes");
  DLB_REQUIRE(num_local_experts > 0 && num_local_experts <= MASKED_MAX_EXPERTS && rows_per_expert > 0, DLB_ERR_INVALID,
              "p2p_push_rows_masked: experts=%d (at most %d), rows_per_expert=%d", num_local_experts, MASKED_MAX_EXPERTS,
              rows_per_expert);
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD, DLB_ERR_INVALID, "p2p_push_rows_masked: bad world");
  DLB_REQUIRE(src && masked_m && row_rank && row_pos && (uintptr_t)src % 16 == 0, DLB_ERR_INVALID,
              "p2p_push_rows_masked: null or misaligned pointer");
  PeerPtrs pd;
  int rc = fill_peers(pd, peer_dst, world, "p2p_push_rows_masked");
  if (rc != DLB_OK) return rc;
  push_rows_masked_kernel<<<2 * sm_count(), THREADS, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(src), row_bytes / 16, masked_m, num_local_experts, rows_per_expert, row_rank, row_pos,
      pd);
  count_launch();
  DLB_CHECK_LAUNCH("push_rows_masked_kernel");
  return DLB_OK;
}

extern "C" int dlb_p2p_barrier(const void* const* peer_signals, int world, int my_rank, uint32_t* counter,
                               uint64_t limit_ns, int32_t* status, void* stream) {
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD && my_rank >= 0 && my_rank < world, DLB_ERR_INVALID,
              "p2p_barrier: world=%d (max %d), rank=%d", world, MAX_WORLD, my_rank);
  DLB_REQUIRE(limit_ns > 0, DLB_ERR_INVALID, "p2p_barrier: the wait needs a limit");
  DLB_REQUIRE(counter != nullptr, DLB_ERR_INVALID, "p2p_barrier: null counter");
  PeerPtrs ps;
  for (int r = 0; r < world; ++r) {
    DLB_REQUIRE(peer_signals != nullptr && peer_signals[r] != nullptr && (uintptr_t)peer_signals[r] % 4 == 0,
                DLB_ERR_INVALID, "p2p_barrier: bad signal pointer for rank %d", r);
    ps.p[r] = const_cast<void*>(peer_signals[r]);
  }
  rank_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ps, world, my_rank, counter, limit_ns, status);
  count_launch();
  DLB_CHECK_LAUNCH("rank_barrier_kernel");
  return DLB_OK;
}

extern "C" int dlb_p2p_all_gather_small(const void* src, int64_t bytes, int world, int my_rank,
                                        const void* const* peer_dst, void* stream) {
  DLB_REQUIRE(src && bytes > 0 && bytes % 16 == 0 && (uintptr_t)src % 16 == 0 && bytes <= (1 << 24), DLB_ERR_INVALID,
              "p2p_all_gather_small: bytes=%lld must be a positive multiple of 16 (at most 16 MiB), src 16-byte aligned",
              (long long)bytes);
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD && my_rank >= 0 && my_rank < world, DLB_ERR_INVALID,
              "p2p_all_gather_small: world=%d (max %d), rank=%d", world, MAX_WORLD, my_rank);
  PeerPtrs pd;
  int rc = fill_peers(pd, peer_dst, world, "p2p_all_gather_small");
  if (rc != DLB_OK) return rc;
  const int vecs = (int)(bytes / 16);
  dim3 grid((unsigned)min((long long)ceil_div(vecs, THREADS), 64ll), (unsigned)world);
  all_gather_small_kernel<<<grid, THREADS, 0, (cudaStream_t)stream>>>(reinterpret_cast<const uint4*>(src), vecs, world,
                                                                     my_rank, pd);
  count_launch();
  DLB_CHECK_LAUNCH("all_gather_small_kernel");
  return DLB_OK;
}

extern "C" int dlb_p2p_ll_plan(const int32_t* counts, int cnt_stride, int world, int num_experts, int my_rank,
                               int num_local_experts, int rows_per_expert, const int64_t* topk_ids,
                               const int32_t* rank_in_expert, int64_t pairs, int32_t* pair_rank, int32_t* pair_row,
                               int32_t* pair_pos, int32_t* ids_sent, int32_t* masked_m, int32_t* row_rank,
                               int32_t* row_pos, void* stream) {
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD && my_rank >= 0 && my_rank < world, DLB_ERR_INVALID,
              "p2p_ll_plan: world=%d (max %d), rank=%d", world, MAX_WORLD, my_rank);
  DLB_REQUIRE(num_experts > 0 && num_local_experts > 0 && num_experts == num_local_experts * world &&
                  cnt_stride >= num_experts && rows_per_expert > 0 && pairs >= 0 && pairs < (1ll << 31),
              DLB_ERR_INVALID, "p2p_ll_plan: experts=%d, local=%d, stride=%d, rows_per_expert=%d, pairs=%lld", num_experts,
              num_local_experts, cnt_stride, rows_per_expert, (long long)pairs);
  DLB_REQUIRE(counts && masked_m && row_rank && row_pos && (pairs == 0 || (topk_ids && rank_in_expert && pair_rank &&
                                                                           pair_row && pair_pos && ids_sent)),
              DLB_ERR_INVALID, "p2p_ll_plan: null pointer");
  const size_t smem = (size_t)2 * world * num_experts * sizeof(int);
  DLB_REQUIRE(smem <= 200 * 1024, DLB_ERR_UNSUPPORTED, "p2p_ll_plan: %d ranks x %d experts do not fit in shared memory",
              world, num_experts);
  if (smem > 48 * 1024) {
    int rc = check_cuda(cudaFuncSetAttribute(ll_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "cudaFuncSetAttribute(ll_plan_kernel)");
    if (rc != DLB_OK) return rc;
  }
  const long long work = max((long long)pairs, (long long)num_local_experts * rows_per_expert);
  const int grid = (int)min((long long)ceil_div(work, (int64_t)THREADS), 128ll);
  ll_plan_kernel<<<grid, THREADS, smem, (cudaStream_t)stream>>>(
      counts, cnt_stride, world, num_experts, my_rank, num_local_experts, rows_per_expert,
      reinterpret_cast<const long long*>(topk_ids), rank_in_expert, (int)pairs, pair_rank, pair_row, pair_pos, ids_sent,
      masked_m, row_rank, row_pos);
  count_launch();
  DLB_CHECK_LAUNCH("ll_plan_kernel");
  return DLB_OK;
}

extern "C" int dlb_p2p_ll_quant_push(const void* x, int x_dtype, int64_t tokens, int64_t k, int64_t ldx, int mode,
                                     float eps, const int32_t* pair_rank, const int32_t* pair_row, int top_k, int world,
                                     const void* const* peer_q, const void* const* peer_scales, void* stream) {
  DLB_REQUIRE(tokens >= 0 && k > 0 && k % 128 == 0, DLB_ERR_INVALID, "p2p_ll_quant_push: k=%lld must be a multiple of 128",
              (long long)k);
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD && top_k > 0, DLB_ERR_INVALID, "p2p_ll_quant_push: bad world / top_k");
  DLB_REQUIRE(x_dtype == DLB_BF16 || x_dtype == DLB_F16, DLB_ERR_INVALID, "p2p_ll_quant_push: x must be bf16 or fp16");
  DLB_REQUIRE(mode == DLB_QUANT_RECIP_MUL || mode == DLB_QUANT_DIV_EPS, DLB_ERR_INVALID, "p2p_ll_quant_push: bad mode");
  if (tokens == 0) return DLB_OK;
  DLB_REQUIRE(x && pair_rank && pair_row, DLB_ERR_INVALID, "p2p_ll_quant_push: null pointer");
  DLB_REQUIRE((uintptr_t)x % 16 == 0 && (ldx * 2) % 16 == 0, DLB_ERR_INVALID,
              "p2p_ll_quant_push: x rows must be 16-byte aligned");
  PeerPtrs pq, ps;
  int rc;
  if ((rc = fill_peers(pq, peer_q, world, "p2p_ll_quant_push(q)")) != DLB_OK) return rc;
  if ((rc = fill_peers(ps, peer_scales, world, "p2p_ll_quant_push(scales)")) != DLB_OK) return rc;
  const int grid = grid_for(tokens * (k / 8));
  cudaStream_t st = (cudaStream_t)stream;
  if (x_dtype == DLB_BF16)
    ll_quant_push_kernel<true><<<grid, THREADS, 0, st>>>(x, tokens, k, ldx, mode, eps, pair_rank, pair_row, top_k, pq, ps);
  else
    ll_quant_push_kernel<false><<<grid, THREADS, 0, st>>>(x, tokens, k, ldx, mode, eps, pair_rank, pair_row, top_k, pq, ps);
  count_launch();
  DLB_CHECK_LAUNCH("ll_quant_push_kernel");
  return DLB_OK;
}

extern "C" int dlb_p2p_push_rows_indexed(const void* src, int64_t row_bytes, int64_t rows, const int32_t* row_rank,
                                         const int32_t* row_pos, int world, const void* const* peer_dst, void* stream) {
  DLB_REQUIRE(rows >= 0 && row_bytes > 0 && row_bytes % 16 == 0, DLB_ERR_INVALID,
              "p2p_push_rows_indexed: rows must be multiples of 16 bytes");
  DLB_REQUIRE(world > 0 && world <= MAX_WORLD, DLB_ERR_INVALID, "p2p_push_rows_indexed: bad world");
  if (rows == 0) return DLB_OK;
  DLB_REQUIRE(src && row_rank && row_pos && (uintptr_t)src % 16 == 0, DLB_ERR_INVALID,
              "p2p_push_rows_indexed: null or misaligned pointer");
  PeerPtrs pd;
  int rc = fill_peers(pd, peer_dst, world, "p2p_push_rows_indexed");
  if (rc != DLB_OK) return rc;
  const long long vpr = row_bytes / 16;
  push_rows_indexed_kernel<<<grid_for(rows * vpr), THREADS, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(src), vpr, rows, row_rank, row_pos, pd);
  count_launch();
  DLB_CHECK_LAUNCH("push_rows_indexed_kernel");
  return DLB_OK;
}
