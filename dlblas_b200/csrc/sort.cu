// Stable token-by-expert counting sort and the tile lists of the grouped GEMMs.
//
// Replaces `argsort` + `_start_end_kernel` of the reference
// (dlblas/layers/moe/kernels/fused_moe.py:27-51, 83-88): O(S) instead of a radix sort plus
// an O(E*S) scan, and a defined (stable) order inside each expert segment.
//
// Buckets: 0 holds ids < 0 ("not routed here", sorted first like argsort does with -1),
// 1..E hold experts 0..E-1, E+1 holds ids >= E (sorted last, never part of a segment).
// Every warp owns a contiguous chunk of the flat id array, which keeps the order stable:
//   count:   per-chunk histogram                    -> cnt[chunk][bucket]
//   scan:    exclusive prefix over chunks per bucket, then over buckets
//   scatter: position = bucket base + chunk prefix + rank inside the chunk
// Small inputs run all three phases in one CTA with the histograms in shared memory.
#include <mutex>

#include "common.cuh"
#include "sort.cuh"

namespace dlb {
namespace {

constexpr int SMALL_WARPS = 32;        // single-CTA path: 32 warps, one chunk each
constexpr int WARPS_PER_BLOCK = 8;     // multi-CTA path

template <typename IdT>
__device__ __forceinline__ int bucket_of(const IdT* ids, long long f, long long n, int num_experts) {
  if (f >= n) return num_experts + 2;  // spare slot for idle lanes
  const long long v = (long long)ids[f];
  if (v < 0) return 0;
  if (v >= num_experts) return num_experts + 1;
  return (int)v + 1;
}

// One step of the stable in-warp ranking: returns the value of hist[bucket] before this
// group of 32 ids and the lane's rank among the lanes of the group with the same bucket.
__device__ __forceinline__ int warp_rank_step(int* hist, int bucket, int lane, int& rank) {
  const unsigned peers = __match_any_sync(0xffffffffu, bucket);
  rank = __popc(peers & ((1u << lane) - 1u));
  const int old = hist[bucket];
  __syncwarp();
  if (rank == 0) hist[bucket] = old + __popc(peers);
  __syncwarp();
  return old;
}

struct SortOut {
  long long* sorted_idx;
  long long* exp_start;
  long long* exp_end;
  int* slot_pos;
  int* rank_in_expert;
  int* counts;
};

// bucket bases -> exp_start / exp_end / counts.  total[] and base[] have nb = E + 2 entries.
__device__ __forceinline__ void write_segments(const int* total, const int* base, int num_experts, const SortOut& o,
                                               int tid, int nthreads) {
  for (int e = tid; e < num_experts; e += nthreads) {
    const int c = total[e + 1];
    const long long s = c > 0 ? (long long)base[e + 1] : 0ll;   // empty expert: start = end = 0
    if (o.exp_start) o.exp_start[e] = s;
    if (o.exp_end) o.exp_end[e] = s + c;
    if (o.counts) o.counts[e] = c;
  }
}

template <typename IdT>
__device__ __forceinline__ void scatter_chunk(const IdT* ids, long long n, int num_experts, long long begin,
                                              long long end, int* hist, const int* base, int lane, const SortOut& o) {
  for (long long f0 = begin; f0 < end; f0 += 32) {
    const long long f = f0 + lane;
    const int b = bucket_of(ids, f < end ? f : n, n, num_experts);
    int rank;
    const int old = warp_rank_step(hist, b, lane, rank);
    if (f < end) {
      const int pos = old + rank;
      if (o.sorted_idx) o.sorted_idx[pos] = f;
      if (o.slot_pos) o.slot_pos[f] = (b == 0 || b == num_experts + 1) ? -(pos + 1) : pos;
      if (o.rank_in_expert) o.rank_in_expert[f] = (b >= 1 && b <= num_experts) ? pos - base[b] : -1;
    }
  }
}

// ---- single-CTA path -------------------------------------------------------------
template <typename IdT>
__global__ void __launch_bounds__(SMALL_WARPS * 32) sort_small_kernel(const IdT* ids, long long n, int num_experts,
                                                                      SortOut o) {
  extern __shared__ int sm[];
  const int nb = num_experts + 2;
  const int stride = nb + 1;              // + spare slot for idle lanes
  int* hist = sm;                         // [SMALL_WARPS][stride]
  int* total = sm + SMALL_WARPS * stride; // [nb]
  int* base = total + nb;                 // [nb]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < SMALL_WARPS * stride; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  long long chunk = (n + SMALL_WARPS - 1) / SMALL_WARPS;
  chunk = (chunk + 31) / 32 * 32;
  const long long begin = min((long long)warp * chunk, n), end = min(begin + chunk, n);
  int* my = hist + warp * stride;
  for (long long f0 = begin; f0 < end; f0 += 32) {
    const long long f = f0 + lane;
    const int b = bucket_of(ids, f < end ? f : n, n, num_experts);
    int rank;
    warp_rank_step(my, b, lane, rank);
  }
  __syncthreads();
  // exclusive prefix over the warps' chunks, per bucket
  for (int b = threadIdx.x; b < nb; b += blockDim.x) {
    int run = 0;
    for (int w = 0; w < SMALL_WARPS; ++w) {
      const int c = hist[w * stride + b];
      hist[w * stride + b] = run;
      run += c;
    }
    total[b] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int b = 0; b < nb; ++b) {
      base[b] = run;
      run += total[b];
    }
  }
  __syncthreads();
  write_segments(total, base, num_experts, o, threadIdx.x, blockDim.x);
  for (int b = lane; b < nb; b += 32) my[b] += base[b];
  __syncwarp();
  scatter_chunk(ids, n, num_experts, begin, end, my, base, lane, o);
}

// ---- multi-CTA path ----------------------------------------------------------------
template <typename IdT>
__global__ void __launch_bounds__(WARPS_PER_BLOCK * 32) sort_count_kernel(const IdT* ids, long long n, int num_experts,
                                                                          long long chunk, int num_chunks, int* cnt) {
  extern __shared__ int sm[];
  const int nb = num_experts + 2, stride = nb + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* my = sm + warp * stride;
  for (int i = lane; i < stride; i += 32) my[i] = 0;
  __syncwarp();
  const int c = blockIdx.x * WARPS_PER_BLOCK + warp;
  if (c >= num_chunks) return;
  const long long begin = (long long)c * chunk, end = min(begin + chunk, n);
  for (long long f0 = begin; f0 < end; f0 += 32) {
    const long long f = f0 + lane;
    const int b = bucket_of(ids, f < end ? f : n, n, num_experts);
    int rank;
    warp_rank_step(my, b, lane, rank);
  }
  for (int b = lane; b < nb; b += 32) cnt[(long long)c * nb + b] = my[b];
}

// One CTA per bucket: exclusive prefix over chunks (in place) and the bucket total.
__global__ void __launch_bounds__(256) sort_scan_chunks_kernel(int* cnt, int num_chunks, int nb, int* total) {
  __shared__ int warp_sums[8];
  __shared__ int carry_s;
  const int b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < num_chunks; c0 += 256) {
    const int c = c0 + threadIdx.x;
    const int v = c < num_chunks ? cnt[(long long)c * nb + b] : 0;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += y;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    int woff = 0;
    for (int w = 0; w < warp; ++w) woff += warp_sums[w];
    const int carry = carry_s;
    if (c < num_chunks) cnt[(long long)c * nb + b] = carry + woff + inc - v;
    __syncthreads();
    if (threadIdx.x == 255) carry_s = carry + woff + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) total[b] = carry_s;
}

__global__ void __launch_bounds__(1024) sort_scan_buckets_kernel(const int* total, int* base, int nb, int num_experts,
                                                                 SortOut o) {
  extern __shared__ int sm[];  // [nb] bases
  if (threadIdx.x == 0) {
    int run = 0;
    for (int b = 0; b < nb; ++b) {
      sm[b] = run;
      run += total[b];
    }
  }
  __syncthreads();
  for (int b = threadIdx.x; b < nb; b += blockDim.x) base[b] = sm[b];
  write_segments(total, sm, num_experts, o, threadIdx.x, blockDim.x);
}

template <typename IdT>
__global__ void __launch_bounds__(WARPS_PER_BLOCK * 32) sort_scatter_kernel(const IdT* ids, long long n,
                                                                            int num_experts, long long chunk,
                                                                            int num_chunks, const int* cnt,
                                                                            const int* base, SortOut o) {
  extern __shared__ int sm[];
  const int nb = num_experts + 2, stride = nb + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* my = sm + warp * stride;
  int* sbase = sm + WARPS_PER_BLOCK * stride;
  for (int b = threadIdx.x; b < nb; b += blockDim.x) sbase[b] = base[b];
  __syncthreads();
  const int c = blockIdx.x * WARPS_PER_BLOCK + warp;
  if (c >= num_chunks) return;
  for (int b = lane; b < nb; b += 32) my[b] = sbase[b] + cnt[(long long)c * nb + b];
  if (lane == 0) my[nb] = 0;
  __syncwarp();
  const long long begin = (long long)c * chunk, end = min(begin + chunk, n);
  scatter_chunk(ids, n, num_experts, begin, end, my, sbase, lane, o);
}

struct Plan {
  bool small;
  long long chunk;
  int num_chunks;
  size_t cnt_bytes;   // [num_chunks][nb] int32
  size_t total_off, base_off, bytes;
};

Plan make_plan(long long n, int num_experts) {
  Plan p;
  const int nb = num_experts + 2;
  p.small = n <= 16384 && (size_t)(SMALL_WARPS * (nb + 1) + 2 * nb) * 4 <= 200 * 1024;
  long long chunk = (n + 1023) / 1024;
  chunk = (chunk + 31) / 32 * 32;
  if (chunk < 256) chunk = 256;
  p.chunk = chunk;
  p.num_chunks = (int)((n + chunk - 1) / chunk);
  p.cnt_bytes = ((size_t)p.num_chunks * nb * 4 + 255) / 256 * 256;
  p.total_off = p.cnt_bytes;
  p.base_off = p.total_off + ((size_t)nb * 4 + 255) / 256 * 256;
  p.bytes = p.base_off + ((size_t)nb * 4 + 255) / 256 * 256;
  return p;
}

template <typename IdT>
int run_sort(const IdT* ids, long long n, int num_experts, const SortOut& o, void* ws, size_t ws_bytes,
             cudaStream_t st) {
  const int nb = num_experts + 2;
  const Plan p = make_plan(n, num_experts);
  if (p.small) {
    const size_t smem = (size_t)(SMALL_WARPS * (nb + 1) + 2 * nb) * 4;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev < 64 && !configured[dev]) {
      int rc = check_cuda(cudaFuncSetAttribute(sort_small_kernel<IdT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               200 * 1024),
                          "cudaFuncSetAttribute(sort_small_kernel)");
      if (rc != DLB_OK) return rc;
      configured[dev] = true;
    }
    sort_small_kernel<IdT><<<1, SMALL_WARPS * 32, smem, st>>>(ids, n, num_experts, o);
    count_launch();
    DLB_CHECK_LAUNCH("sort_small_kernel");
    return DLB_OK;
  }
  DLB_REQUIRE(ws != nullptr && ws_bytes >= p.bytes, DLB_ERR_WORKSPACE,
              "sort_by_expert: workspace of %zu bytes needed, %zu given", p.bytes, ws_bytes);
  DLB_REQUIRE(nb + 1 <= 1100, DLB_ERR_UNSUPPORTED, "sort_by_expert: more than 1097 experts need the small path");
  int* cnt = reinterpret_cast<int*>(ws);
  int* total = reinterpret_cast<int*>(reinterpret_cast<char*>(ws) + p.total_off);
  int* base = reinterpret_cast<int*>(reinterpret_cast<char*>(ws) + p.base_off);
  const int blocks = (p.num_chunks + WARPS_PER_BLOCK - 1) / WARPS_PER_BLOCK;
  const size_t smem1 = (size_t)WARPS_PER_BLOCK * (nb + 1) * 4;
  sort_count_kernel<IdT><<<blocks, WARPS_PER_BLOCK * 32, smem1, st>>>(ids, n, num_experts, p.chunk, p.num_chunks, cnt);
  count_launch();
  DLB_CHECK_LAUNCH("sort_count_kernel");
  sort_scan_chunks_kernel<<<nb, 256, 0, st>>>(cnt, p.num_chunks, nb, total);
  count_launch();
  DLB_CHECK_LAUNCH("sort_scan_chunks_kernel");
  sort_scan_buckets_kernel<<<1, 1024, (size_t)nb * 4, st>>>(total, base, nb, num_experts, o);
  count_launch();
  DLB_CHECK_LAUNCH("sort_scan_buckets_kernel");
  const size_t smem3 = smem1 + (size_t)nb * 4;
  sort_scatter_kernel<IdT><<<blocks, WARPS_PER_BLOCK * 32, smem3, st>>>(ids, n, num_experts, p.chunk, p.num_chunks,
                                                                      cnt, base, o);
  count_launch();
  DLB_CHECK_LAUNCH("sort_scatter_kernel");
  return DLB_OK;
}

// ---- tile lists -------------------------------------------------------------------
// tiles[0] = {num_tiles, 0, 0, 0}; tiles[1 + i] = {expert, first row, valid rows, 0}.
__global__ void __launch_bounds__(1024) build_tiles_kernel(const long long* exp_start, const long long* exp_end,
                                                           const int* masked_m, int expert_offset, int num_local,
                                                           int rows_per_expert, int tile_rows, int4* tiles,
                                                           int max_tiles) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int e0 = 0; e0 < num_local; e0 += blockDim.x) {
    const int e = e0 + threadIdx.x;
    long long start = 0;
    int rows = 0;
    if (e < num_local) {
      if (masked_m != nullptr) {
        rows = min(max(masked_m[e], 0), rows_per_expert);
        start = (long long)e * rows_per_expert;
      } else {
        start = exp_start[e + expert_offset];
        rows = (int)(exp_end[e + expert_offset] - start);
        if (rows < 0) rows = 0;
      }
    }
    const int nt = (rows + tile_rows - 1) / tile_rows;
    int inc = nt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += y;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    int woff = 0;
    for (int w = 0; w < warp; ++w) woff += warp_sums[w];
    const int carry = carry_s;
    const int first = carry + woff + inc - nt;
    for (int i = 0; i < nt; ++i) {
      const int idx = first + i;
      if (idx < max_tiles)
        tiles[1 + idx] = make_int4(e, (int)(start + (long long)i * tile_rows), min(tile_rows, rows - i * tile_rows), 0);
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry_s = carry + woff + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) tiles[0] = make_int4(min(carry_s, max_tiles), 0, 0, 0);
}

}  // namespace

size_t sort_workspace_size(long long n, int num_experts) { return make_plan(n, num_experts).bytes; }

int sort_by_expert(const void* ids, int ids_dtype, long long n, int num_experts, long long* sorted_idx,
                   long long* exp_start, long long* exp_end, int* slot_pos, int* rank_in_expert, int* counts,
                   void* ws, size_t ws_bytes, cudaStream_t st) {
  DLB_REQUIRE(n >= 0 && n < (1ll << 31) && num_experts > 0, DLB_ERR_INVALID,
              "sort_by_expert: bad sizes num_slots=%lld num_experts=%d", n, num_experts);
  DLB_REQUIRE(ids_dtype == DLB_I32 || ids_dtype == DLB_I64, DLB_ERR_INVALID, "sort_by_expert: ids must be int32/int64");
  const SortOut o = {sorted_idx, exp_start, exp_end, slot_pos, rank_in_expert, counts};
  if (n == 0) {
    // no slots: every expert is empty
    if (exp_start) cudaMemsetAsync(exp_start, 0, sizeof(long long) * num_experts, st);
    if (exp_end) cudaMemsetAsync(exp_end, 0, sizeof(long long) * num_experts, st);
    if (counts) cudaMemsetAsync(counts, 0, sizeof(int) * num_experts, st);
    return DLB_OK;
  }
  DLB_REQUIRE(ids != nullptr, DLB_ERR_INVALID, "sort_by_expert: null ids");
  if (ids_dtype == DLB_I32) return run_sort<int>(reinterpret_cast<const int*>(ids), n, num_experts, o, ws, ws_bytes, st);
  return run_sort<long long>(reinterpret_cast<const long long*>(ids), n, num_experts, o, ws, ws_bytes, st);
}

}  // namespace dlb

using namespace dlb;

extern "C" size_t dlb_sort_by_expert_workspace_size(int64_t num_slots, int num_experts) {
  if (num_slots <= 0 || num_experts <= 0) return 0;
  return sort_workspace_size(num_slots, num_experts);
}

extern "C" int dlb_sort_by_expert(const void* ids, int ids_dtype, int64_t num_slots, int num_experts,
                                  int64_t* sorted_idx, int64_t* exp_start, int64_t* exp_end, int32_t* slot_pos,
                                  int32_t* rank_in_expert, int32_t* counts, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  return sort_by_expert(ids, ids_dtype, num_slots, num_experts, reinterpret_cast<long long*>(sorted_idx),
                        reinterpret_cast<long long*>(exp_start), reinterpret_cast<long long*>(exp_end), slot_pos,
                        rank_in_expert, counts, workspace, workspace_bytes, (cudaStream_t)stream);
}

// ---- variant of the sort that never allocates -----------------------------------------
// Some callers cannot hand over a workspace: an inference engine that reserved all device
// memory for its own pool at start-up has nothing left for cudaMalloc to give, and code that
// runs where an allocation's implicit device-wide synchronisation is not acceptable must not
// call the allocator at all.  For them the chunk histograms live in a fixed array that is
// part of the loaded module (every GPU that loads the library holds these bytes until exit).
namespace {
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)4 * 1024 * 1024 + 16 * 1024;
static __device__ __align__(256) unsigned char g_sort_scratch[STATIC_SCRATCH_BYTES];

// In host code `g_sort_scratch` is only a handle for the runtime, not a device address; the
// address the kernels need is looked up once per device, with that device current.
void* g_scratch_ptr[64] = {};
std::mutex g_scratch_mutex;

int static_scratch(void** out) {
  int dev = 0;
  int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (rc != DLB_OK) return rc;
  DLB_REQUIRE(dev >= 0 && dev < 64, DLB_ERR_UNSUPPORTED, "sort_by_expert_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    rc = check_cuda(cudaGetSymbolAddress(&p, g_sort_scratch), "cudaGetSymbolAddress(g_sort_scratch)");
    if (rc != DLB_OK) return rc;
    DLB_REQUIRE(p != nullptr, DLB_ERR_CUDA, "sort_by_expert_static: the scratch array has no device address");
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return DLB_OK;
}
}  // namespace

extern "C" size_t dlb_sort_by_expert_static_capacity(void) { return STATIC_SCRATCH_BYTES; }

extern "C" int dlb_sort_by_expert_static(const void* ids, int ids_dtype, int64_t num_slots, int num_experts,
                                         int64_t* sorted_idx, int64_t* exp_start, int64_t* exp_end,
                                         int32_t* slot_pos, int32_t* rank_in_expert, int32_t* counts, void* stream) {
  DLB_REQUIRE(num_slots >= 0 && num_experts > 0, DLB_ERR_INVALID,
              "sort_by_expert_static: bad sizes num_slots=%lld num_experts=%d", (long long)num_slots, num_experts);
  const size_t need = num_slots > 0 ? sort_workspace_size(num_slots, num_experts) : 0;
  DLB_REQUIRE(need <= STATIC_SCRATCH_BYTES, DLB_ERR_WORKSPACE,
              "sort_by_expert_static: num_slots=%lld with num_experts=%d needs %zu bytes of scratch, the built-in "
              "array holds %zu; use dlb_sort_by_expert with a caller-provided workspace",
              (long long)num_slots, num_experts, need, STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc != DLB_OK) return rc;
  // Every word of the scratch that the kernels read is written earlier in the same call (the
  // count kernel fills the whole histogram matrix), so leftovers of a previous call are harmless.
  return sort_by_expert(ids, ids_dtype, num_slots, num_experts, reinterpret_cast<long long*>(sorted_idx),
                        reinterpret_cast<long long*>(exp_start), reinterpret_cast<long long*>(exp_end), slot_pos,
                        rank_in_expert, counts, scratch, STATIC_SCRATCH_BYTES, (cudaStream_t)stream);
}

extern "C" int dlb_moe_build_tiles(const int64_t* exp_start, const int64_t* exp_end, int expert_offset,
                                   int num_local_experts, int32_t* tiles, int max_tiles, void* stream) {
  DLB_REQUIRE(exp_start && exp_end && tiles, DLB_ERR_INVALID, "build_tiles: null pointer");
  DLB_REQUIRE(num_local_experts > 0 && expert_offset >= 0 && max_tiles >= 0, DLB_ERR_INVALID, "build_tiles: bad sizes");
  DLB_REQUIRE((uintptr_t)tiles % 16 == 0, DLB_ERR_INVALID, "build_tiles: tiles must be 16-byte aligned");
  build_tiles_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(reinterpret_cast<const long long*>(exp_start),
                                                           reinterpret_cast<const long long*>(exp_end), nullptr,
                                                           expert_offset, num_local_experts, 0, 128,
                                                           reinterpret_cast<int4*>(tiles), max_tiles);
  count_launch();
  DLB_CHECK_LAUNCH("build_tiles_kernel");
  return DLB_OK;
}

extern "C" int dlb_moe_build_tiles_rows(const int64_t* exp_start, const int64_t* exp_end, int expert_offset,
                                        int num_local_experts, int tile_rows, int32_t* tiles, int max_tiles,
                                        void* stream) {
  DLB_REQUIRE(exp_start && exp_end && tiles, DLB_ERR_INVALID, "build_tiles_rows: null pointer");
  DLB_REQUIRE(num_local_experts > 0 && expert_offset >= 0 && max_tiles >= 0, DLB_ERR_INVALID,
              "build_tiles_rows: bad sizes");
  DLB_REQUIRE(tile_rows == 128 || tile_rows == 256, DLB_ERR_INVALID, "build_tiles_rows: tile_rows must be 128 or 256");
  DLB_REQUIRE((uintptr_t)tiles % 16 == 0, DLB_ERR_INVALID, "build_tiles_rows: tiles must be 16-byte aligned");
  build_tiles_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(reinterpret_cast<const long long*>(exp_start),
                                                           reinterpret_cast<const long long*>(exp_end), nullptr,
                                                           expert_offset, num_local_experts, 0, tile_rows,
                                                           reinterpret_cast<int4*>(tiles), max_tiles);
  count_launch();
  DLB_CHECK_LAUNCH("build_tiles_kernel");
  return DLB_OK;
}

extern "C" int dlb_moe_build_tiles_masked(const int32_t* masked_m, int num_local_experts, int rows_per_expert,
                                          int32_t* tiles, int max_tiles, void* stream) {
  DLB_REQUIRE(masked_m && tiles, DLB_ERR_INVALID, "build_tiles_masked: null pointer");
  DLB_REQUIRE(num_local_experts > 0 && rows_per_expert > 0 && max_tiles >= 0, DLB_ERR_INVALID,
              "build_tiles_masked: bad sizes");
  DLB_REQUIRE((uintptr_t)tiles % 16 == 0, DLB_ERR_INVALID, "build_tiles_masked: tiles must be 16-byte aligned");
  build_tiles_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(nullptr, nullptr, masked_m, 0, num_local_experts,
                                                           rows_per_expert, 128, reinterpret_cast<int4*>(tiles),
                                                           max_tiles);
  count_launch();
  DLB_CHECK_LAUNCH("build_tiles_kernel");
  return DLB_OK;
}
