// Grouped (and dense) GEMM on 16-bit operands for sm_100a: C[rows of group g] = A[rows of g] * B[g]^T with
// A [M, K] and B [G, N, K] both K-major, fp32 accumulation in TMEM over the whole K, one rounding to the
// 16-bit output (m_grouped_gemm of dlblas/kernels/grouped_gemm/BF16/m_grouped_gemm.py:235-352, trans_b = True).
//
// Same skeleton as the block-scaled FP8 kernel, without its per-K-block promotion:
//   warp 8   TMA producer: A tile [128 x 128 B] and B tile [256 x 128 B] per 64-element K block
//   warp 9   tcgen05.mma kind::f16 (128 x 256 x 16, four per K block), whole K into one of two TMEM accumulators
//   warps 0-7  drain a finished accumulator (tcgen05.ld), round to the output type into a padded staging tile
//   warps 10-11  send the staging rows out with one bulk copy each
// While a tile is drained and stored the MMA warp already fills the other accumulator.  Waits are bounded.
//
// Two variants of the same kernel.  CTAS = 1: one CTA per 128 x 256 tile.  CTAS = 2: clusters of two CTAs
// compute 256 x 256 tiles with tcgen05.mma.cta_group::2: each CTA loads its 128 rows of A and only half of the
// B tile, the leader CTA issues the MMAs for both, and every CTA drains and stores its own 128 rows.  A single
// CTA moves each operand byte through shared memory twice (TMA write, MMA read: 96 KB per 512 tensor-pipe
// cycles, 1.5 x what the 128 B/clk port delivers); halving the B traffic lifts that bound (measured:
// 1.12 -> 1.44 PFLOP/s on 8192 x 4096 x 7168).  The pair variant is used when the row groups are large enough
// to fill 256-row tiles.  The pair's loads name no cluster-wide delivery: each CTA fetches its own half.
#include "umma.cuh"

namespace dlb {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int A_STAGE_BYTES = BM * UMMA_BK_BYTES;
// per CTA: the whole B tile (CTAS = 1) or its half (CTAS = 2)
template <int CTAS> struct Geo {
  static constexpr int B_STAGE_BYTES = (BN / CTAS) * UMMA_BK_BYTES;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = CTAS == 1 ? 3 : 4;
  static constexpr int STAGING_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = STAGING_OFF + BM * (BN * 2 + 16);
  static constexpr int NUM_BARS = 3 * STAGES + 2 * 2 + 3;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = MISC_OFF + 16 + 1024;
};
constexpr int DRAIN_WARPS = 8;
constexpr int PRODUCER_WARP = 8;
constexpr int MMA_WARP = 9;
constexpr int STORE_WARP0 = 10;
constexpr int STORE_WARPS = 2;
constexpr int NUM_THREADS = 384;
constexpr int TMEM_COLS = 512;
constexpr int TMEM_BUFS = 2;
constexpr int STAGING_ROW_BYTES = BN * 2 + 16;

struct Args16 {
  void* c;
  long long ldc;
  const int4* tiles;     // nullptr: one group, M tiles derived from m
  int m, n, k_bytes;
  int num_m_tiles_static, num_n_tiles;
  // Groups along the reduction dimension (k_grouped_gemm): the operands are A [k_total, m] and B [k_total, n], both
  // MN-major (a row holds one k), tile {g, row0, rows} multiplies columns [row0, row0 + rows) of A by columns
  // [n0, ...) of B over the K rows of group g, kseg[g] = {first K row, number of 64-row K blocks (>= 1), valid rows of
  // the last block (0 ... 64), 0}, and writes rows g * c_group_rows + row0 ... of C.  Otherwise kseg is null, the
  // operands are [rows, k] K-major, the K range is the whole K, B holds one [n, k] matrix per group
  // (b_group_rows = n) and c_group_rows = 0.
  const int4* kseg;
  int group_m_tiles;   // m tiles per group when kseg is given
  int band;            // n tiles per band of the tile order when kseg is given
  // Per-worker tile lists (a worker is a CTA or a pair): worker w runs tiles sched[w * sched_stride + i] for
  // i < sched_count[w].  Null: worker w runs tiles w, w + workers, ...
  const int* sched;
  const int* sched_count;
  int sched_stride;
  int b_group_rows;
  bool b_mn;           // kseg null: B is [groups, k, n] (MN-major, b_group_rows = k) instead of [groups, n, k]
  long long c_group_rows;
  uint32_t idesc;
  int* status;
  unsigned long long timeout_cycles;
};

// kind::f16: fp32 accumulate, A and B K-major, both of format `fmt` (0 = fp16, 1 = bf16), M = 128, N = BN
constexpr uint32_t make_idesc16(uint32_t fmt, int ctas) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((ctas * BM) >> 4) << 24);
}

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One instruction for the pair: M = 256 (128 rows from each CTA), B halves taken from both CTAs.
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Shared-memory descriptor of an MN-major operand tile with 128-byte swizzle: rows of 128 bytes hold 64 consecutive
// M (or N) elements of one k; 64 such rows (8 KB) per block of 64 columns, the blocks 8 KB apart (leading byte offset),
// groups of 8 k rows 1 KB apart (stride byte offset).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
  d |= (uint64_t)(8192 >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Zeroes K rows [valid, 64) of every 64-column block of a stage (whole 128-byte rows, so the swizzle inside a row does
// not matter) and orders the writes before the tensor core's reads.  Called by one whole warp.
__device__ __forceinline__ void clear_k_rows(uint8_t* stage, int blocks, int valid, int lane) {
  const int units = (64 - valid) * 8;
  for (int c = 0; c < blocks; ++c) {
    uint4* p = reinterpret_cast<uint4*>(stage + c * 8192 + valid * 128);
    for (int u = lane; u < units; u += 32) p[u] = make_uint4(0u, 0u, 0u, 0u);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

struct Tile16 {
  int e, row0, rows, n0;
};
constexpr int KG_BAND = 4;   // default n tiles per band in the tile order of k-grouped launches

template <int CTAS> __device__ __forceinline__ Tile16 decode16(const Args16& g, int t) {
  Tile16 ti;
  int m_tile = t / g.num_n_tiles;
  int n_tile = t - m_tile * g.num_n_tiles;
  if (g.kseg != nullptr) {
    // Every group has the same m x n grid of tiles.  Walk it in bands of `band` n tiles, m tile by m tile inside a
    // band, so that the tiles in flight at one time share rows of both operands and a band of B can stay in L2 while
    // A streams past it.  Measured on 128 ragged groups (K 0 ... 10 k): bands of 3 to 8 are within 3 % of one another
    // and up to 10 % faster than whole rows of n tiles; DLBLAS_KGROUP_BAND overrides the default.
    const int per_group = g.group_m_tiles * g.num_n_tiles;
    const int grp = t / per_group, l = t - grp * per_group;
    const int band = l / (g.group_m_tiles * g.band), li = l - band * g.group_m_tiles * g.band;
    const int width = min(g.band, g.num_n_tiles - band * g.band);
    const int mt = li / width;
    m_tile = grp * g.group_m_tiles + mt;
    n_tile = band * g.band + (li - mt * width);
  }
  if (g.tiles != nullptr) {
    const int4 v = __ldg(g.tiles + 1 + m_tile);
    ti.e = v.x;
    ti.row0 = v.y;
    ti.rows = v.z;
  } else {
    ti.e = 0;
    ti.row0 = m_tile * CTAS * BM;
    ti.rows = min(CTAS * BM, g.m - ti.row0);
  }
  ti.n0 = n_tile * BN;
  return ti;
}

template <typename T> __device__ __forceinline__ uint32_t pack16(float a, float b);
template <> __device__ __forceinline__ uint32_t pack16<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack16<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T, int CTAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Args16 g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using G = Geo<CTAS>;
  constexpr int STAGES = G::STAGES;
  constexpr int STAGE_BYTES = G::STAGE_BYTES;
  constexpr bool PAIR = CTAS == 2;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + G::BAR_OFF;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + TMEM_BUFS + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 2 * TMEM_BUFS);
  const uint32_t staged_bar = drain_bar + 8u;
  const uint32_t sfree_bar = drain_bar + 16u;
  auto land_bar = [&](int s) { return drain_bar + 24u + 8u * s; };   // k-grouped launches: this CTA's loads of a stage
  uint8_t* staging = smem + G::STAGING_OFF;
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + G::MISC_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + G::MISC_OFF + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;   // 0 = leader of a pair: it issues the MMAs
  const int worker = blockIdx.x / CTAS;                   // CTA or pair index
  const int workers = gridDim.x / CTAS;
  const int kblocks = (g.k_bytes + UMMA_BK_BYTES - 1) / UMMA_BK_BYTES;
  const int num_m_tiles = g.tiles != nullptr ? __ldg(reinterpret_cast<const int*>(g.tiles)) : g.num_m_tiles_static;
  const int total_tiles = num_m_tiles * g.num_n_tiles;
  const int my_tiles = g.sched != nullptr ? __ldg(g.sched_count + worker)
                                          : (worker < total_tiles ? (total_tiles - worker + workers - 1) / workers : 0);
  const int* my_sched = g.sched != nullptr ? g.sched + (long long)worker * g.sched_stride : nullptr;
  auto tile_at = [&](int i) { return my_sched != nullptr ? __ldg(my_sched + i) : worker + i * workers; };
  const unsigned long long limit = g.timeout_cycles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(land_bar(s), 1);
    }
    for (int b = 0; b < TMEM_BUFS; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), CTAS * DRAIN_WARPS);   // pair: the drain warps of both CTAs release the leader's
    }
    mbar_init(drain_bar, 1);
    mbar_init(staged_bar, DRAIN_WARPS);
    mbar_init(sfree_bar, STORE_WARPS);
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(const_cast<uint32_t*>(tmem_holder))),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(const_cast<uint32_t*>(tmem_holder))),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();   // both CTAs' barriers exist before anything remote touches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == PRODUCER_WARP) {
    uint32_t it = 0;
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i) {
      const int t = tile_at(i);
      const Tile16 ti = decode16<CTAS>(g, t);
      const bool mn = g.kseg != nullptr;
      const int4 ks = mn ? __ldg(g.kseg + ti.e) : make_int4(0, kblocks, 64, 0);
      for (int kb = 0; kb < ks.y; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1u) ^ 1u, abort_flag, limit)) {
          ok = false;
          break;
        }
        const uint32_t a_dst = smem_base + s * STAGE_BYTES;
        const uint32_t b_dst = a_dst + A_STAGE_BYTES;
        if (mn) {
          // MN-major operands: boxes of 64 K rows x 128 bytes (64 columns), one per 64 columns of the tile.  A block
          // that ends inside its box (rows of the next group follow) lands on this CTA's own barrier; the MMA warp
          // clears those rows before the block is used.  Every other block goes the usual way, and the own barrier
          // is stepped by hand so that its phase follows the stage's.
          const bool ragged = kb == ks.y - 1 && ks.z < 64;
          const int ky = ks.x + kb * 64;
          const int ax = 2 * (ti.row0 + (int)rank * BM), bx = 2 * (ti.n0 + (int)rank * (BN / CTAS));
          if (elect_one()) {
            if (ragged) {
              mbar_expect_tx(land_bar(s), STAGE_BYTES);
#pragma unroll
              for (int c = 0; c < BM / 64; ++c) tma_load_2d(a_dst + c * 8192, &tmap_a, ax + 128 * c, ky, land_bar(s));
#pragma unroll
              for (int c = 0; c < BN / CTAS / 64; ++c)
                tma_load_2d(b_dst + c * 8192, &tmap_b, bx + 128 * c, ky, land_bar(s));
            } else {
              mbar_arrive(land_bar(s));
              if constexpr (PAIR) {
                const uint32_t lead_full = mapa(full_bar(s), 0);
                if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
#pragma unroll
                for (int c = 0; c < BM / 64; ++c)
                  tma_load_2d_pair(a_dst + c * 8192, &tmap_a, ax + 128 * c, ky, lead_full);
#pragma unroll
                for (int c = 0; c < BN / CTAS / 64; ++c)
                  tma_load_2d_pair(b_dst + c * 8192, &tmap_b, bx + 128 * c, ky, lead_full);
              } else {
                mbar_expect_tx(full_bar(s), STAGE_BYTES);
#pragma unroll
                for (int c = 0; c < BM / 64; ++c) tma_load_2d(a_dst + c * 8192, &tmap_a, ax + 128 * c, ky, full_bar(s));
#pragma unroll
                for (int c = 0; c < BN / 64; ++c) tma_load_2d(b_dst + c * 8192, &tmap_b, bx + 128 * c, ky, full_bar(s));
              }
            }
          }
          __syncwarp();
          continue;
        }
        const int kx = kb * UMMA_BK_BYTES;
        const int a_row = ti.row0;
        const int b_row = ti.n0 + ti.e * g.b_group_rows;
        // B as [groups, k, n] (b_mn): boxes of 64 K rows x 64 columns at row e * k + 64 kb, as for k-grouped launches
        const int bx = 2 * (ti.n0 + (int)rank * (BN / CTAS)), by = ti.e * g.b_group_rows + kb * 64;
        if constexpr (PAIR) {
          const uint32_t lead_full = mapa(full_bar(s), 0);
          if (elect_one()) {
            if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);      // the loads of both CTAs
            tma_load_2d_pair(a_dst, &tmap_a, kx, a_row + (int)rank * BM, lead_full);
            if (g.b_mn) {
#pragma unroll
              for (int c = 0; c < BN / 2 / 64; ++c) tma_load_2d_pair(b_dst + c * 8192, &tmap_b, bx + 128 * c, by, lead_full);
            } else {
              tma_load_2d_pair(b_dst, &tmap_b, kx, b_row + (int)rank * (BN / 2), lead_full);
            }
          }
        } else if (elect_one()) {
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          tma_load_2d(a_dst, &tmap_a, kx, a_row, full_bar(s));
          if (g.b_mn) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(b_dst + c * 8192, &tmap_b, bx + 128 * c, by, full_bar(s));
          } else {
            tma_load_2d(b_dst, &tmap_b, kx, b_row, full_bar(s));
            tma_load_2d(b_dst + 128 * UMMA_BK_BYTES, &tmap_b, kx, b_row + 128, full_bar(s));
          }
        }
        __syncwarp();
      }
    }
    if (!ok) {
      const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0u;
      for (uint32_t i = first; i < it; ++i)
        mbar_wait(full_bar(i % STAGES), (i / STAGES) & 1u, abort_flag + 1, 40000000ull);
    }
  } else if (warp == MMA_WARP) {
    uint32_t it = 0, tile_no = 0;
    bool ok = true;
    const bool mn = g.kseg != nullptr;
    // The other CTA of a pair issues nothing.  With MN-major operands it still clears the rows past the end of each
    // tile's last K block in its own shared memory and then completes the leader's barrier of that stage.  It follows
    // every use of every stage's barrier, block by block: a parity wait only tells the current phase from the one
    // before it, so a waiter that skipped uses could take an earlier phase for the one it wants.
    for (int i = 0; PAIR && mn && rank != 0 && i < my_tiles && ok; ++i) {
      const int4 ks = __ldg(g.kseg + decode16<CTAS>(g, tile_at(i)).e);
      for (int kb = 0; kb < ks.y; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(land_bar(s), (it / STAGES) & 1u, abort_flag, limit)) {
          ok = false;
          break;
        }
        if (kb == ks.y - 1 && ks.z < 64) {
          clear_k_rows(smem + s * STAGE_BYTES, STAGE_BYTES / 8192, ks.z, lane);
          __syncwarp();
          if (elect_one()) mbar_arrive_cluster(mapa(full_bar(s), 0));
          __syncwarp();
        }
      }
    }
    for (int i = 0; i < my_tiles && ok && rank == 0; ++i, ++tile_no) {
      const int t = tile_at(i);
      const int b = tile_no % TMEM_BUFS;
      if (!mbar_wait(tempty_bar(b), ((tile_no / TMEM_BUFS) & 1u) ^ 1u, abort_flag, limit)) {
        ok = false;
        break;
      }
      const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
      const int4 ks = mn ? __ldg(g.kseg + decode16<CTAS>(g, t).e) : make_int4(0, kblocks, 64, 0);
      const int nkb = ks.y;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % STAGES;
        if (mn && kb == nkb - 1 && ks.z < 64) {
          if (!mbar_wait(land_bar(s), (it / STAGES) & 1u, abort_flag, limit)) {
            ok = false;
            break;
          }
          clear_k_rows(smem + s * STAGE_BYTES, STAGE_BYTES / 8192, ks.z, lane);
          __syncwarp();
          if constexpr (!PAIR) {
            if (elect_one()) mbar_arrive(full_bar(s));   // nothing else completes this stage's barrier
            __syncwarp();
          }
        }
        if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, abort_flag, limit)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_base + s * STAGE_BYTES;
        const bool b_mn = mn || g.b_mn;
        const uint64_t a_desc = mn ? make_smem_desc_mn(a_addr) : make_smem_desc(a_addr);
        const uint64_t b_desc = b_mn ? make_smem_desc_mn(a_addr + A_STAGE_BYTES) : make_smem_desc(a_addr + A_STAGE_BYTES);
        // 16 K further on: two 8-row swizzle atoms (MN-major) or 32 bytes along the row (K-major)
        const uint32_t kstep_a = mn ? (2048u >> 4) : 2u, kstep_b = b_mn ? (2048u >> 4) : 2u;
        if (elect_one()) {
          if constexpr (PAIR) {
#pragma unroll
            for (int kk = 0; kk < UMMA_BK_BYTES / 32; ++kk)
              tc_mma_f16_pair(d_tmem, a_desc + kstep_a * kk, b_desc + kstep_b * kk, g.idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            tc_commit_pair(empty_bar(s));                          // frees the stage in both CTAs
            if (kb == nkb - 1) tc_commit_pair(tfull_bar(b));       // both CTAs' drain warps
          } else {
#pragma unroll
            for (int kk = 0; kk < UMMA_BK_BYTES / 32; ++kk)
              tc_mma_f16(d_tmem, a_desc + kstep_a * kk, b_desc + kstep_b * kk, g.idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            tc_commit(empty_bar(s));
            if (kb == nkb - 1) tc_commit(tfull_bar(b));
          }
        }
        __syncwarp();
      }
    }
    if (!ok && rank == 0) {
      if (elect_one()) {
        if constexpr (PAIR)
          asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(drain_bar)
                       : "memory");
        else
          tc_commit(drain_bar);
      }
      __syncwarp();
      mbar_wait(drain_bar, 0, abort_flag + 1, 40000000ull);
    }
  } else if (warp >= STORE_WARP0) {
    const int ew = warp - STORE_WARP0;
    uint32_t tile_no = 0;
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i, ++tile_no) {
      const int t = tile_at(i);
      const Tile16 ti = decode16<CTAS>(g, t);
      if (!mbar_wait(staged_bar, tile_no & 1u, abort_flag, limit)) {
        ok = false;
        break;
      }
      const uint32_t bytes = (uint32_t)min(BN, g.n - ti.n0) * 2u;
      const int my_row0 = ti.row0 + (int)rank * BM;               // this CTA's 128 rows of the tile
      const int my_rows = min(BM, max(0, ti.rows - (int)rank * BM));
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = ew * 64 + h * 32 + lane;
        if (row < my_rows)
          bulk_store(reinterpret_cast<T*>(g.c) + ((long long)my_row0 + row + ti.e * g.c_group_rows) * g.ldc + ti.n0,
                     smem_u32(staging + row * STAGING_ROW_BYTES), bytes);
      }
      bulk_commit();
      bulk_wait_read();
      __syncwarp();
      if (lane == 0) mbar_arrive(sfree_bar);
    }
    bulk_wait_all();
  } else {
    // ---- drain warps ----
    const int wg = warp >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    uint8_t* srow = staging + r * STAGING_ROW_BYTES + wg * 128 * 2;
    uint32_t tile_no = 0;
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i, ++tile_no) {
      const int t = tile_at(i);
      const int b = tile_no % TMEM_BUFS;
      if (!mbar_wait(tfull_bar(b), (tile_no / TMEM_BUFS) & 1u, abort_flag, limit) ||
          !mbar_wait(sfree_bar, (tile_no & 1u) ^ 1u, abort_flag, limit)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t col0 = lane_addr + (uint32_t)(b * BN + wg * 128);
      uint32_t s0[32], s1[32];
      tmem_ld32(col0, s0);
      tmem_ld32(col0 + 32, s1);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        tmem_ld_wait(s0, s1);
        if (q == 1) {
          // the whole accumulator is in registers: the MMA warp may reuse it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (rank == 0) mbar_arrive(tempty_bar(b));
            else mbar_arrive_cluster(mapa(tempty_bar(b), 0));
          }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t (&s)[32] = half == 0 ? s0 : s1;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            v.x = pack16<T>(__uint_as_float(s[j]), __uint_as_float(s[j + 1]));
            v.y = pack16<T>(__uint_as_float(s[j + 2]), __uint_as_float(s[j + 3]));
            v.z = pack16<T>(__uint_as_float(s[j + 4]), __uint_as_float(s[j + 5]));
            v.w = pack16<T>(__uint_as_float(s[j + 6]), __uint_as_float(s[j + 7]));
            *reinterpret_cast<uint4*>(srow + ((2 * q + half) * 32 + j) * 2) = v;
          }
        }
        if (q == 0) {
          tmem_ld32(col0 + 64, s0);
          tmem_ld32(col0 + 96, s1);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(staged_bar);
    }
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();   // no CTA leaves while its partner may still signal its barriers
  if (threadIdx.x == 0 && *abort_flag != 0 && g.status != nullptr) atomicExch(g.status, DLB_STATUS_TIMEOUT);
  if (warp == MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <typename T, int CTAS>
int launch16(const CUtensorMap& ma, const CUtensorMap& mb, const Args16& g, int grid, cudaStream_t st) {
  auto kern = gemm16_kernel<T, CTAS>;
  constexpr int SMEM_BYTES = Geo<CTAS>::SMEM_BYTES;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES),
                        "cudaFuncSetAttribute(gemm16_kernel)");
    if (rc != DLB_OK) return rc;
    configured[dev] = true;
  }
  if constexpr (CTAS == 1) {
    kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, g);
    DLB_CHECK_LAUNCH("gemm16_kernel");
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, kern, ma, mb, g), "cudaLaunchKernelEx(gemm16_kernel, pairs)");
    if (rc != DLB_OK) return rc;
  }
  count_launch();
  return DLB_OK;
}

// ---- groups along the reduction dimension (k_grouped_gemm) ----------------------------------------------------------
// C[g] = A_g^T B_g with A [k_total, m], B [k_total, n] row-major and group g owning rows [start_g, start_g + size_g).
// Both operands are MN-major for the tensor cores (a row of memory holds one k), which tcgen05.mma takes as they are:
// nothing is transposed or copied.  TMA places no alignment rule on the outer (K) coordinate, so a group may start at
// any row; its last 64-row block may run into the next group's rows, which the MMA warp clears in shared memory.  An
// empty group gets one block with no valid row so that its tiles still run and write zeros.

// One block.  Thread 0 scans the group sizes; all threads then write the tile list {group, row0, rows}.
__global__ void k_group_plan_kernel(const long long* __restrict__ sizes, int groups, long long k_total, int m,
                                    int tile_rows, int4* __restrict__ kseg, int4* __restrict__ tiles) {
  if (threadIdx.x == 0) {
    long long run = 0;
    for (int g = 0; g < groups; ++g) {
      long long sz = sizes[g];
      sz = sz < 0 ? 0 : sz;
      sz = sz > k_total - run ? k_total - run : sz;
      const long long nkb = sz == 0 ? 1 : (sz + 63) / 64;
      kseg[g] = make_int4((int)run, (int)nkb, (int)(sz - 64 * (nkb - 1)), 0);
      run += sz;
    }
  }
  const int m_tiles = (m + tile_rows - 1) / tile_rows;
  if (threadIdx.x == 0) tiles[0] = make_int4(groups * m_tiles, 0, 0, 0);
  for (int i = threadIdx.x; i < groups * m_tiles; i += blockDim.x) {
    const int g = i / m_tiles, t = i - g * m_tiles;
    tiles[1 + i] = make_int4(g, t * tile_rows, min(tile_rows, m - t * tile_rows), 0);
  }
}

// Tile lists for the workers of the GEMM, built in two steps.  Tiles are handed out in tile order,
// group by group, each to the worker that a greedy scheduler would find free first, with a tile's cost taken as its
// K blocks (at least KG_MIN_COST, the part of a tile that does not shrink with K).  All tiles of a group cost the same,
// so inside a group the order of the workers by the time they become free does not change: tile l of the group goes to
// the worker of rank l mod workers, and the order is updated once per group.  Tiles that follow one another in tile
// order (and share rows of A or B) thus start at about the same time whatever the K ranges of the groups before them;
// handing tile t to worker t mod workers lets the workers drift apart by whole tiles once the groups differ in K, and
// the operands were then read from DRAM 4.4 times instead of 2 (32 groups, K ranges uniform in 0 ... 10 k).
constexpr int KG_MIN_COST = 8;

// Step 1, one small block (the loop over the groups is sequential and pays one block barrier per group, so the block is
// no larger than the workers need): for every group the workers in the order in which they become free (who_of) and
// how many tiles each already holds (held_before); at the end every worker's tile count.
__global__ void __launch_bounds__(256)
k_group_schedule_kernel(const int4* __restrict__ kseg, int groups, int tiles_per_group, int workers,
                        int* __restrict__ who_of, int* __restrict__ held_before, int* __restrict__ sched_count) {
  // free_at[b][r] and who[b][r] for rank r, double-buffered so that a group needs one barrier
  __shared__ long long free_at[2][256];
  __shared__ int who[2][256];
  __shared__ int held_of[2][256]; // a worker changes rank from group to group: its tile count travels with it
  __shared__ int cost_of[1024];   // the groups' tile costs, 1024 groups at a time (one global load per group would
                                  // sit on the critical path of the loop below)
  const int r = threadIdx.x;
  if (r < workers) {
    free_at[0][r] = 0;
    who[0][r] = r;
    held_of[0][r] = 0;
  }
  __syncthreads();
  const int full = tiles_per_group / workers, rest = tiles_per_group - full * workers;
  int cur = 0;
  for (int g = 0; g < groups; ++g, cur ^= 1) {
    if ((g & 1023) == 0) {
      for (int j = threadIdx.x; j < min(1024, groups - g); j += blockDim.x)
        cost_of[j] = max(KG_MIN_COST, __ldg(&kseg[g + j]).y);
      __syncthreads();
    }
    // The first `rest` workers take one tile more than the others.  Both parts stay sorted, so the new order is a merge
    // of the two: each worker finds its new rank with one binary search in the other part.
    const long long cost = cost_of[g & 1023];
    if (r < workers) {
      const int me = who[cur][r], held = held_of[cur][r];
      who_of[(long long)g * workers + r] = me;
      held_before[(long long)g * workers + r] = held;      // indexed by rank, like who_of
      const int got = full + (r < rest ? 1 : 0);
      const long long mine = free_at[cur][r] + got * cost;
      int lo, hi, new_rank;
      if (r < rest) {   // after the workers of the other part that are free no later
        lo = rest, hi = workers;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (free_at[cur][mid] + full * cost <= mine) lo = mid + 1; else hi = mid;
        }
        new_rank = r + (lo - rest);
      } else {          // after the workers of the other part that are free strictly earlier
        lo = 0, hi = rest;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (free_at[cur][mid] + (full + 1) * cost < mine) lo = mid + 1; else hi = mid;
        }
        new_rank = (r - rest) + lo;
      }
      free_at[cur ^ 1][new_rank] = mine;
      who[cur ^ 1][new_rank] = me;
      held_of[cur ^ 1][new_rank] = held + got;
    }
    __syncthreads();
  }
  if (r < workers) sched_count[who[cur][r]] = held_of[cur][r];
}

// Step 2, one thread per tile: tile l of group g goes to the worker at rank l mod workers of that group's order, behind
// the tiles the worker already holds.
__global__ void __launch_bounds__(256)
k_group_tile_lists_kernel(const int* __restrict__ who_of, const int* __restrict__ held_before, int groups,
                          int tiles_per_group, int workers, int* __restrict__ sched, int sched_stride) {
  const long long total = (long long)groups * tiles_per_group;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int g = (int)(t / tiles_per_group), l = (int)(t - (long long)g * tiles_per_group);
    const int round = l / workers, rank = l - round * workers;
    const long long at = (long long)g * workers + rank;
    sched[(long long)__ldg(who_of + at) * sched_stride + __ldg(held_before + at) + round] = (int)t;
  }
}

// Maps, arguments and launch shared by the two entry points.  The tensor maps see a as [a_map_rows, a_row_bytes] and b
// as [b_map_rows, b_row_bytes] with boxes of box_rows rows; m rows (columns when kseg is given) of A meet n of B.
static int run_gemm16(const void* a, int64_t a_map_rows, int64_t a_row_bytes, int a_box_rows, const void* b,
                      int64_t b_map_rows, int64_t b_row_bytes, int b_box_rows, int dtype, int64_t m, int64_t n, int64_t k,
                      const int4* kseg, bool b_mn, int b_group_rows, long long c_group_rows, const int32_t* tiles,
                      int max_tiles, int tile_rows, void* c, int64_t ldc, int32_t* status, void* stream,
                      const int* sched = nullptr, const int* sched_count = nullptr, int sched_stride = 0) {
  int rc = check_device();
  if (rc != DLB_OK) return rc;
  CUtensorMap ma, mb;
  if ((rc = make_map_box(&ma, a, (uint64_t)a_map_rows, (uint64_t)a_row_bytes, (uint32_t)a_box_rows)) != DLB_OK) return rc;
  if ((rc = make_map_box(&mb, b, (uint64_t)b_map_rows, (uint64_t)b_row_bytes, (uint32_t)b_box_rows)) != DLB_OK) return rc;
  Args16 g = {};
  g.c = c;
  g.ldc = ldc;
  g.tiles = reinterpret_cast<const int4*>(tiles);
  g.m = (int)m;
  g.n = (int)n;
  g.k_bytes = (int)(2 * k);
  g.kseg = kseg;
  g.group_m_tiles = (int)ceil_div(m, (int64_t)tile_rows);
  const char* band_env = getenv("DLBLAS_KGROUP_BAND");
  g.band = band_env != nullptr && atoi(band_env) > 0 ? atoi(band_env) : KG_BAND;
  g.sched = sched;
  g.sched_count = sched_count;
  g.sched_stride = sched_stride;
  g.b_group_rows = b_group_rows;
  g.b_mn = b_mn;
  g.c_group_rows = c_group_rows;
  const int ctas = tile_rows / BM;
  g.num_m_tiles_static = (int)ceil_div(m, (int64_t)tile_rows);
  g.num_n_tiles = (int)ceil_div(n, (int64_t)BN);
  g.idesc = make_idesc16(dtype == DLB_BF16 ? 1u : 0u, ctas);
  if (kseg != nullptr) g.idesc |= 1u << 15;            // A MN-major
  if (kseg != nullptr || b_mn) g.idesc |= 1u << 16;    // B MN-major
  g.status = status;
  g.timeout_cycles = wait_limit_cycles(DEFAULT_TIMEOUT_CYCLES);
  const int workers = sm_count() / ctas;
  const long long total = (long long)(tiles != nullptr ? max_tiles : g.num_m_tiles_static) * g.num_n_tiles;
  const int grid = ctas * (int)(total < workers ? total : workers);
  cudaStream_t st = (cudaStream_t)stream;
  if (ctas == 2) {
    if (dtype == DLB_BF16) return launch16<__nv_bfloat16, 2>(ma, mb, g, grid, st);
    return launch16<__half, 2>(ma, mb, g, grid, st);
  }
  if (dtype == DLB_BF16) return launch16<__nv_bfloat16, 1>(ma, mb, g, grid, st);
  return launch16<__half, 1>(ma, mb, g, grid, st);
}

}  // namespace
}  // namespace dlb

using namespace dlb;

// b_kn: B is [num_groups, k, n] (read as an MN-major operand) instead of [num_groups, n, k]
static int grouped_gemm_16bit(const void* a, const void* b, bool b_kn, int dtype, int64_t rows, int num_groups, int64_t n,
                              int64_t k, const int32_t* tiles, int max_tiles, int tile_rows, void* c, int64_t ldc,
                              int32_t* status, void* stream) {
  DLB_REQUIRE(rows >= 0 && n > 0 && k > 0 && num_groups > 0, DLB_ERR_INVALID,
              "grouped_gemm_16bit: bad sizes rows=%lld n=%lld k=%lld groups=%d", (long long)rows, (long long)n,
              (long long)k, num_groups);
  DLB_REQUIRE(dtype == DLB_BF16 || dtype == DLB_F16, DLB_ERR_INVALID, "grouped_gemm_16bit: dtype must be bf16 or fp16");
  DLB_REQUIRE(k % 8 == 0 && n % 8 == 0 && ldc % 8 == 0, DLB_ERR_INVALID,
              "grouped_gemm_16bit: k=%lld, n=%lld and ldc=%lld must be multiples of 8 (16-byte rows)", (long long)k,
              (long long)n, (long long)ldc);
  DLB_REQUIRE(!b_kn || k % 64 == 0, DLB_ERR_INVALID,
              "grouped_gemm_16bit: b as [groups, k, n] needs k=%lld to be a multiple of 64 (a K block must not run into "
              "the next group's rows)", (long long)k);
  DLB_REQUIRE(rows < (1ll << 31) && (long long)num_groups * n < (1ll << 31) && (long long)num_groups * k < (1ll << 31) &&
                  2 * k < (1ll << 31) && 2 * n < (1ll << 31),
              DLB_ERR_INVALID, "grouped_gemm_16bit: size too large");
  DLB_REQUIRE(tiles != nullptr || num_groups == 1, DLB_ERR_INVALID, "grouped_gemm_16bit: several groups need a tile list");
  DLB_REQUIRE(tile_rows == 128 || tile_rows == 256, DLB_ERR_INVALID, "grouped_gemm_16bit: tile_rows must be 128 or 256");
  if (rows == 0 || (tiles != nullptr && max_tiles == 0)) return DLB_OK;
  DLB_REQUIRE(a && b && c, DLB_ERR_INVALID, "grouped_gemm_16bit: null pointer");
  DLB_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)c % 16 == 0) &&
                  ((uintptr_t)tiles % 16 == 0),
              DLB_ERR_INVALID, "grouped_gemm_16bit: a, b, c and tiles must be 16-byte aligned");
  if (b_kn)
    return run_gemm16(a, rows, 2 * k, 128, b, (int64_t)num_groups * k, 2 * n, 64, dtype, rows, n, k, nullptr, true, (int)k,
                      0, tiles, max_tiles, tile_rows, c, ldc, status, stream);
  return run_gemm16(a, rows, 2 * k, 128, b, (int64_t)num_groups * n, 2 * k, 128, dtype, rows, n, k, nullptr, false, (int)n,
                    0, tiles, max_tiles, tile_rows, c, ldc, status, stream);
}

extern "C" int dlb_grouped_gemm_16bit(const void* a, const void* b, int dtype, int64_t rows, int num_groups, int64_t n,
                                      int64_t k, const int32_t* tiles, int max_tiles, int tile_rows, void* c,
                                      int64_t ldc, int32_t* status, void* stream) {
  return grouped_gemm_16bit(a, b, false, dtype, rows, num_groups, n, k, tiles, max_tiles, tile_rows, c, ldc, status,
                            stream);
}

extern "C" int dlb_grouped_gemm_16bit_b_kn(const void* a, const void* b, int dtype, int64_t rows, int num_groups,
                                           int64_t n, int64_t k, const int32_t* tiles, int max_tiles, int tile_rows,
                                           void* c, int64_t ldc, int32_t* status, void* stream) {
  return grouped_gemm_16bit(a, b, true, dtype, rows, num_groups, n, k, tiles, max_tiles, tile_rows, c, ldc, status,
                            stream);
}

// Workspace of dlb_k_grouped_gemm_16bit, in bytes: the tile list, the K ranges and the workers' tile lists.
extern "C" int64_t dlb_k_grouped_gemm_workspace_bytes(int64_t k_total, int64_t m, int64_t n, int num_groups,
                                                      int tile_rows) {
  if (k_total < 0 || m <= 0 || n <= 0 || num_groups <= 0 || (tile_rows != 128 && tile_rows != 256)) return -1;
  const int64_t m_tiles = ceil_div(m, (int64_t)tile_rows);
  const int64_t per_group = m_tiles * ceil_div(n, (int64_t)BN);
  // tile lists: at most per_group / workers + 1 tiles per group and worker; sized for any worker count up to 256
  // + per group the workers' order and their tile counts before the group (two ints per worker, up to 256 workers)
  const int64_t sched_ints = 256 + num_groups * (per_group + 256) + 2 * (int64_t)num_groups * 256;
  return 16 * (1 + num_groups * m_tiles) + 16 * (int64_t)num_groups + 4 * sched_ints;
}

extern "C" int dlb_k_grouped_gemm_16bit(const void* a, const void* b, int dtype, int64_t k_total, int64_t m, int64_t n,
                                        const int64_t* group_sizes, int num_groups, int tile_rows, void* workspace,
                                        int64_t workspace_bytes, void* c, int32_t* status, void* stream) {
  DLB_REQUIRE(k_total >= 0 && m > 0 && n > 0 && num_groups > 0, DLB_ERR_INVALID,
              "k_grouped_gemm_16bit: bad sizes k_total=%lld m=%lld n=%lld groups=%d", (long long)k_total, (long long)m,
              (long long)n, num_groups);
  DLB_REQUIRE(dtype == DLB_BF16 || dtype == DLB_F16, DLB_ERR_INVALID, "k_grouped_gemm_16bit: dtype must be bf16 or fp16");
  DLB_REQUIRE(m % 8 == 0 && n % 8 == 0, DLB_ERR_INVALID,
              "k_grouped_gemm_16bit: m=%lld and n=%lld must be multiples of 8 (16-byte rows)", (long long)m, (long long)n);
  DLB_REQUIRE(tile_rows == 128 || tile_rows == 256, DLB_ERR_INVALID, "k_grouped_gemm_16bit: tile_rows must be 128 or 256");
  const int64_t m_tiles = ceil_div(m, (int64_t)tile_rows);
  const int64_t per_group = m_tiles * ceil_div(n, (int64_t)BN);
  const int64_t all_tiles = per_group * num_groups;
  DLB_REQUIRE(k_total < (1ll << 31) - 64 && 2 * m < (1ll << 31) && 2 * n < (1ll << 31) && all_tiles < (1ll << 30),
              DLB_ERR_INVALID, "k_grouped_gemm_16bit: size too large");
  if (k_total == 0) {   // nothing to reduce over: every group is empty
    DLB_REQUIRE(c != nullptr, DLB_ERR_INVALID, "k_grouped_gemm_16bit: null pointer");
    return check_cuda(cudaMemsetAsync(c, 0, (size_t)(2 * num_groups * m * n), (cudaStream_t)stream),
                      "cudaMemsetAsync(k_grouped_gemm_16bit, c)");
  }
  DLB_REQUIRE(a && b && c && group_sizes && workspace, DLB_ERR_INVALID, "k_grouped_gemm_16bit: null pointer");
  DLB_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)c % 16 == 0) &&
                  ((uintptr_t)workspace % 16 == 0),
              DLB_ERR_INVALID, "k_grouped_gemm_16bit: a, b, c and workspace must be 16-byte aligned");
  DLB_REQUIRE(workspace_bytes >= dlb_k_grouped_gemm_workspace_bytes(k_total, m, n, num_groups, tile_rows), DLB_ERR_INVALID,
              "k_grouped_gemm_16bit: workspace of %lld bytes is too small", (long long)workspace_bytes);
  int rc = check_device();
  if (rc != DLB_OK) return rc;
  int4* tiles = reinterpret_cast<int4*>(workspace);
  int4* kseg = tiles + 1 + num_groups * m_tiles;
  int* sched_count = reinterpret_cast<int*>(kseg + num_groups);
  int* sched = sched_count + 256;
  const int max_workers = sm_count() / (tile_rows / BM);
  const int workers = (int)(all_tiles < max_workers ? all_tiles : max_workers);   // as run_gemm16 sizes its grid
  DLB_REQUIRE(workers <= 256, DLB_ERR_INVALID, "k_grouped_gemm_16bit: more than 256 workers");
  const int sched_stride = (int)(num_groups * (per_group / workers + 1));
  cudaStream_t st = (cudaStream_t)stream;
  k_group_plan_kernel<<<1, 256, 0, st>>>(reinterpret_cast<const long long*>(group_sizes), num_groups, k_total, (int)m,
                                         tile_rows, kseg, tiles);
  if ((rc = check_cuda(cudaGetLastError(), "k_group_plan_kernel")) != DLB_OK) return rc;
  count_launch();
  int* who_of = sched + (long long)num_groups * (per_group + 256);
  int* held_before = who_of + (long long)num_groups * 256;
  const int sched_threads = (workers + 31) / 32 * 32;
  k_group_schedule_kernel<<<1, sched_threads, 0, st>>>(kseg, num_groups, (int)per_group, workers, who_of, held_before,
                                                       sched_count);
  if ((rc = check_cuda(cudaGetLastError(), "k_group_schedule_kernel")) != DLB_OK) return rc;
  count_launch();
  k_group_tile_lists_kernel<<<(unsigned)min((long long)ceil_div(all_tiles, (int64_t)256), 1024ll), 256, 0, st>>>(
      who_of, held_before, num_groups, (int)per_group, workers, sched, sched_stride);
  if ((rc = check_cuda(cudaGetLastError(), "k_group_tile_lists_kernel")) != DLB_OK) return rc;
  count_launch();
  return run_gemm16(a, k_total, 2 * m, 64, b, k_total, 2 * n, 64, dtype, m, n, 64, kseg, false, 0, m,
                    reinterpret_cast<const int32_t*>(tiles), (int)(num_groups * m_tiles), tile_rows, c, n, status, stream,
                    sched, sched_count, sched_stride);
}
