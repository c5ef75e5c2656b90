// Block-scaled FP8 (e4m3) GEMMs for sm_100a: dense and grouped over ragged expert
// segments.  One persistent, warp-specialised kernel:
//
//   warp 8  (1 thread)  TMA producer: A tile [128 x 128B] and B tile [BN x 128B] per
//                       128-wide K block into a ring of 128B-swizzled smem stages.
//   warp 9  (1 thread)  issues tcgen05.mma kind::f8f6f4 (128 x BN x 32, four per K block)
//                       into a ring of TMEM accumulators, one accumulator per K block.
//   warps 0-7           promotion: tcgen05.ld each K block's partial product,
//                       acc += partial * a_scale[row, kb] * b_scale[nblk, kb] on the CUDA
//                       cores (the scales are arbitrary fp32, so the hardware block-scale
//                       path, which wants UE8M0 scales, does not apply).  At the end of a tile
//                       they round the accumulators to the 16-bit output type, park them in a
//                       shared-memory staging tile and go straight on to the next tile.
//   warps 10-11         epilogue: rows of the staging tile leave with one bulk copy each
//                       (store / scatter), or are turned into silu(gate)*up, quantised per 128
//                       columns and stored as e4m3 (fused w13 epilogue), while the other roles
//                       already work on the next tile.  (With fp32 output the tile does not fit
//                       the staging buffer and the promotion warps store it themselves.)
//
// (A 16-warp variant, four promotion warps per scheduler partition with 64 accumulator columns
// each, was measured too: 5 % faster on large dense problems, but its 96-register budget spills
// in the fused silu*up epilogue and it was 15 % slower on the grouped w13 GEMM, so the 8-warp
// layout below is the one kept.)
//
// Register budget: an accumulator tile is 128 x BN fp32 = half of the register file at
// BN = 256, and hiding the TMEM load latency needs 64 more staging registers per promotion
// thread, so the promotion warpgroups run at 232 registers and the third warpgroup at 40.
//
// The arithmetic follows dlblas/kernels/fp8_gemm.py:50-59 and
// dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py:95-156 of the reference: fp32
// accumulation over K blocks in increasing order, one rounding to the output type.
//
// All mbarrier waits are bounded (about 2 s of SM clock cycles): a wait that exceeds its limit raises a CTA-wide
// abort flag, every role leaves its loop, the status word is set to DLB_STATUS_TIMEOUT
// and the kernel returns after draining what it issued.
#include "umma.cuh"

namespace dlb {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;              // bytes == elements (e4m3)
constexpr int A_STAGE_BYTES = BM * BK;
constexpr int EPI_WARPS = 8;         // two warpgroups
constexpr int PRODUCER_WARP = 8;
constexpr int MMA_WARP = 9;
constexpr int STORE_WARP0 = 10;       // warps 10 and 11: epilogue out of the staging tile
constexpr int STORE_WARPS = 2;
constexpr int NUM_THREADS = 384;      // three warpgroups
constexpr int REGS_PROMOTION = 232;    // 256 * 232 + 128 * 40 = 384 * 168
constexpr int REGS_OTHER = 40;
constexpr int TMEM_COLS = 512;

struct GemmArgs {
  const float* a_s;
  long long a_s_rs, a_s_ks;   // a_s[row * rs + kb * ks]
  const float* b_s;
  long long b_s_es;           // per-expert stride; inside: [nblk * kblocks + kb]
  void* c;
  long long ldc;
  float* q_scale;             // SWIGLU_QUANT: [rows, n_half/128]
  int quant_mode;
  float quant_eps;
  const int4* tiles;          // nullptr: dense, M tiles derived from m
  int m, n, k;
  int n_half;                 // SWIGLU_QUANT: intermediate size (n / 2)
  int num_m_tiles_static;
  int num_n_tiles;
  int n_tile0;   // first n tile of the launch (a launch may cover a window of the columns; 0 otherwise)
  const long long* sorted_idx;
  const float* weights;
  int* status;
  unsigned long long timeout_cycles;
  int withhold_loads;         // self-test of the time-out path: the producer issues no load
};

// kind::f8f6f4, A and B e4m3 K-major, fp32 accumulate, M = 128, N = bn.
__host__ __device__ constexpr uint32_t make_idesc(int bn, int ctas = 1) {
  return (1u << 4) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)((ctas * BM) >> 4) << 24);
}

// CTAS = 2: pairs of CTAs on 256-row tiles (tcgen05 cta_group::2); every CTA then stages only half of the B tile
template <int BN, int CTAS = 1> struct Cfg {
  static constexpr int B_STAGE_BYTES = (BN / CTAS) * BK;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (BN == 256) ? (CTAS == 2 ? 4 : 3) : 5;
  static constexpr int TMEM_BUFS = TMEM_COLS / BN;
  static constexpr int SEG = BN / 4;  // columns per thread segment (two segments per thread)
  // Staging tile of the epilogue: BM rows of BN 16-bit values.  Rows are padded by 16 bytes so
  // that the 16-byte stores of 32 threads holding 32 different rows spread over all banks.
  static constexpr int STAGING_ROW_BYTES = BN * 2 + 16;
  static constexpr int STAGING_BYTES = BM * STAGING_ROW_BYTES;
  // dynamic smem: stages | staging tile | barriers (full, empty, tmem_full, tmem_empty, drain,
  // staged, staging_free) | misc
  static constexpr int STAGING_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = STAGING_OFF + STAGING_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 2 * TMEM_BUFS + 3;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = MISC_OFF + 16 + 1024;  // + slack for 1024 B alignment
};

struct Tile {
  int e, row0, rows, n0;
};

// The part of tile t that CTA `rank` of a pair works on (CTAS = 2: rows [rank * 128, rank * 128 + 128) of the
// 256-row tile; its `rows` is 0 when the tile ends before them).
template <int BN, int MODE, int CTAS = 1>
__device__ __forceinline__ Tile decode_tile(const GemmArgs& g, int t, int rank = 0) {
  Tile ti;
  const int m_tile = t / g.num_n_tiles;
  const int n_tile = t - m_tile * g.num_n_tiles;
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
  if constexpr (CTAS == 2) {
    ti.row0 += rank * BM;
    ti.rows = min(BM, max(0, ti.rows - rank * BM));
  }
  ti.n0 = (n_tile + g.n_tile0) * (MODE == DLB_EPI_SWIGLU_QUANT ? BN / 2 : BN);
  return ti;
}

template <typename OutT> struct Pack;
template <> struct Pack<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t two(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct Pack<__half> {
  static __device__ __forceinline__ uint32_t two(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// Stores NCOLS accumulators (a compile-time count, multiple of 8) of one row; only the first
// `valid` columns exist.  dst is 16-byte aligned.  Fully unrolled so `acc` stays in registers.
template <typename OutT, int NCOLS>
__device__ __forceinline__ void store_row(OutT* dst, const float (&acc)[NCOLS], int valid) {
  if constexpr (sizeof(OutT) == 4) {
#pragma unroll
    for (int j = 0; j < NCOLS; j += 4) {
      if (j < valid)
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + j) =
            make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < NCOLS; j += 8) {
      if (j < valid) {
        uint4 v;
        v.x = Pack<OutT>::two(acc[j], acc[j + 1]);
        v.y = Pack<OutT>::two(acc[j + 2], acc[j + 3]);
        v.z = Pack<OutT>::two(acc[j + 4], acc[j + 5]);
        v.w = Pack<OutT>::two(acc[j + 6], acc[j + 7]);
        *reinterpret_cast<uint4*>(dst + j) = v;
      }
    }
  }
}

template <int BN, int MODE, typename OutT, int CTAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmArgs g) {
  using C = Cfg<BN, CTAS>;
  constexpr bool PAIR = CTAS == 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + C::BAR_OFF;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * C::STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * C::STAGES + C::TMEM_BUFS + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * C::STAGES + 2 * C::TMEM_BUFS);
  const uint32_t staged_bar = drain_bar + 8u;   // promotion warps -> epilogue warps: tile is in the staging buffer
  const uint32_t sfree_bar = drain_bar + 16u;   // epilogue warps -> promotion warps: staging buffer may be reused
  uint8_t* staging = smem + C::STAGING_OFF;
  constexpr bool STAGED = sizeof(OutT) == 2;
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + C::MISC_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::MISC_OFF + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;   // 0 = leader of a pair: it issues the MMAs
  const int worker = blockIdx.x / CTAS;                   // CTA or pair index
  const int workers = gridDim.x / CTAS;
  const int kblocks = g.k / BK;
  const int num_m_tiles = g.tiles != nullptr ? __ldg(reinterpret_cast<const int*>(g.tiles)) : g.num_m_tiles_static;
  const int total_tiles = num_m_tiles * g.num_n_tiles;
  const unsigned long long limit = g.timeout_cycles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < C::TMEM_BUFS; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), CTAS * EPI_WARPS);   // pair: the promotion warps of both CTAs release the leader's
    }
    mbar_init(drain_bar, 1);
    mbar_init(staged_bar, EPI_WARPS);
    mbar_init(sfree_bar, STORE_WARPS);
    abort_flag[0] = 0;
    abort_flag[1] = 0;   // private flag of the drain waits
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

  if (warp >= EPI_WARPS) {
    // third warpgroup: give registers away, then run the producer / MMA roles
    reg_dec<REGS_OTHER>();
  // The producer and MMA warps run their loops with all 32 lanes converged and elect one lane
  // only around the TMA / tcgen05 instructions: addresses, descriptors and barrier operands then
  // live in uniform registers.  With a single lane running the whole loop the same instructions
  // were issued from per-thread registers and each tcgen05.mma held the warp's scheduler
  // partition for ~120 cycles, starving the two promotion warps that share it.
  if (warp == PRODUCER_WARP) {
    {
      uint32_t it = 0;
      bool ok = true;
      for (int t = worker; t < total_tiles && ok; t += workers) {
        const Tile ti = decode_tile<BN, MODE, CTAS>(g, t, (int)rank);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, limit)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          if (g.withhold_loads) {
            // nothing is loaded: the consumers' waits run into their limit
          } else if constexpr (PAIR) {
            // each CTA fetches its 128 rows of A and its half of the B tile (the gate slab in the leader, the up
            // slab in its partner for the fused w13 epilogue); all of it is counted on the leader's barrier
            const uint32_t lead_full = mapa(full_bar(s), 0);
            if (elect_one()) {
              if (rank == 0) mbar_expect_tx(full_bar(s), 2 * C::STAGE_BYTES);
              tma_load_2d_pair(a_dst, &tmap_a, kb * BK, ti.row0, lead_full);
              const int b_row = (MODE == DLB_EPI_SWIGLU_QUANT) ? ti.e * g.n + (int)rank * g.n_half + ti.n0
                                                                : ti.e * g.n + ti.n0 + (int)rank * (BN / 2);
              tma_load_2d_pair(b_dst, &tmap_b, kb * BK, b_row, lead_full);
            }
          } else if (elect_one()) {
            mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
            tma_load_2d(a_dst, &tmap_a, kb * BK, ti.row0, full_bar(s));
            if constexpr (MODE == DLB_EPI_SWIGLU_QUANT) {
              // gate rows [n0, n0+128) and up rows [n_half + n0, ...+128) of expert e
              tma_load_2d(b_dst, &tmap_b, kb * BK, ti.e * g.n + ti.n0, full_bar(s));
              tma_load_2d(b_dst + 128 * BK, &tmap_b, kb * BK, ti.e * g.n + g.n_half + ti.n0, full_bar(s));
            } else {
#pragma unroll
              for (int h = 0; h < BN / 128; ++h)
                tma_load_2d(b_dst + h * 128 * BK, &tmap_b, kb * BK, ti.e * g.n + ti.n0 + h * 128, full_bar(s));
            }
          }
          __syncwarp();
        }
      }
      if (!ok && !g.withhold_loads) {
        // drain: give the loads of the last STAGES iterations a bounded chance to land
        const uint32_t first = it > (uint32_t)C::STAGES ? it - C::STAGES : 0u;
        for (uint32_t i = first; i < it; ++i)
          mbar_wait(full_bar(i % C::STAGES), (i / C::STAGES) & 1u, abort_flag + 1, 40000000ull);
      }
    }
  } else if (warp == MMA_WARP) {
    {
      constexpr uint32_t idesc = make_idesc(BN, CTAS);
      uint32_t it = 0;
      bool ok = true;
      for (int t = worker; t < total_tiles && ok && rank == 0; t += workers) {
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % C::STAGES;
          const int b = it % C::TMEM_BUFS;
          if (!mbar_wait(full_bar(s), (it / C::STAGES) & 1u, abort_flag, limit) ||
              !mbar_wait(tempty_bar(b), ((it / C::TMEM_BUFS) & 1u) ^ 1u, abort_flag, limit)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * C::STAGE_BYTES;
          const uint64_t a_desc = make_smem_desc(a_addr);
          const uint64_t b_desc = make_smem_desc(a_addr + A_STAGE_BYTES);
          const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
          if constexpr (PAIR) {
            if (elect_one()) {
#pragma unroll
              for (int kk = 0; kk < BK / 32; ++kk)
                tc_mma_f8_pair(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc, kk > 0 ? 1u : 0u);
              tc_commit_pair(empty_bar(s));   // both CTAs' stages
              tc_commit_pair(tfull_bar(b));   // both CTAs' promotion warps
            }
          } else {
            if (elect_one()) {
#pragma unroll
              for (int kk = 0; kk < BK / 32; ++kk) {
                // +32 bytes along K inside the 128 B swizzle row == +2 in the (addr >> 4) field
                tc_mma_f8(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc, kk > 0 ? 1u : 0u);
              }
              tc_commit(empty_bar(s));   // smem stage reusable once these MMAs retire
              tc_commit(tfull_bar(b));   // accumulator ready for the promotion warps
            }
          }
          __syncwarp();
        }
      }
      if (!ok) {
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
    }
  } else if (STAGED) {
    // ---- epilogue warps: empty the staging tile while the next tile is being computed ----
    const int ew = warp - STORE_WARP0;
    uint32_t tile_no = 0;
    bool ok = true;
    for (int t = worker; t < total_tiles && ok; t += workers, ++tile_no) {
      const Tile ti = decode_tile<BN, MODE, CTAS>(g, t, (int)rank);
      if constexpr (MODE == DLB_EPI_SWIGLU_QUANT) {
        // A staging row holds the tile's 128 gate columns, then its 128 up columns, already
        // rounded to OutT.  Reference rounding points: silu(gate)*up -> OutT, then
        // scale = absmax * (1/448), q = h / scale (dlblas/kernels/moe.py:398-417), or the
        // max(absmax, eps) / 448 form of dlblas/kernels/fp8.py:9-182.  Same arithmetic as
        // silu_mul_quant_kernel, bit for bit.
        if (!mbar_wait(staged_bar, tile_no & 1u, abort_flag, limit)) {
          ok = false;
          break;
        }
        const long long groups = g.n_half / 128;
        // half a warp per row, eight columns per lane: two rows per pass, eight independent
        // chains per lane to cover the exp / divide latencies
        const int sub = lane >> 4;
        const int cl = lane & 15;
        for (int row0 = ew * 2; row0 < ti.rows; row0 += 2 * STORE_WARPS) {
          const int row = row0 + sub;
          const bool act = row < ti.rows;
          const uint8_t* srow = staging + (act ? row : row0) * C::STAGING_ROW_BYTES;
          const uint4 gv = *reinterpret_cast<const uint4*>(srow + cl * 16);
          const uint4 uv = *reinterpret_cast<const uint4*>(srow + BN + cl * 16);
          const OutT* gp = reinterpret_cast<const OutT*>(&gv);
          const OutT* up = reinterpret_cast<const OutT*>(&uv);
          float h[8];
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float gt = to_f32<OutT>(gp[j]);
            h[j] = to_f32<OutT>(from_f32<OutT>(silu_fast(gt) * to_f32<OutT>(up[j])));
            amax = fmaxf(amax, fabsf(h[j]));
          }
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          const float scale =
              g.quant_mode == DLB_QUANT_RECIP_MUL ? amax * (1.0f / 448.0f) : fmaxf(amax, g.quant_eps) / 448.0f;
          if (act) {
            const long long p = (long long)ti.row0 + row;
            const uint2 q = quant8_rcp(h, 1.0f / scale);
            *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(g.c) + p * g.ldc + ti.n0 + cl * 8) = q;
            if (cl == 0) g.q_scale[p * groups + ti.n0 / 128] = scale;
          }
        }
      } else {
        // this lane sends rows ew*64 + lane and ew*64 + 32 + lane
        long long crow[2];
        bool valid[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int row = ew * 64 + i * 32 + lane;
          valid[i] = row < ti.rows;
          crow[i] = (long long)ti.row0 + row;
          if constexpr (MODE == DLB_EPI_SCATTER_WEIGHT) {
            if (valid[i]) crow[i] = g.sorted_idx[crow[i]];
          }
        }
        if (!mbar_wait(staged_bar, tile_no & 1u, abort_flag, limit)) {
          ok = false;
          break;
        }
        const uint32_t bytes = (uint32_t)min(BN, g.n - ti.n0) * 2u;   // n % 8 == 0
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (valid[i]) {
            const int row = ew * 64 + i * 32 + lane;
            bulk_store(reinterpret_cast<OutT*>(g.c) + crow[i] * g.ldc + ti.n0,
                       smem_u32(staging + row * C::STAGING_ROW_BYTES), bytes);
          }
        }
        bulk_commit();
        bulk_wait_read();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(sfree_bar);
    }
    bulk_wait_all();
  }
  } else {
    // ---- promotion + epilogue warps ------------------------------------------
    reg_inc<REGS_PROMOTION>();
    const int wg = warp >> 2;                 // 0 or 1
    const int quad = warp & 3;                // TMEM lane quadrant of this warp
    const int r = quad * 32 + lane;           // row inside the tile
    constexpr int SEG = C::SEG;
    // TMEM column offsets of this thread's two segments, and matching output columns
    int seg_col[2];
    if constexpr (MODE == DLB_EPI_SWIGLU_QUANT) {
      seg_col[0] = wg * SEG;                  // gate columns
      seg_col[1] = BN / 2 + wg * SEG;         // up columns
    } else {
      seg_col[0] = wg * 2 * SEG;
      seg_col[1] = wg * 2 * SEG + SEG;
    }
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    uint32_t it = 0;
    uint32_t tile_no = 0;
    bool ok = true;
    for (int t = worker; t < total_tiles && ok; t += workers, ++tile_no) {
      const Tile ti = decode_tile<BN, MODE, CTAS>(g, t, (int)rank);
      const bool row_ok = r < ti.rows;
      const long long p = (long long)ti.row0 + r;          // row of A / sorted position
      // threads without a row read the scales of a row that exists (a pair's second CTA can hold an empty
      // half tile whose first row lies beyond the end of A)
      const float* as_ptr = g.a_s + (row_ok ? p : (long long)min(ti.row0, g.m - 1)) * g.a_s_rs;
      // scale blocks of the two segments
      const float* bs_ptr[2];
      {
        const float* be = g.b_s + (long long)ti.e * g.b_s_es;
        int nb0, nb1;
        if constexpr (MODE == DLB_EPI_SWIGLU_QUANT) {
          nb0 = ti.n0 / 128;
          nb1 = (g.n_half + ti.n0) / 128;
        } else {
          nb0 = (ti.n0 + seg_col[0]) / 128;
          nb1 = (ti.n0 + seg_col[1]) / 128;
          const int nb_max = (g.n + 127) / 128 - 1;
          nb0 = min(nb0, nb_max);
          nb1 = min(nb1, nb_max);
        }
        bs_ptr[0] = be + (long long)nb0 * kblocks;
        bs_ptr[1] = be + (long long)nb1 * kblocks;
      }
      uint64_t acc2[SEG];                 // 2 * SEG fp32 accumulators, packed in pairs
#pragma unroll
      for (int j = 0; j < SEG; ++j) acc2[j] = 0ull;
      // row / weight of the scatter epilogue, fetched now so that the two dependent loads are
      // long done when the tile's last K block arrives
      long long crow = p;
      float row_w = 1.f;
      if constexpr (MODE == DLB_EPI_SCATTER_WEIGHT) {
        if (row_ok) {
          crow = g.sorted_idx[p];
          row_w = g.weights[crow];
        }
      }

      // scales are fetched two K blocks ahead: under full TMA load an L2 round trip can take
      // longer than one K block
      float a_sc = __ldg(as_ptr), b_sc0 = __ldg(bs_ptr[0]), b_sc1 = __ldg(bs_ptr[1]);
      float a_n1 = 0.f, b0_n1 = 0.f, b1_n1 = 0.f;
      if (kblocks > 1) {
        a_n1 = __ldg(as_ptr + g.a_s_ks);
        b0_n1 = __ldg(bs_ptr[0] + 1);
        b1_n1 = __ldg(bs_ptr[1] + 1);
      }
      // Two 32-column staging buffers.  A K block is drained in NB batches of two loads; the
      // loads of the next batch (or of the next K block's first batch) are issued as soon as a
      // staging buffer has been folded into the accumulators, so a load is always in flight.
      constexpr int CH = 2 * SEG / 32;   // 32-column chunks per thread and K block (2 or 4)
      constexpr int NB = CH / 2;
      auto chunk_col = [&](int c) { return (c * 32 < SEG) ? seg_col[0] + c * 32 : seg_col[1] + c * 32 - SEG; };
      uint32_t s0[32], s1[32];
      bool pending = false;              // first batch of the current K block already issued
      for (int kb = 0; kb < kblocks && ok; ++kb, ++it) {
        const int b = it % C::TMEM_BUFS;
        const uint32_t buf_addr = lane_addr + (uint32_t)(b * BN);
        float a_n2 = 0.f, b0_n2 = 0.f, b1_n2 = 0.f;
        if (kb + 2 < kblocks) {
          a_n2 = __ldg(as_ptr + (long long)(kb + 2) * g.a_s_ks);
          b0_n2 = __ldg(bs_ptr[0] + kb + 2);
          b1_n2 = __ldg(bs_ptr[1] + kb + 2);
        }
        if (!pending) {
          if (!mbar_wait(tfull_bar(b), (it / C::TMEM_BUFS) & 1u, abort_flag, limit)) {
            ok = false;
            break;
          }
          tc_fence_after();
          tmem_ld32(buf_addr + chunk_col(0), s0);
          tmem_ld32(buf_addr + chunk_col(1), s1);
        }
        pending = false;
        const float sc0f = a_sc * b_sc0, sc1f = a_sc * b_sc1;
        const uint64_t sc0 = pack2(sc0f, sc0f);
        const uint64_t sc1 = pack2(sc1f, sc1f);
        const bool has_next = kb + 1 < kblocks;
        const int nb_buf = (it + 1) % C::TMEM_BUFS;
        const uint32_t next_addr = lane_addr + (uint32_t)(nb_buf * BN);
#pragma unroll
        for (int q = 0; q < NB; ++q) {
          tmem_ld_wait(s0, s1);
          const bool last = (q == NB - 1);
          if (last) {
            // every column of this accumulator is in registers: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (rank == 0) mbar_arrive(tempty_bar(b));
              else mbar_arrive_cluster(mapa(tempty_bar(b), 0));
            }
          }
          {
            const uint64_t sc = ((2 * q) * 32 < SEG) ? sc0 : sc1;
#pragma unroll
            for (int j = 0; j < 16; ++j) fma2(acc2[(2 * q) * 16 + j], s0[2 * j], s0[2 * j + 1], sc);
          }
          if (!last) {
            tmem_ld32(buf_addr + chunk_col(2 * q + 2), s0);
          } else if (has_next) {
            if (!mbar_wait(tfull_bar(nb_buf), ((it + 1) / C::TMEM_BUFS) & 1u, abort_flag, limit)) {
              ok = false;
            } else {
              tc_fence_after();
              tmem_ld32(next_addr + chunk_col(0), s0);
            }
          }
          {
            const uint64_t sc = ((2 * q + 1) * 32 < SEG) ? sc0 : sc1;
#pragma unroll
            for (int j = 0; j < 16; ++j) fma2(acc2[(2 * q + 1) * 16 + j], s1[2 * j], s1[2 * j + 1], sc);
          }
          if (!last) {
            tmem_ld32(buf_addr + chunk_col(2 * q + 3), s1);
          } else if (has_next && ok) {
            tmem_ld32(next_addr + chunk_col(1), s1);
            pending = true;
          }
        }
        if (!ok) {
          tmem_ld_wait_plain();
          break;
        }
        a_sc = a_n1;
        b_sc0 = b0_n1;
        b_sc1 = b1_n1;
        a_n1 = a_n2;
        b0_n1 = b0_n2;
        b1_n1 = b1_n2;
      }
      if (!ok) break;

      // ---- hand the tile over ------------------------------------------------
      float acc[2 * SEG];
#pragma unroll
      for (int j = 0; j < SEG; ++j) unpack2(acc2[j], acc[2 * j], acc[2 * j + 1]);
      if constexpr (MODE == DLB_EPI_SCATTER_WEIGHT) {
#pragma unroll
        for (int j = 0; j < 2 * SEG; ++j) acc[j] *= row_w;
      }
      if constexpr (STAGED) {
        // the staging tile must have been emptied by the epilogue warps (previous tile)
        if (!mbar_wait(sfree_bar, (tile_no & 1u) ^ 1u, abort_flag, limit)) {
          ok = false;
          break;
        }
        uint8_t* srow = staging + r * C::STAGING_ROW_BYTES;
        // byte offsets of this thread's two segments inside the staging row; the fused w13
        // epilogue wants all gate columns first, then all up columns
        const int off0 = (MODE == DLB_EPI_SWIGLU_QUANT) ? wg * SEG * 2 : seg_col[0] * 2;
        const int off1 = (MODE == DLB_EPI_SWIGLU_QUANT) ? BN + wg * SEG * 2 : seg_col[1] * 2;
#pragma unroll
        for (int j = 0; j < 2 * SEG; j += 8) {
          uint4 v;
          v.x = Pack<OutT>::two(acc[j], acc[j + 1]);
          v.y = Pack<OutT>::two(acc[j + 2], acc[j + 3]);
          v.z = Pack<OutT>::two(acc[j + 4], acc[j + 5]);
          v.w = Pack<OutT>::two(acc[j + 6], acc[j + 7]);
          const int off = (j < SEG) ? off0 + j * 2 : off1 + (j - SEG) * 2;
          *reinterpret_cast<uint4*>(srow + off) = v;
        }
        // the rows leave through the async proxy (bulk copies): order these writes before it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(staged_bar);
      } else {
        if (row_ok) {
          const int col0 = ti.n0 + seg_col[0];
          OutT* dst = reinterpret_cast<OutT*>(g.c) + crow * g.ldc + col0;
          const int ncols = min(2 * SEG, g.n - col0);   // n % 8 == 0
          store_row<OutT, 2 * SEG>(dst, acc, ncols);
        }
      }
    }
  }

  // ---- teardown ----------------------------------------------------------------
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

template <int BN, int MODE, typename OutT, int CTAS = 1>
int launch_one(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& g, int grid, cudaStream_t st) {
  auto kern = gemm_fp8_kernel<BN, MODE, OutT, CTAS>;
  constexpr int SMEM = Cfg<BN, CTAS>::SMEM_BYTES;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM),
                        "cudaFuncSetAttribute(gemm_fp8_kernel)");
    if (rc != DLB_OK) return rc;
    configured[dev] = true;
  }
  if constexpr (CTAS == 1) {
    kern<<<grid, NUM_THREADS, SMEM, st>>>(ma, mb, g);
    DLB_CHECK_LAUNCH("gemm_fp8_kernel");
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, kern, ma, mb, g), "cudaLaunchKernelEx(gemm_fp8_kernel, pairs)");
    if (rc != DLB_OK) return rc;
  }
  count_launch();
  return DLB_OK;
}

template <int MODE>
int launch_typed(int bn, int ctas, int c_dtype, const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& g,
                 int grid, cudaStream_t st) {
  if (ctas == 2) {
    // pairs exist for 256-wide tiles with a 16-bit output (the ones that go through the staging tile)
    if (bn == 256 && c_dtype == DLB_BF16) return launch_one<256, MODE, __nv_bfloat16, 2>(ma, mb, g, grid, st);
    if (bn == 256 && c_dtype == DLB_F16) return launch_one<256, MODE, __half, 2>(ma, mb, g, grid, st);
    return fail(DLB_ERR_INVALID, "256-row tiles need 256-wide tiles and a 16-bit output");
  }
  if (bn == 256) {
    if (c_dtype == DLB_BF16) return launch_one<256, MODE, __nv_bfloat16>(ma, mb, g, grid, st);
    if (c_dtype == DLB_F16) return launch_one<256, MODE, __half>(ma, mb, g, grid, st);
    if constexpr (MODE != DLB_EPI_SWIGLU_QUANT)
      if (c_dtype == DLB_F32) return launch_one<256, MODE, float>(ma, mb, g, grid, st);
  } else {
    if constexpr (MODE != DLB_EPI_SWIGLU_QUANT) {
      if (c_dtype == DLB_BF16) return launch_one<128, MODE, __nv_bfloat16>(ma, mb, g, grid, st);
      if (c_dtype == DLB_F16) return launch_one<128, MODE, __half>(ma, mb, g, grid, st);
      if (c_dtype == DLB_F32) return launch_one<128, MODE, float>(ma, mb, g, grid, st);
    }
  }
  return fail(DLB_ERR_INVALID, "unsupported output dtype %d for this GEMM epilogue", c_dtype);
}


}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" int dlb_fp8_gemm(const void* a, const void* b, const float* a_s, int64_t a_s_row_stride,
                            int64_t a_s_kb_stride, const float* b_s, void* c, int c_dtype, int64_t m, int64_t n,
                            int64_t k, int tile_rows, int32_t* status, void* stream) {
  DLB_REQUIRE(m >= 0 && n > 0 && k > 0, DLB_ERR_INVALID, "fp8_gemm: bad sizes m=%lld n=%lld k=%lld", (long long)m,
              (long long)n, (long long)k);
  DLB_REQUIRE(k % 128 == 0, DLB_ERR_INVALID, "fp8_gemm: k=%lld must be a multiple of 128", (long long)k);
  DLB_REQUIRE(n % 8 == 0, DLB_ERR_INVALID, "fp8_gemm: n=%lld must be a multiple of 8", (long long)n);
  DLB_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), DLB_ERR_INVALID, "fp8_gemm: size too large");
  if (m == 0) return DLB_OK;
  DLB_REQUIRE(a && b && a_s && b_s && c, DLB_ERR_INVALID, "fp8_gemm: null pointer");
  DLB_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)c % 16 == 0), DLB_ERR_INVALID,
              "fp8_gemm: a, b and c must be 16-byte aligned");
  int rc = check_device();
  if (rc != DLB_OK) return rc;
  CUtensorMap ma, mb;
  if ((rc = make_map(&ma, a, (uint64_t)m, (uint64_t)k)) != DLB_OK) return rc;
  if ((rc = make_map(&mb, b, (uint64_t)n, (uint64_t)k)) != DLB_OK) return rc;
  DLB_REQUIRE(tile_rows == 0 || tile_rows == 128 || tile_rows == 256, DLB_ERR_INVALID,
              "fp8_gemm: tile_rows must be 0 (choose), 128 or 256");
  const int sms = sm_count();
  // Pairs of CTAs only on request: with one hand-shake per K block between the MMA warp of the leader and the
  // promotion warps of both CTAs, the cluster-wide signalling doubles the K-block period (measured: 1.04 against
  // 1.96 PFLOP/s on 8192 x 4096 x 7168), although the MMAs themselves get cheaper.
  const int ctas = tile_rows == 256 ? 2 : 1;
  const int m_tiles = (int)ceil_div(m, (int64_t)(ctas * BM));
  // 256-wide tiles feed the tensor cores best; fall back to 128 when that would leave SMs idle
  int bn = 256;
  if (ctas == 1 && m_tiles * ceil_div(n, 256) < sms) bn = 128;
  GemmArgs g = {};
  g.a_s = a_s;
  g.a_s_rs = a_s_row_stride;
  g.a_s_ks = a_s_kb_stride;
  g.b_s = b_s;
  g.b_s_es = 0;
  g.c = c;
  g.ldc = n;
  g.tiles = nullptr;
  g.m = (int)m;
  g.n = (int)n;
  g.k = (int)k;
  g.num_m_tiles_static = m_tiles;
  g.num_n_tiles = (int)ceil_div(n, bn);
  g.status = status;
  g.timeout_cycles = wait_limit_cycles(DEFAULT_TIMEOUT_CYCLES);
  g.withhold_loads = withhold_loads() ? 1 : 0;
  const long long total = (long long)m_tiles * g.num_n_tiles;
  const int workers = sms / ctas;
  const int grid = ctas * (int)(total < workers ? total : workers);
  return launch_typed<DLB_EPI_STORE>(bn, ctas, c_dtype, ma, mb, g, grid, (cudaStream_t)stream);
}

// n_begin, n_count: the window of output columns this launch computes (whole tiles of 256; 0, n = everything);
// sm_margin: SMs left free for kernels of other streams (0 = use them all).
static int moe_grouped_gemm(const void* a, const float* a_s, int64_t rows_a, const void* b, const float* b_s,
                            int num_local_experts, int64_t n, int64_t k, const int32_t* tiles, int max_tiles,
                            int tile_rows, int epilogue, void* c, int c_dtype, int64_t ldc, float* q_scale,
                            int quant_mode, float quant_eps, const int64_t* sorted_idx, const float* weights,
                            int32_t* status, void* stream, int64_t n_begin, int64_t n_count, int sm_margin) {
  DLB_REQUIRE(rows_a >= 0 && n > 0 && k > 0 && num_local_experts > 0 && max_tiles >= 0, DLB_ERR_INVALID,
              "grouped_gemm: bad sizes rows=%lld n=%lld k=%lld experts=%d", (long long)rows_a, (long long)n,
              (long long)k, num_local_experts);
  DLB_REQUIRE(k % 128 == 0, DLB_ERR_INVALID, "grouped_gemm: k=%lld must be a multiple of 128", (long long)k);
  DLB_REQUIRE(n % 128 == 0, DLB_ERR_INVALID, "grouped_gemm: n=%lld must be a multiple of 128", (long long)n);
  DLB_REQUIRE(rows_a < (1ll << 31) && (long long)num_local_experts * n < (1ll << 31) && k < (1ll << 31),
              DLB_ERR_INVALID, "grouped_gemm: size too large");
  if (rows_a == 0 || max_tiles == 0) return DLB_OK;
  DLB_REQUIRE(a && a_s && b && b_s && c && tiles, DLB_ERR_INVALID, "grouped_gemm: null pointer");
  DLB_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)c % 16 == 0) &&
                  ((uintptr_t)tiles % 16 == 0),
              DLB_ERR_INVALID, "grouped_gemm: a, b, c and tiles must be 16-byte aligned");
  int rc = check_device();
  if (rc != DLB_OK) return rc;
  CUtensorMap ma, mb;
  if ((rc = make_map(&ma, a, (uint64_t)rows_a, (uint64_t)k)) != DLB_OK) return rc;
  if ((rc = make_map(&mb, b, (uint64_t)num_local_experts * (uint64_t)n, (uint64_t)k)) != DLB_OK) return rc;
  const bool window = n_begin != 0 || n_count != n;
  DLB_REQUIRE(n_begin >= 0 && n_count > 0 && n_begin + n_count <= n && n_begin % 256 == 0 &&
                  (n_count % 256 == 0 || n_begin + n_count == n),
              DLB_ERR_INVALID, "grouped_gemm: column window [%lld, +%lld) of n=%lld must consist of whole 256-column tiles",
              (long long)n_begin, (long long)n_count, (long long)n);
  DLB_REQUIRE(!window || epilogue != DLB_EPI_SWIGLU_QUANT, DLB_ERR_INVALID,
              "grouped_gemm: the swiglu epilogue pairs gate and up columns and takes no column window");
  DLB_REQUIRE(sm_margin >= 0 && sm_margin < sm_count(), DLB_ERR_INVALID, "grouped_gemm: sm_margin=%d", sm_margin);
  const int sms = sm_count() - sm_margin;
  GemmArgs g = {};
  g.a_s = a_s;
  g.a_s_rs = k / 128;
  g.a_s_ks = 1;
  g.b_s = b_s;
  g.b_s_es = (n / 128) * (k / 128);
  g.c = c;
  g.ldc = ldc;
  g.q_scale = q_scale;
  g.quant_mode = quant_mode;
  g.quant_eps = quant_eps;
  g.tiles = reinterpret_cast<const int4*>(tiles);
  g.m = (int)rows_a;
  g.n = (int)n;
  g.k = (int)k;
  g.n_half = (int)(n / 2);
  g.sorted_idx = reinterpret_cast<const long long*>(sorted_idx);
  g.weights = weights;
  g.status = status;
  g.timeout_cycles = wait_limit_cycles(DEFAULT_TIMEOUT_CYCLES);
  g.withhold_loads = withhold_loads() ? 1 : 0;
  DLB_REQUIRE(tile_rows == 128 || tile_rows == 256, DLB_ERR_INVALID, "grouped_gemm: tile_rows must be 128 or 256");
  const int ctas = tile_rows / BM;
  int bn = 256;
  if (epilogue == DLB_EPI_SWIGLU_QUANT) {
    DLB_REQUIRE(n % 256 == 0, DLB_ERR_INVALID, "grouped_gemm: swiglu epilogue needs n %% 256 == 0 (n=%lld)",
                (long long)n);
    DLB_REQUIRE(q_scale != nullptr, DLB_ERR_INVALID, "grouped_gemm: swiglu epilogue needs q_scale");
    DLB_REQUIRE(ldc % 16 == 0, DLB_ERR_INVALID, "grouped_gemm: ldc must be a multiple of 16 for e4m3 output");
    g.num_n_tiles = (int)(n / 256);
  } else {
    DLB_REQUIRE(epilogue == DLB_EPI_STORE || epilogue == DLB_EPI_SCATTER_WEIGHT, DLB_ERR_INVALID,
                "grouped_gemm: unknown epilogue %d", epilogue);
    if (epilogue == DLB_EPI_SCATTER_WEIGHT)
      DLB_REQUIRE(sorted_idx && weights, DLB_ERR_INVALID, "grouped_gemm: scatter epilogue needs sorted_idx and weights");
    DLB_REQUIRE(ldc % 8 == 0, DLB_ERR_INVALID, "grouped_gemm: ldc must be a multiple of 8");
    if (!window && ctas == 1 && (long long)max_tiles * ceil_div(n, 256) < sms) bn = 128;
    g.num_n_tiles = (int)ceil_div(n_count, bn);
    g.n_tile0 = (int)(n_begin / bn);
  }
  const long long total = (long long)max_tiles * g.num_n_tiles;
  const int workers = sms / ctas;
  const int grid = ctas * (int)(total < workers ? total : workers);
  cudaStream_t st = (cudaStream_t)stream;
  if (epilogue == DLB_EPI_STORE) return launch_typed<DLB_EPI_STORE>(bn, ctas, c_dtype, ma, mb, g, grid, st);
  if (epilogue == DLB_EPI_SCATTER_WEIGHT)
    return launch_typed<DLB_EPI_SCATTER_WEIGHT>(bn, ctas, c_dtype, ma, mb, g, grid, st);
  return launch_typed<DLB_EPI_SWIGLU_QUANT>(bn, ctas, c_dtype, ma, mb, g, grid, st);
}

extern "C" int dlb_moe_grouped_gemm(const void* a, const float* a_s, int64_t rows_a, const void* b, const float* b_s,
                                    int num_local_experts, int64_t n, int64_t k, const int32_t* tiles, int max_tiles,
                                    int tile_rows, int epilogue, void* c, int c_dtype, int64_t ldc, float* q_scale,
                                    int quant_mode, float quant_eps,
                                    const int64_t* sorted_idx, const float* weights, int32_t* status, void* stream) {
  return moe_grouped_gemm(a, a_s, rows_a, b, b_s, num_local_experts, n, k, tiles, max_tiles, tile_rows, epilogue, c,
                          c_dtype, ldc, q_scale, quant_mode, quant_eps, sorted_idx, weights, status, stream, 0, n, 0);
}

extern "C" int dlb_moe_grouped_gemm_window(const void* a, const float* a_s, int64_t rows_a, const void* b,
                                           const float* b_s, int num_local_experts, int64_t n, int64_t k,
                                           const int32_t* tiles, int max_tiles, int tile_rows, int epilogue, void* c,
                                           int c_dtype, int64_t ldc, float* q_scale, int quant_mode, float quant_eps,
                                           const int64_t* sorted_idx, const float* weights, int32_t* status,
                                           void* stream, int64_t n_begin, int64_t n_count, int sm_margin) {
  return moe_grouped_gemm(a, a_s, rows_a, b, b_s, num_local_experts, n, k, tiles, max_tiles, tile_rows, epilogue, c,
                          c_dtype, ldc, q_scale, quant_mode, quant_eps, sorted_idx, weights, status, stream, n_begin,
                          n_count, sm_margin);
}
