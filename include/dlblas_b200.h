/*
 * dlblas_b200 — C ABI of the B200 (sm_100a) FP8 MoE expert path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (cudaStream_t passed as void*).  The caller owns every buffer: inputs,
 * outputs and workspaces; nothing is allocated inside a call and no pointer is
 * kept after return.  Calls
 * return DLB_OK (0) or a negative code; dlb_last_error_string() gives the
 * message of the last failure on the calling thread.  Kernels are enqueued on
 * the given stream and the calls do not synchronise.
 *
 * Each declaration names the interface of the reference project
 * (DeepLink-org/DLBlas, paths relative to its root) that it stands in for.
 */
#ifndef DLBLAS_B200_H
#define DLBLAS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DLB_API __attribute__((visibility("default")))
#else
#define DLB_API
#endif

#define DLB_OK 0
#define DLB_ERR_INVALID (-1)     /* bad shape, dtype, stride or alignment          */
#define DLB_ERR_WORKSPACE (-2)   /* workspace missing or too small                 */
#define DLB_ERR_CUDA (-3)        /* a CUDA runtime / driver call failed            */
#define DLB_ERR_UNSUPPORTED (-4) /* device is not sm_100 or feature not built      */

/* element types */
#define DLB_F32 0
#define DLB_BF16 1
#define DLB_F16 2
#define DLB_I32 3
#define DLB_I64 4

/* scale arithmetic of the 1xG quantisers */
#define DLB_QUANT_RECIP_MUL 0 /* scale = absmax * (1/448), no epsilon  (dlblas/kernels/moe.py:398-417)  */
#define DLB_QUANT_DIV_EPS 1   /* scale = max(absmax, eps) / 448        (dlblas/kernels/fp8.py:44-48)    */

/* epilogues of the grouped GEMM */
#define DLB_EPI_STORE 0          /* C[p, :] = cast(acc)                                          */
#define DLB_EPI_SCATTER_WEIGHT 1 /* C[sorted_idx[p], :] = cast(acc * weights[sorted_idx[p]])     */
#define DLB_EPI_SWIGLU_QUANT 2   /* h = silu(gate)*up with the reference's two bf16 roundings,   */
                                 /* then 1x128 FP8 quantisation: q[p, :], q_scale[p, :]          */

/* Status word written by kernels that wait on barriers (bounded waits). */
#define DLB_STATUS_OK 0
#define DLB_STATUS_TIMEOUT 1

DLB_API int dlb_version(void);
/* Policy of the bounded barrier waits inside the GEMM kernels, for every launch that follows from any thread
 * of the process (no counterpart in the reference, whose one device-side wait spins without a limit,
 * dlblas/kernels/allgather_grpo_loss.py:58-81).  A wait that lasts longer than `limit_cycles` SM clock cycles
 * makes the kernel stop, give back its tensor memory and set the caller's status word to DLB_STATUS_TIMEOUT;
 * 0 restores the default of about two seconds.  `withhold_loads` != 0 is a self-test switch: the role that
 * loads the operands issues nothing, so the first wait of every other role runs out and the time-out path can
 * be exercised (with a small limit) without any fault on the device; results of such a launch are undefined. */
DLB_API int dlb_set_wait_policy(uint64_t limit_cycles, int withhold_loads);
DLB_API const char* dlb_last_error_string(void);
/* Number of kernels launched by this library on the calling thread since the last reset. */
DLB_API int64_t dlb_launch_count(int reset);

/* ---- token-by-expert stable sort -----------------------------------------
 * Replaces _dlblas_get_sorted_idx + _start_end_kernel
 * (dlblas/layers/moe/kernels/fused_moe.py:27-51, 83-88).
 * ids: [num_slots] int32 or int64 expert ids, -1 = not routed here.
 * sorted_idx[p] = flat slot index at sorted position p (stable: `-1` entries first,
 * ascending flat index inside an expert).  exp_start/exp_end: int64 [num_experts],
 * start = end = 0 for an expert without tokens.  Optional outputs (may be NULL):
 * slot_pos[f] = sorted position p of flat slot f (int32); for a slot whose id is not an expert
 * (id < 0, or id >= num_experts) it is stored as -(p + 1) so that the permutation kernels, which skip
 * negative destinations, move no data for it.
 * rank_in_expert[f] = position of slot f inside its expert's segment (int32, -1 for id < 0),
 * counts[e] (int32). */
DLB_API size_t dlb_sort_by_expert_workspace_size(int64_t num_slots, int num_experts);
DLB_API int dlb_sort_by_expert(const void* ids, int ids_dtype, int64_t num_slots, int num_experts,
                       int64_t* sorted_idx, int64_t* exp_start, int64_t* exp_end, int32_t* slot_pos,
                       int32_t* rank_in_expert, int32_t* counts, void* workspace, size_t workspace_bytes,
                       void* stream);

/* Same sort for callers that cannot allocate device memory (no counterpart in the reference).
 * A serving engine that has handed all device memory to its own pool at start-up, or a latency-
 * critical path that must never trigger the allocator's device-wide synchronisation, has no
 * workspace to pass and cannot create one.  This variant keeps the chunk histograms in a fixed
 * array inside the library image (dlb_sort_by_expert_static_capacity() bytes, about 4 MiB, held on
 * every GPU that loads the library until the process exits) and allocates nothing, neither directly
 * nor through a library.  Inputs and outputs are the caller's, as above.
 *  - Limit: fails with DLB_ERR_WORKSPACE when dlb_sort_by_expert_workspace_size(num_slots,
 *    num_experts) exceeds the capacity (only beyond about 1000 experts together with a few hundred
 *    thousand slots; every size at 256 experts fits); use the variant with a workspace then.
 *  - The first call on each device looks up the array's device address; make that call before any
 *    stream capture starts on that device.
 *  - All calls on a device share the one array: calls whose kernels may overlap on the GPU
 *    (different streams, no dependency) race on it and give wrong results; order them.  Nothing
 *    needs to be cleared between calls: each call overwrites every word it later reads. */
DLB_API size_t dlb_sort_by_expert_static_capacity(void);
DLB_API int dlb_sort_by_expert_static(const void* ids, int ids_dtype, int64_t num_slots, int num_experts,
                              int64_t* sorted_idx, int64_t* exp_start, int64_t* exp_end, int32_t* slot_pos,
                              int32_t* rank_in_expert, int32_t* counts, void* stream);

/* Tile list for the grouped GEMMs: tiles[0] = {num_tiles,0,0,0}, tiles[1+i] =
 * {local expert, first row, valid rows (<= 128), 0}.  Needs room for 1 + max_tiles int4.
 * Built on the device from exp_start/exp_end (sorted layout; replaces the E-times
 * over-provisioned grid of fused_moe_blocked_f8_kernel,
 * dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py:69-92, 197-199) or from masked_m
 * (masked layout [E, rows_per_expert, K] of FusedMoELowLatency, dlblas/layers/moe/ep_moe.py:199-261). */
DLB_API int dlb_moe_build_tiles(const int64_t* exp_start, const int64_t* exp_end, int expert_offset,
                        int num_local_experts, int32_t* tiles, int max_tiles, void* stream);
/* Same list with tiles of `tile_rows` rows (128 or 256). */
DLB_API int dlb_moe_build_tiles_rows(const int64_t* exp_start, const int64_t* exp_end, int expert_offset,
                             int num_local_experts, int tile_rows, int32_t* tiles, int max_tiles, void* stream);
DLB_API int dlb_moe_build_tiles_masked(const int32_t* masked_m, int num_local_experts, int rows_per_expert,
                               int32_t* tiles, int max_tiles, void* stream);

/* ---- 1xG FP8 (e4m3) quantisation -------------------------------------------
 * Replaces quant_fp8 (dlblas/kernels/moe.py:377-474), per_token_group_quant_fp8
 * (dlblas/kernels/fp8.py:9-182) and tma_align_input_scale (dlblas/kernels/quant_dequant.py:22-83,
 * through the scale strides).  x: [m, k] with row stride ldx (elements).  q: [rows_out, k]
 * e4m3, scales fp32 at scales[row * scale_row_stride + group * scale_group_stride].
 * dst_pos == NULL: output row = input row.  Otherwise input row t is written to rows
 * dst_pos[t * fanout + j], j < fanout (negative entries skipped): the quantiser fused
 * with the token-by-expert permutation. */
DLB_API int dlb_quant_fp8(const void* x, int x_dtype, int64_t m, int64_t k, int64_t ldx, int group_size, int mode,
                  float eps, void* q, float* scales, int64_t scale_row_stride, int64_t scale_group_stride,
                  const int32_t* dst_pos, int fanout, void* stream);

/* Row permutation of already quantised rows (+ their scales): the data movement of
 * ep_scatter (dlblas/kernels/fused_moe_v3.py:49-93) with deterministic destinations. */
DLB_API int dlb_permute_rows(const void* q, int64_t row_bytes, const float* scales, int64_t groups, int64_t m,
                     const int32_t* dst_pos, int fanout, void* out_q, float* out_scales, void* stream);

/* ---- activation -------------------------------------------------------------
 * silu_and_mul (dlblas/layers/moe/kernels/activation.py:17-95, dlblas/kernels/activation.py:89-131):
 * out[r, j] = cast(silu_f32(in[r, j]) * in[r, n + j]). */
DLB_API int dlb_silu_and_mul(const void* gate_up, int dtype, int64_t rows, int64_t n, int64_t ld_in, void* out,
                     int64_t ld_out, void* stream);
/* Fused silu*up + 1x128 quantisation.  round_silu != 0 rounds silu(gate) to the input
 * dtype before the multiply (silu_and_mul_masked_post_quant_fwd, dlblas/kernels/moe.py:204-319);
 * round_silu == 0 rounds only the product (silu_and_mul followed by quant_fp8,
 * dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py:313-315).  masked_m != NULL: input is
 * [experts, rows_per_expert, 2n] and only rows < masked_m[e] are processed. */
DLB_API int dlb_silu_mul_quant(const void* gate_up, int dtype, int64_t rows, int64_t n, int quant_mode, float eps,
                       int round_silu, const int32_t* masked_m, int64_t rows_per_expert, void* q,
                       float* scales, void* stream);

/* ---- FP8 block-scaled GEMMs (tcgen05 + TMA) ----------------------------------
 * fp8_gemm (dlblas/kernels/fp8_gemm.py:17-89): C[m,n] = sum_kb (A_kb . B_kb^T) a_s[m,kb] b_s[n/128,kb].
 * a: [m,k] e4m3 row-major, b: [n,k] e4m3 row-major, a_s fp32 at a_s[row*a_s_row_stride + kb*a_s_kb_stride],
 * b_s fp32 [ceil(n/128), k/128] row-major, c: [m,n] of c_dtype (DLB_BF16/F16/F32).  k % 128 == 0,
 * n % 8 == 0.  tile_rows: 0 or 128 = one CTA per 128-row tile, 256 = pairs of CTAs on 256-row tiles (tcgen05
 * cta_group::2; 16-bit outputs only; same results, currently slower: see gemm_fp8.cu).  status (may be NULL): device int set
 * to DLB_STATUS_TIMEOUT if a bounded wait gave up. */
DLB_API int dlb_fp8_gemm(const void* a, const void* b, const float* a_s, int64_t a_s_row_stride, int64_t a_s_kb_stride,
                 const float* b_s, void* c, int c_dtype, int64_t m, int64_t n, int64_t k, int tile_rows,
                 int32_t* status, void* stream);

/* Grouped GEMM over ragged expert segments; replaces fused_moe_blocked_f8_kernel + launcher
 * (dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py:30-242) and the DeepGEMM calls
 * m_grouped_fp8_gemm_nt_contiguous / _masked (dlblas/kernels/fused_moe_v3.py:235-245,
 * dlblas/layers/moe/ep_moe.py:180-197).  a: [rows_a, k] e4m3 in expert-contiguous order,
 * a_s: [rows_a, k/128]; b: [experts, n, k] e4m3; b_s: [experts, n/128, k/128]; tiles from
 * dlb_moe_build_tiles* with tiles of `tile_rows` rows (128, or 256 = pairs of CTAs: same results, currently slower).  Epilogues: see DLB_EPI_*.  For DLB_EPI_SWIGLU_QUANT n is the width of
 * b (2 * intermediate, gate rows first), c receives e4m3 [rows_a, n/2] and q_scale fp32 [rows_a, n/256];
 * quant_mode / quant_eps choose the scale arithmetic of that re-quantisation (DLB_QUANT_*). */
DLB_API int dlb_moe_grouped_gemm(const void* a, const float* a_s, int64_t rows_a, const void* b, const float* b_s,
                         int num_local_experts, int64_t n, int64_t k, const int32_t* tiles, int max_tiles,
                         int tile_rows, int epilogue, void* c, int c_dtype, int64_t ldc, float* q_scale,
                         int quant_mode, float quant_eps,
                         const int64_t* sorted_idx, const float* weights, int32_t* status, void* stream);
/* The same over a window of the output columns: only columns [n_begin, n_begin + n_count) of c are computed (whole
 * tiles of 256 columns; not with DLB_EPI_SWIGLU_QUANT), on at most (SMs - sm_margin) CTAs, so that a caller can hand
 * the finished columns to a kernel of another stream (the expert-parallel push of the first half of the hidden
 * dimension runs on the SMs left free while the second half is computed). */
DLB_API int dlb_moe_grouped_gemm_window(const void* a, const float* a_s, int64_t rows_a, const void* b, const float* b_s,
                                int num_local_experts, int64_t n, int64_t k, const int32_t* tiles, int max_tiles,
                                int tile_rows, int epilogue, void* c, int c_dtype, int64_t ldc, float* q_scale,
                                int quant_mode, float quant_eps, const int64_t* sorted_idx, const float* weights,
                                int32_t* status, void* stream, int64_t n_begin, int64_t n_count, int sm_margin);

/* ---- combine -----------------------------------------------------------------
 * out[t, :] = cast(sum_j y[t*top_k + j, :]) with fp32 accumulation in slot order: the
 * `intermediate_cache2.sum(dim=1)` of dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py:337.
 * ids (may be NULL; int32/int64 [tokens*top_k]): slots whose id is outside [id_lo, id_hi) count as
 * zero rows and are not read (the reference zero-fills them instead, :291, :317).  skip_unrouted_rows != 0:
 * a token none of whose slots is in range is not written at all (padding rows of a receive buffer). */
DLB_API int dlb_moe_sum_topk(const void* y, int dtype, int64_t tokens, int top_k, int64_t h, const void* ids,
                     int ids_dtype, int64_t id_lo, int64_t id_hi, int skip_unrouted_rows, void* out, void* stream);
/* ep_gather (dlblas/kernels/fused_moe_v3.py:159-233): out[t] = sum_j w[t,j] * in[index[t,j]] over
 * slots with ids[t,j] >= 0, fp32 accumulation in slot order.  ids/index: int32 or int64 (idx_dtype). */
DLB_API int dlb_ep_gather(const void* in, int dtype, int64_t h, const void* ids, const void* index, int idx_dtype,
                  const float* weights, int64_t tokens, int top_k, void* out, void* stream);
/* ep_scatter (dlblas/kernels/fused_moe_v3.py:19-155): expert_start_loc = exclusive cumsum of
 * counts, m_indices[row] = expert of the row, output_index[t,j] = destination row (token-major,
 * slot-minor order inside an expert: deterministic), rows and scales copied.  ids int32 or int64. */
DLB_API size_t dlb_ep_scatter_workspace_size(int64_t tokens, int top_k, int num_experts);
DLB_API int dlb_ep_scatter(const void* x, int64_t row_bytes, const float* x_scale, int64_t groups, const void* ids,
                   int idx_dtype, int64_t tokens, int top_k, const int32_t* counts, int num_experts,
                   int32_t* expert_start_loc, void* out_x, float* out_scale, int32_t* m_indices,
                   int64_t m_indices_len, void* output_index, void* workspace, size_t workspace_bytes,
                   void* stream);

/* Destination ranks of an expert-parallel dispatch (the layout step of DeepEP's
 * Buffer.get_dispatch_layout, dlblas/layers/moe/token_dispatcher.py:330): dest[t*world + r] = r if any
 * of token t's ids belongs to rank r (ids / num_local_experts == r), else world.  Sorting this array
 * with dlb_sort_by_expert(num_experts = world) yields every (token, rank) pair's row in the send buffer. */
DLB_API int dlb_ep_dest_ranks(const void* ids, int ids_dtype, int64_t tokens, int top_k, int num_local_experts,
                      int world, int32_t* dest, void* stream);

/* ---- expert-parallel exchange by peer-to-peer stores ------------------------------------------
 * In-kernel replacement of deep_ep.Buffer.dispatch / combine (dlblas/layers/moe/token_dispatcher.py:345,
 * 427) for GPUs of one NVLink domain.  Every rank holds receive buffers of `world` regions of
 * `region_rows` rows (region s = rows sent by rank s); peer_* are arrays of `world` device pointers to
 * the same buffer on every rank (symmetric allocation).  The caller puts a cross-rank barrier on the
 * stream after each push before the destination reads.
 * dlb_p2p_quant_push: per_token_group_quant_fp8 arithmetic (mode/eps as in dlb_quant_fp8, groups of 128)
 *   fused with the dispatch: token t's e4m3 row, scales and `meta_ints` int32 of metadata are stored into
 *   region my_rank, row within[t*world + r], of every rank r with within >= 0; counts[r] (rows sent to r)
 *   is stored into peer_counts[r][my_rank].
 * dlb_p2p_unpack_meta: on the receiver, metadata rows (top_k global ids, then at int offset meta_ints/2 the
 *   top_k weights' bit patterns) -> local ids int64 (-1 for other ranks' experts and unused rows) + weights.
 * dlb_p2p_push_rows: combine direction; row j < counts[s] of region s goes to rank s, region my_rank, row j. */
DLB_API int dlb_p2p_quant_push(const void* x, int x_dtype, int64_t tokens, int64_t k, int64_t ldx, int mode, float eps,
                       const int32_t* within, int world, int my_rank, int64_t region_rows,
                       const void* const* peer_q, const void* const* peer_scales, const void* const* peer_meta,
                       const int32_t* meta, int meta_ints, const void* const* peer_counts, const int32_t* counts,
                       void* stream);
DLB_API int dlb_p2p_unpack_meta(const int32_t* meta, int meta_ints, int top_k, const int32_t* counts, int world,
                        int64_t region_rows, int expert_lo, int num_local_experts, int64_t* ids, float* weights,
                        void* stream);
DLB_API int dlb_p2p_push_rows(const void* src, int64_t row_bytes, const int32_t* counts, int world, int my_rank,
                      int64_t region_rows, const void* const* peer_dst, void* stream);
/* Expert-side combine fused with the push: out row = sum (fp32, slot order) of y[row * top_k + q] over the slots q
 * whose local expert id ids[row, q] is >= 0, rounded to dtype and stored into the source rank's buffer like
 * dlb_p2p_push_rows does.  y [rows * top_k, h] bf16 / fp16, ids int64 [rows, top_k]. */
DLB_API int dlb_p2p_sum_push(const void* y, int dtype, const int64_t* ids, int top_k, int64_t h, const int32_t* counts,
                     int world, int my_rank, int64_t region_rows, const void* const* peer_dst, void* stream);
/* The same for columns [col_begin, col_begin + col_count) of every row (multiples of 8), on at most max_blocks thread
 * blocks of 256 threads when max_blocks > 0. */
DLB_API int dlb_p2p_sum_push_cols(const void* y, int dtype, const int64_t* ids, int top_k, int64_t h, const int32_t* counts,
                          int world, int my_rank, int64_t region_rows, const void* const* peer_dst, void* stream,
                          int64_t col_begin, int64_t col_count, int max_blocks);

/* Barrier among the ranks (one per GPU) between the push phases above; stands in for the ordering DeepEP's
 * `Buffer.dispatch` / `combine` provide inside the library (dlblas/layers/moe/token_dispatcher.py:345-357, 427-433).
 * peer_signals[r] points at rank r's array of `world` 32-bit words (zero at start, in memory every rank can
 * store to); `counter` is this rank's own count of barriers on these words (one 32-bit word in device memory, zero
 * at start): the kernel advances it, so a launch replayed from a CUDA graph keeps counting; every rank must run the
 * same sequence of barriers.  The wait is bounded by `limit_ns`: on expiry *status becomes DLB_STATUS_TIMEOUT and the
 * kernel returns. */
DLB_API int dlb_p2p_barrier(const void* const* peer_signals, int world, int my_rank, uint32_t* counter, uint64_t limit_ns,
                    int32_t* status, void* stream);

/* Low-latency (decode) exchange on the masked layout [E_local, rows_per_expert, k], in place of
 * Buffer.low_latency_dispatch / low_latency_combine (dlblas/layers/moe/token_dispatcher.py:496-535, 567-582), with no
 * host round trip: dlb_p2p_all_gather_small shares the per-expert pair counts (`bytes` of this rank's vector land in
 * slot "my rank" of every peer's array), dlb_p2p_ll_quant_push quantises each token once
 * (per_token_group_quant_fp8 arithmetic) and stores it for every routed slot f into row pair_row[f] of rank
 * pair_rank[f] (negative: dropped), and dlb_p2p_push_rows_indexed sends row i of the experts' output to row
 * row_pos[i] of rank row_rank[i] (negative: not sent). */
DLB_API int dlb_p2p_all_gather_small(const void* src, int64_t bytes, int world, int my_rank, const void* const* peer_dst,
                             void* stream);
/* The index arithmetic between the two: from the all-gathered counts [world, cnt_stride] (int32), this rank's expert ids
 * topk_ids int64 [pairs] and their rank_in_expert (dlb_sort_by_expert) it writes, for the rank as a source, pair_rank /
 * pair_row / pair_pos int32 [pairs] (pair_pos: row of the own return buffer, ordered by expert, then by that rank) and
 * ids_sent (the id, -1 for a slot that is not sent: no expert, or the expert's block of rows_per_expert rows is full);
 * for the rank as an owner, masked_m int32 [num_local_experts] and row_rank / row_pos int32
 * [num_local_experts * rows_per_expert] as dlb_p2p_push_rows_indexed takes them. */
DLB_API int dlb_p2p_ll_plan(const int32_t* counts, int cnt_stride, int world, int num_experts, int my_rank,
                    int num_local_experts, int rows_per_expert, const int64_t* topk_ids, const int32_t* rank_in_expert,
                    int64_t pairs, int32_t* pair_rank, int32_t* pair_row, int32_t* pair_pos, int32_t* ids_sent,
                    int32_t* masked_m, int32_t* row_rank, int32_t* row_pos, void* stream);
DLB_API int dlb_p2p_ll_quant_push(const void* x, int x_dtype, int64_t tokens, int64_t k, int64_t ldx, int mode, float eps,
                          const int32_t* pair_rank, const int32_t* pair_row, int top_k, int world,
                          const void* const* peer_q, const void* const* peer_scales, void* stream);
DLB_API int dlb_p2p_push_rows_indexed(const void* src, int64_t row_bytes, int64_t rows, const int32_t* row_rank,
                              const int32_t* row_pos, int world, const void* const* peer_dst, void* stream);
/* The same for a masked layout [num_local_experts, rows_per_expert, row_bytes] of which only the first masked_m[e] rows
 * of every expert are in use: the kernel walks those rows only (a decode step uses a few hundred of tens of
 * thousands). */
DLB_API int dlb_p2p_push_rows_masked(const void* src, int64_t row_bytes, const int32_t* masked_m, int num_local_experts,
                             int rows_per_expert, const int32_t* row_rank, const int32_t* row_pos, int world,
                             const void* const* peer_dst, void* stream);

/* ---- 16-bit grouped GEMM -----------------------------------------------------------------
 * m_grouped_gemm with trans_b = True (dlblas/kernels/grouped_gemm/BF16/m_grouped_gemm.py:235-352):
 * c[row, :] = a[row, :] * b[g]^T for the rows of group g; a [rows, k] and b [num_groups, n, k] bf16 or fp16,
 * K-major; c [rows, ldc] of the same type, fp32 accumulation.  `tiles` is a tile list over the groups' row ranges
 * built by dlb_moe_build_tiles_rows with the same `tile_rows` (NULL: one group, dense).  tile_rows = 128: one
 * CTA per tile; 256: pairs of CTAs on 256-row tiles (tcgen05 cta_group::2), the faster choice when groups hold
 * several hundred rows.  k, n, ldc multiples of 8. */
DLB_API int dlb_grouped_gemm_16bit(const void* a, const void* b, int dtype, int64_t rows, int num_groups, int64_t n,
                           int64_t k, const int32_t* tiles, int max_tiles, int tile_rows, void* c, int64_t ldc,
                           int32_t* status, void* stream);
/* The same with b as [num_groups, k, n] (m_grouped_gemm's default, trans_b = False): the tensor cores read b as an
 * MN-major operand, nothing is transposed.  k must be a multiple of 64. */
DLB_API int dlb_grouped_gemm_16bit_b_kn(const void* a, const void* b, int dtype, int64_t rows, int num_groups, int64_t n,
                                int64_t k, const int32_t* tiles, int max_tiles, int tile_rows, void* c, int64_t ldc,
                                int32_t* status, void* stream);

/* k_grouped_gemm (dlblas/kernels/grouped_gemm/BF16/k_grouped_gemm.py:126-176, :254-330): groups along the reduction
 * dimension.  a [k_total, m] and b [k_total, n] row-major bf16 or fp16; group g owns the next group_sizes[g] rows of
 * both (int64 on the device; the sizes are clipped to k_total); c [num_groups, m, n] of the same type with
 * c[g] = a_g^T b_g, fp32 accumulation, zeros for an empty group.  m and n multiples of 8.  The tensor cores read both
 * operands where they lie (MN-major tcgen05 descriptors): nothing is transposed or copied.  `workspace`
 * (dlb_k_grouped_gemm_workspace_bytes bytes, 16-byte aligned, device memory) holds the K ranges, the tile list over
 * [group, m tile, n tile] and the per-CTA tile order, all built on the device; tile_rows as for
 * dlb_grouped_gemm_16bit.  Nothing synchronises with the host. */
DLB_API int64_t dlb_k_grouped_gemm_workspace_bytes(int64_t k_total, int64_t m, int64_t n, int num_groups, int tile_rows);
DLB_API int dlb_k_grouped_gemm_16bit(const void* a, const void* b, int dtype, int64_t k_total, int64_t m, int64_t n,
                             const int64_t* group_sizes, int num_groups, int tile_rows, void* workspace,
                             int64_t workspace_bytes, void* c, int32_t* status, void* stream);

/* ---- training-side permutation (dlblas/kernels/permute/moe_triton_kernels.py) ------------------
 * row_id_map int32 [top_k * tokens], k-major: destination row of (token, slot) in the permuted tensor, -1 for
 * unrouted slots.  Permute forward is dlb_sort_by_expert + dlb_permute_rows.
 * dlb_unpermute = moe_recover_topk_op_triton (:274-301) and, with probs = NULL, moe_permute_topk_bwd_op
 * (:190-213): out[t] = sum_k prob[t,k] * in[row_id_map[k,t]], rounded to the tensor type after every product
 * and add.  dlb_unpermute_bwd = moe_recover_topk_bwd_op_triton (:480-528): act_grad fp32 [rows, h] (rows that no
 * slot maps to are left untouched: zero them first), prob_grad fp32 [tokens, top_k]. */
DLB_API int dlb_unpermute(const void* in, int dtype, const int32_t* row_id_map, const float* probs, int64_t tokens,
                  int top_k, int64_t h, void* out, void* stream);
DLB_API int dlb_unpermute_bwd(const void* grad_out, const void* fwd_in, int dtype, const int32_t* row_id_map,
                      const float* probs, int64_t tokens, int top_k, int64_t h, float* act_grad, float* prob_grad,
                      void* stream);

/* ---- expert-parallel load balancing ------------------------------------------------
 * map_logic_to_physical_idx_hash_random (dlblas/kernels/moe.py:524-579): every (token, slot) of topk_idx
 * [tokens, top_k] (int32 or int64) is sent to one of the logcnt[e] physical replicas log2phy[e, 0..) of its
 * logical expert e, chosen by a 32-bit hash of (token, slot, seed); -1 for negative ids and for experts
 * without replicas.  physical_idx int32 [tokens, top_k]. */
DLB_API int dlb_eplb_map_hash(const void* topk_idx, int ids_dtype, const int32_t* log2phy, const int32_t* logcnt,
                      int64_t tokens, int top_k, int num_logical, int max_replica, uint32_t seed,
                      int32_t* physical_idx, void* stream);

/* ---- routing -------------------------------------------------------------------
 * topk(softmax(logits, fp32), k) with lowest-index tie-break, optional w / sum(w): the routing the
 * reference's callers run in torch (tests/kernels/test_fused_moe_v2.py:100-102) + _renormalize
 * (dlblas/layers/moe/kernels/blocked_fp8_fused_moe.py:245-250).  weights fp32 [t,k]; ids int32/int64. */
DLB_API int dlb_route_softmax_topk(const void* logits, int dtype, int64_t tokens, int experts, int top_k,
                           int renormalize, float* weights, void* ids, int ids_dtype, void* stream);
/* biased_grouped_topk (dlblas/kernels/moe.py:477-521): sigmoid scores + bias, group score = top-2 sum,
 * keep topk_group groups, top-k inside, weights = unbiased scores (renormalised on request).
 * Slots come out in descending biased score, ties to the lowest index. */
DLB_API int dlb_route_grouped_topk(const void* logits, int dtype, const float* bias, int64_t tokens, int experts,
                           int num_groups, int topk_group, int top_k, int renormalize, float* weights,
                           int32_t* ids, void* stream);
/* dlblas.topk_gating forward (dlblas/__init__.py:15-25, dlblas/kernels/topk_gating.py:245-268 and the
 * part1/2/3 kernels): capacity-limited softmax top-k gating.  Outputs: l_aux (1 element, logits dtype),
 * ec_idx int32 [k*t] (k-major), gate weights [k*t] (logits dtype), select int64 [experts*capacity]. */
DLB_API size_t dlb_topk_gating_workspace_size(int64_t tokens, int experts, int top_k);
DLB_API int dlb_topk_gating(const void* logits, int dtype, int64_t tokens, int experts, int top_k, int64_t capacity,
                    void* l_aux, int32_t* ec_idx, void* gate_weights, int64_t* select, void* workspace,
                    size_t workspace_bytes, void* stream);
/* Backward of dlb_topk_gating (TopKGatingFunc.backward, dlblas/kernels/topk_gating.py:270-285;
 * topk_gating_bwd.py:13-68): gradient of l_aux and, if grad_weights (logits dtype, [k*tokens]) is given, of
 * token_exp_weights with respect to the logits.  `workspace` is the forward call's workspace, unmodified.
 * The reference's own weight path (topk_gating.py:139-242) cannot be reached through autograd (it reads the
 * gradient of the integer index output) and divides the saved weights by the denominator twice; this entry
 * computes the true gradient.  grad_l_aux is a device scalar of the logits dtype. */
DLB_API int dlb_topk_gating_bwd(const void* workspace, size_t workspace_bytes, int dtype, int64_t tokens, int experts,
                        int top_k, int64_t capacity, const void* grad_l_aux, const void* grad_weights,
                        void* grad_logits, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DLBLAS_B200_H */
