// Internal interface of the stable token-by-expert sort (sort.cu), shared with the
// permutation and gating entry points that need ranks inside expert segments.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace dlb {
size_t sort_workspace_size(long long n, int num_experts);
// Any output pointer may be null.  See dlb_sort_by_expert in include/dlblas_b200.h.
int sort_by_expert(const void* ids, int ids_dtype, long long n, int num_experts, long long* sorted_idx,
                   long long* exp_start, long long* exp_end, int* slot_pos, int* rank_in_expert, int* counts,
                   void* ws, size_t ws_bytes, cudaStream_t st);
}  // namespace dlb
