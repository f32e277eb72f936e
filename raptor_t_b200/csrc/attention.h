// error_word_dev: device word the kernel reports a given-up wait in; nullptr selects the
// library's per-device word (allocated on first use).
// Internal launcher of the block-sparse attention kernel (device work list given
// as raw pointers) shared by the C ABI and the encoder object.
#pragma once
#include <cuda_runtime.h>

#include "metadata.h"

namespace rt {

rt_status check_config(const rt_config* cfg);

// Split lists: groups of partial results to merge after the main kernel (n_groups = 0: none).
struct AttnSplit {
  const int32_t* groups_dev = nullptr;  // 6 int32 per group
  int n_groups = 0;
  float* part_o = nullptr;              // [slots][128][64] fp32
  float* part_ml = nullptr;             // [slots][128][2]  (row max in log2 units, row sum)
};

rt_status launch_sparse_attention(void* ctx, const void* q, const void* k, const void* v, const AttnItem* items_dev,
                                  const int32_t* entries_dev, const int32_t* cta_ptr_dev, int n_ctas,
                                  int total_tokens, int heads, float scale, int dtype, cudaStream_t st,
                                  int* error_word_dev = nullptr, const AttnSplit& split = AttnSplit{});

}  // namespace rt
