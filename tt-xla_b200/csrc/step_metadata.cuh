// One-launch build of a step's attention metadata from device-resident scheduler state:
// cache_position, page_table (unused and parked rows zeroed), fill_page_table (rolled left by
// the computed blocks, narrowed) and slot_mapping.  One CTA per row.
#pragma once
#include "ptx.cuh"

namespace b200attn {

struct StepMetadataParams {
  const int32_t* num_computed;    // [n]
  const int32_t* num_scheduled;   // [n]
  const int32_t* block_table;     // [>= n, width]
  int64_t block_table_stride;
  int n, rows, width, fill_width, tokens_per_row, block_size;
  int32_t* cache_position;        // [rows]
  int32_t* page_table;            // [rows, width]
  int32_t* fill_page_table;       // [rows, fill_width]
  int64_t* slot_mapping;          // [rows, tokens_per_row]
};

__global__ void __launch_bounds__(128) build_step_metadata_kernel(const StepMetadataParams p) {
  const int r = blockIdx.x;
  const bool live = r < p.n;
  const int computed = live ? p.num_computed[r] : 0;
  const int scheduled = live ? p.num_scheduled[r] : 0;
  const bool parked = !live || scheduled == 0;      // parked rows point at the null block
  if (threadIdx.x == 0) p.cache_position[r] = live ? computed + scheduled - 1 : -1;
  const int32_t* src = p.block_table + static_cast<int64_t>(r) * p.block_table_stride;
  const int shift = computed / p.block_size;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    const int32_t v = parked ? 0 : src[c];
    p.page_table[static_cast<int64_t>(r) * p.width + c] = v;
  }
  for (int c = threadIdx.x; c < p.fill_width; c += blockDim.x) {
    int32_t v = 0;
    if (!parked) v = src[(c + shift) % p.width];    // roll left by `shift`
    p.fill_page_table[static_cast<int64_t>(r) * p.fill_width + c] = v;
  }
  for (int t = threadIdx.x; t < p.tokens_per_row; t += blockDim.x) {
    int64_t slot = -1;
    if (!parked && t < scheduled) {
      const int pos = computed + t;
      const int col = pos / p.block_size;
      if (col < p.width) slot = static_cast<int64_t>(src[col]) * p.block_size + pos % p.block_size;
    }
    p.slot_mapping[static_cast<int64_t>(r) * p.tokens_per_row + t] = slot;
  }
}

}  // namespace b200attn
