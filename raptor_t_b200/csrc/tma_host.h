// Host-side creation of TMA tensor maps (cuTensorMapEncodeTiled obtained through
// the runtime's driver-entry-point query, so the library does not link libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.h"

namespace rt {

// 2D row-major tensor of 16-bit elements: `rows` x `cols`, row pitch `pitch_elems`.
// Box = box_cols x box_rows.  swizzle128: box_cols must be 64 (128 bytes).
rt_status make_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                             uint32_t box_rows, uint32_t box_cols, bool swizzle128);

}  // namespace rt
