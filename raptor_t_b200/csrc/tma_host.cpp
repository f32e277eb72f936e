#include "tma_host.h"

#include <mutex>

namespace rt {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_once;

void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<EncodeFn>(fn);
}
}  // namespace

rt_status make_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                             uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  std::call_once(g_once, load_encode);
  RT_REQUIRE(g_encode != nullptr, RT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  RT_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15u) == 0 && (pitch_elems * 2) % 16 == 0, RT_ERR_INVALID,
             "TMA tensor: base and row pitch must be 16-byte aligned");
  RT_REQUIRE(box_rows >= 1 && box_rows <= 256 && box_cols >= 8 && box_cols <= 256 && (box_cols * 2) % 16 == 0,
             RT_ERR_INVALID, "TMA box %ux%u out of range", box_rows, box_cols);
  RT_REQUIRE(!swizzle128 || box_cols == 64, RT_ERR_INVALID, "128-byte swizzle needs a 64-element box row");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RT_REQUIRE(r == CUDA_SUCCESS, RT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  return RT_OK;
}

}  // namespace rt
