#include "tma_host.h"

#include <cstring>
#include <mutex>
#include <unordered_map>

namespace rt {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_once;

// Encoded maps are pure functions of (address, shape, box, swizzle): the encoder's scratch and
// weight buffers keep their addresses from batch to batch, so a forward pass of ~90 launches
// finds all of its ~130 maps here instead of calling the driver for each.
struct MapKey {
  uintptr_t base;
  uint64_t rows, cols, pitch;
  uint32_t box_rows, box_cols, swizzle;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows &&
           box_cols == o.box_cols && swizzle == o.swizzle;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = k.base * 0x9e3779b97f4a7c15ull;
    h ^= (k.rows + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2));
    h ^= (k.cols * 31 + k.pitch * 131 + k.box_rows * 7 + k.box_cols * 3 + k.swizzle + (h << 6) + (h >> 2));
    return static_cast<size_t>(h);
  }
};
std::mutex g_cache_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_cache;
constexpr size_t kMaxCachedMaps = 4096;

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
  const MapKey key{reinterpret_cast<uintptr_t>(base), rows, cols, pitch_elems, box_rows, box_cols, swizzle128 ? 1u : 0u};
  {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    auto it = g_cache.find(key);
    if (it != g_cache.end()) {
      std::memcpy(map, &it->second, sizeof(CUtensorMap));
      return RT_OK;
    }
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RT_REQUIRE(r == CUDA_SUCCESS, RT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    if (g_cache.size() >= kMaxCachedMaps) g_cache.clear();
    g_cache.emplace(key, *map);
  }
  return RT_OK;
}

}  // namespace rt
