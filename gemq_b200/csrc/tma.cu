// Cached cuTensorMapEncodeTiled for 2-D row-major tensors (driver entry point resolved at run
// time, so the library has no link-time dependency on libcuda).
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace gemq {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct MapKey {
  const void* base;
  long long rows;
  int inner, elem, box_inner, box_rows, swz, dev;
  bool operator<(const MapKey& o) const {
    return std::tie(base, rows, inner, elem, box_inner, box_rows, swz, dev) <
           std::tie(o.base, o.rows, o.inner, o.elem, o.box_inner, o.box_rows, o.swz, o.dev);
  }
};

// elem_bytes 4 -> UINT32, 2 -> UINT16 (any 16-bit type).  `inner` elements per row, row stride
// inner * elem_bytes (a multiple of 16).  128B swizzle needs box_inner * elem_bytes <= 128.
bool tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, int inner, long long rows, int box_inner,
                   int box_rows, bool swizzle128) {
  static std::mutex mu;
  static std::map<MapKey, CUtensorMap> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  const MapKey key{base, rows, inner, elem_bytes, box_inner, box_rows, swizzle128 ? 1 : 0, dev};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * elem_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1u, 1u};
  CUtensorMap m;
  const CUresult r = enc(&m, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache[key] = m;
  *out = m;
  return true;
}

}  // namespace gemq
