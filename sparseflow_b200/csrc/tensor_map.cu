#include "tensor_map.h"

#include <cuda_runtime.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

namespace sfb200 {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// Encoded maps are cached: a step re-encodes the same dozen (pointer, shape, box) combinations on
// every launch, and the driver call costs about a microsecond each on the host launch path.
struct MapKey {
  uint64_t v[6];
  bool operator==(const MapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t x : k.v) {
      h ^= x;
      h *= 1099511628211ull;
    }
    return static_cast<size_t>(h);
  }
};
std::mutex g_cache_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_cache;

bool cached(const MapKey& key, CUtensorMap* out) {
  std::lock_guard<std::mutex> lk(g_cache_mu);
  auto it = g_cache.find(key);
  if (it == g_cache.end()) return false;
  *out = it->second;
  return true;
}
void remember(const MapKey& key, const CUtensorMap& m) {
  std::lock_guard<std::mutex> lk(g_cache_mu);
  if (g_cache.size() > 4096) g_cache.clear();
  g_cache.emplace(key, m);
}

}  // namespace

bool make_map_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                 uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle sw, int fmt) {
  int dev = 0;
  cudaGetDevice(&dev);
  const MapKey key = {{reinterpret_cast<uint64_t>(base), rows, cols, pitch_bytes,
                       (static_cast<uint64_t>(box_rows) << 32) | box_cols,
                       (static_cast<uint64_t>(dev) << 40) | (static_cast<uint64_t>(sw) << 8) | static_cast<uint64_t>(fmt)}};
  if (cached(key, m)) return true;
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  if (fn(m, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
         const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  remember(key, *m);
  return true;
}

bool make_map_1d_u64(CUtensorMap* m, const void* base, uint64_t elems, uint32_t box) {
  int dev = 0;
  cudaGetDevice(&dev);
  const MapKey key = {{reinterpret_cast<uint64_t>(base), elems, box, 0, 0, (static_cast<uint64_t>(dev) << 40) | 0xFFu}};
  if (cached(key, m)) return true;
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[1] = {elems};
  cuuint64_t gstr[1] = {0};
  cuuint32_t bx[1] = {box};
  cuuint32_t estr[1] = {1};
  if (fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 1, const_cast<void*>(base), gdim, gstr, bx, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  remember(key, *m);
  return true;
}

}  // namespace sfb200
