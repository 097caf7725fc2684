#include "tensormap.h"

#include <cstring>
#include <mutex>
#include <unordered_map>
#include <string>

namespace fmb {

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn resolve_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(p);
    }
  });
  return fn;
}

struct Key {
  const void* base;
  uint64_t d[5];
  uint64_t s[5];
  uint32_t b[5];
  int rank, eb, swz;
  bool operator==(const Key& o) const { return std::memcmp(this, &o, sizeof(Key)) == 0; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(Key) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return h;
  }
};

std::mutex g_mu;
std::unordered_map<Key, CUtensorMap, KeyHash> g_cache;

CUtensorMapDataType dtype_of(int elem_bytes) {
  switch (elem_bytes) {
    case 1: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    case 2: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case 4: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

CUtensorMapSwizzle swz_of(TmapSwizzle s) {
  switch (s) {
    case TmapSwizzle::B32: return CU_TENSOR_MAP_SWIZZLE_32B;
    case TmapSwizzle::B64: return CU_TENSOR_MAP_SWIZZLE_64B;
    case TmapSwizzle::B128: return CU_TENSOR_MAP_SWIZZLE_128B;
    default: return CU_TENSOR_MAP_SWIZZLE_NONE;
  }
}

}  // namespace

bool make_tmap_nd(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                  const uint64_t* strides_bytes, const uint32_t* box, int elem_bytes, TmapSwizzle swz) {
  if (rank < 1 || rank > 5) return false;
  Key key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  key.rank = rank;
  key.eb = elem_bytes;
  key.swz = static_cast<int>(swz);
  for (int i = 0; i < rank; ++i) {
    key.d[i] = dims[i];
    key.s[i] = i == 0 ? static_cast<uint64_t>(elem_bytes) : strides_bytes[i];
    key.b[i] = box[i];
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_cache.find(key);
    if (it != g_cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeFn enc = resolve_encode();
  if (enc == nullptr) return false;
  {
    // Driver calls need the primary context bound to the calling thread; worker threads (the
    // autograd engine's, for one) may not have touched the runtime yet.
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return false;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i];
  }
  CUtensorMap m;
  CUresult r = enc(&m, dtype_of(elem_bytes), static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr,
                   bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz_of(swz), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_cache.size() > 8192) g_cache.clear();
    g_cache.emplace(key, m);
  }
  *out = m;
  return true;
}

bool make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t box_rows, uint32_t box_cols, int elem_bytes, TmapSwizzle swz) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[2] = {static_cast<uint64_t>(elem_bytes), ld * static_cast<uint64_t>(elem_bytes)};
  uint32_t box[2] = {box_cols, box_rows};
  return make_tmap_nd(out, base, 2, dims, strides, box, elem_bytes, swz);
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

}  // namespace fmb
