#include "tmap.cuh"

#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>

namespace lb {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::mutex g_mu;
EncodeTiledFn g_encode = nullptr;
thread_local std::string g_err;

struct Key {
  uint64_t v[12];
  bool operator==(const Key& o) const { return std::memcmp(v, o.v, sizeof(v)) == 0; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t x : k.v) {
      h ^= x;
      h *= 1099511628211ull;
    }
    return size_t(h);
  }
};
// Descriptors are handed out by pointer, so entries are never moved once created.
std::unordered_map<Key, std::unique_ptr<CUtensorMap>, KeyHash> g_cache;

EncodeTiledFn get_encode() {
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    g_err = std::string("cuTensorMapEncodeTiled not available: ") + cudaGetErrorString(e);
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}

CUtensorMapDataType to_cu(int dtype, uint32_t* elem) {
  switch (dtype) {
    case TM_BF16: *elem = 2; return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case TM_U8: *elem = 1; return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    default: *elem = 4; return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  }
}

const CUtensorMap* encode(const Key& key, int rank, const void* base, const cuuint64_t* dims,
                          const cuuint64_t* strides, const cuuint32_t* box, int dtype, bool swizzle128) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_cache.find(key);
  if (it != g_cache.end()) return it->second.get();
  EncodeTiledFn enc = get_encode();
  if (!enc) return nullptr;
  if (g_cache.size() > 16384) g_cache.clear();
  uint32_t elem;
  CUtensorMapDataType dt = to_cu(dtype, &elem);
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  auto m = std::make_unique<CUtensorMap>();
  CUresult r = enc(m.get(), dt, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with %d (rank %d base %p dims %llu,%llu box %u,%u)",
             int(r), rank, base, (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
    g_err = buf;
    return nullptr;
  }
  const CUtensorMap* p = m.get();
  g_cache.emplace(key, std::move(m));
  return p;
}

}  // namespace

const char* tmap_last_error() { return g_err.c_str(); }

const CUtensorMap* tmap_2d(const void* base, uint64_t rows, uint64_t cols, uint64_t ld_bytes, uint32_t box_rows,
                           uint32_t box_cols, int dtype, bool swizzle128) {
  Key k{};
  k.v[0] = reinterpret_cast<uint64_t>(base);
  k.v[1] = rows; k.v[2] = cols; k.v[3] = ld_bytes; k.v[4] = box_rows; k.v[5] = box_cols;
  k.v[6] = uint64_t(dtype); k.v[7] = swizzle128; k.v[8] = 2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  return encode(k, 2, base, dims, strides, box, dtype, swizzle128);
}

const CUtensorMap* tmap_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes,
                           uint64_t s2_bytes, uint32_t b0, uint32_t b1, uint32_t b2, int dtype, bool swizzle128) {
  Key k{};
  k.v[0] = reinterpret_cast<uint64_t>(base);
  k.v[1] = d0; k.v[2] = d1; k.v[3] = d2; k.v[4] = s1_bytes; k.v[5] = s2_bytes;
  k.v[6] = b0; k.v[7] = b1; k.v[8] = b2; k.v[9] = uint64_t(dtype); k.v[10] = swizzle128; k.v[11] = 3;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  return encode(k, 3, base, dims, strides, box, dtype, swizzle128);
}

namespace {
bool g_pdl = true;
}
bool pdl_enabled() { return g_pdl; }
void set_pdl(bool on) { g_pdl = on; }

}  // namespace lb
