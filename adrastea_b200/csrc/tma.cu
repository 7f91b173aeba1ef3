// Host side of the TMA descriptors: resolves cuTensorMapEncodeTiled through the
// runtime and caches encoded maps per context.
#include <cstring>
#include <map>
#include <vector>

#include "tma.cuh"

namespace adr {

namespace {

struct MapKey {
  uint64_t v[16];
  bool operator<(const MapKey& o) const { return memcmp(v, o.v, sizeof(v)) < 0; }
};

struct TmaCache {
  std::map<MapKey, CUtensorMap> maps;
};

}  // namespace

int tma_init(adr_ctx* ctx) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  ctx->encode_tiled_fn = fn;
  ctx->tma_cache = new TmaCache();
  return ADR_OK;
}

void tma_destroy(adr_ctx* ctx) {
  delete static_cast<TmaCache*>(ctx->tma_cache);
  ctx->tma_cache = nullptr;
}

int tma_get(adr_ctx* ctx, CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
            const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
            CUtensorMapSwizzle swizzle) {
  if (!ctx->encode_tiled_fn || !ctx->tma_cache || rank < 2 || rank > 4) return ADR_ERR_INVALID;
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.v[0] = (uint64_t)(uintptr_t)base;
  key.v[1] = ((uint64_t)dtype << 32) | ((uint64_t)rank << 16) | (uint64_t)swizzle;
  for (int i = 0; i < rank; ++i) {
    key.v[2 + i] = dims[i];
    key.v[9 + i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) key.v[6 + i] = strides_bytes[i];
  TmaCache* cache = static_cast<TmaCache*>(ctx->tma_cache);
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = cache->maps.find(key);
    if (it != cache->maps.end()) {
      *out = it->second;
      return ADR_OK;
    }
  }
  cuuint64_t gdim[4] = {1, 1, 1, 1};
  cuuint64_t gstride[3] = {16, 16, 16};
  cuuint32_t bdim[4] = {1, 1, 1, 1};
  cuuint32_t estride[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) gstride[i] = strides_bytes[i];
  CUtensorMap m;
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled_fn)(
      &m, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bdim, estride,
      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    ctx->last_cuda_error = 10000 + (int)r;  // CUresult, offset to tell it from a cudaError_t
    return ADR_ERR_SHAPE;
  }
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (cache->maps.size() > 4096) cache->maps.clear();  // bound the cache
    cache->maps[key] = m;
  }
  *out = m;
  return ADR_OK;
}

}  // namespace adr
