// Host-side construction of TMA tensor maps, shared by every kernel file that stages operands with
// cp.async.bulk.tensor (grouped GEMM bf16 / fp8, dense GEMM, attention).
//
// cuTensorMapEncodeTiled is reached through the runtime's driver entry point query, so the library links
// against cudart only.  Maps are cached per host thread by (base, element type, extents, stride, box): a
// training step re-issues the same GEMMs on the same buffers (weights, peer workspaces, flat gradient
// buffers), so after the first step nearly every launch finds its three maps in the cache instead of
// encoding them again.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

namespace slab {

typedef CUresult (*TmaEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline TmaEncodeTiledFn tma_encode_fn() {
  static TmaEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TmaEncodeTiledFn>(p);
  }
  return fn;
}

struct TmaMapKey {
  const void* base;
  uint64_t rows, cols, row_stride_bytes;
  uint32_t box_rows, box_cols;
  int dtype;
  int pad;
};

struct TmaMapSlot {
  TmaMapKey key;
  CUtensorMap map;
  bool used;
};

constexpr int TMA_CACHE_SLOTS = 1024;   // direct mapped; a colliding entry is simply re-encoded

inline uint64_t tma_key_hash(const TmaMapKey& k) {
  uint64_t h = 1469598103934665603ull;
  const uint64_t parts[6] = {reinterpret_cast<uint64_t>(k.base), k.rows, k.cols, k.row_stride_bytes,
                             (uint64_t(k.box_rows) << 32) | k.box_cols, uint64_t(k.dtype)};
  for (int i = 0; i < 6; ++i) {
    h ^= parts[i];
    h *= 1099511628211ull;
    h ^= h >> 29;
  }
  return h;
}

// Row-major 2-D tensor [rows, cols] of `esize`-byte elements whose rows are `row_stride_elems` elements
// apart; box = [box_rows, box_cols]; 128-byte swizzle; out-of-bounds elements read as zero and are not
// written.  Returns 0, -1 (driver entry point missing) or -2 - CUresult.
inline int tma_make_map_2d(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int esize, uint64_t rows,
                           uint64_t cols, uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols) {
  static thread_local TmaMapSlot* cache = nullptr;
  static thread_local bool ctx_ready = false;
  TmaMapKey key;
  memset(&key, 0, sizeof(key));
  key.base = base;
  key.rows = rows;
  key.cols = cols;
  key.row_stride_bytes = row_stride_elems * (uint64_t)esize;
  key.box_rows = box_rows;
  key.box_cols = box_cols;
  key.dtype = (int)dt;
  if (!cache) cache = new TmaMapSlot[TMA_CACHE_SLOTS]();
  TmaMapSlot& slot = cache[tma_key_hash(key) % TMA_CACHE_SLOTS];
  if (slot.used && memcmp(&slot.key, &key, sizeof(key)) == 0) {
    *m = slot.map;
    return 0;
  }
  TmaEncodeTiledFn enc = tma_encode_fn();
  if (!enc) return -1;
  // the driver entry point needs a current context; threads that have only been handed tensors (the
  // autograd engine's workers) may not have touched the runtime yet
  if (!ctx_ready) {
    cudaFree(0);
    ctx_ready = true;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {key.row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -2 - (int)r;
  slot.key = key;
  slot.map = *m;
  slot.used = true;
  return 0;
}

inline int tma_make_map_bf16(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                             uint32_t box_cols) {
  return tma_make_map_2d(m, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, cols, cols, box_rows, box_cols);
}

inline int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace slab
