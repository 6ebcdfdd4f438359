// Host-side helpers shared by the C-ABI entry points: last-error string,
// driver entry point for TMA descriptor encoding, launch checks.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "prism_common.cuh"

namespace prism {

// One message per host thread; read back through prism_last_error_string().
inline char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is fetched through the runtime so that the library
// does not link against libcuda (it must load on a machine without a driver).
inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
    (void)cudaGetLastError();
  }
  return fn;
}

// Encoded tensor maps of the calling thread's recent calls.  A map depends only on the address, shape
// and box, so a repeated call (same buffers, same shapes: an inference loop, a training step) reuses
// it instead of going through the driver again -- that matters for the few-token forward, whose
// kernel runs for about 20 microseconds.
struct TmapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_rows, box_cols;
  int dt, swz;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols && dt == o.dt && swz == o.swz;
  }
};
struct TmapCache {
  static constexpr int kEntries = 32;
  TmapKey key[kEntries];
  CUtensorMap map[kEntries];
  bool used[kEntries] = {false};
  int next = 0;
};
inline TmapCache& tmap_cache() {
  static thread_local TmapCache c;
  return c;
}

// 2-D row-major tensor of 16-bit elements: `rows` x `cols`, leading dimension
// `ld` elements; box = box_rows x box_cols. box_cols*2 must be 128 bytes for the
// 128-byte swizzle. Out-of-range box parts read as zero / are not written.
inline int make_tmap_2d(CUtensorMap* out, int dt, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t ld, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  TmapCache& cache = tmap_cache();
  const TmapKey k{base, rows, cols, ld, box_rows, box_cols, dt, swizzle128 ? 1 : 0};
  for (int i = 0; i < TmapCache::kEntries; ++i)
    if (cache.used[i] && cache.key[i] == k) { *out = cache.map[i]; return PRISM_OK; }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(PRISM_ERR_NO_DRIVER, "cuTensorMapEncodeTiled is not available");
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType t =
      (dt == DT_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(out, t, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(PRISM_ERR_CUDA,
                "cuTensorMapEncodeTiled failed (%d) base=%p rows=%llu cols=%llu ld=%llu box=%ux%u",
                (int)r, base, (unsigned long long)rows, (unsigned long long)cols,
                (unsigned long long)ld, box_rows, box_cols);
  const int slot = cache.next;
  cache.next = (cache.next + 1) % TmapCache::kEntries;
  cache.key[slot] = k; cache.map[slot] = *out; cache.used[slot] = true;
  return PRISM_OK;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize, set once per (kernel, device, size) instead of on every launch.
inline int set_max_dynamic_smem(const void* kernel, int bytes, const char* what) {
  struct Entry { const void* fn; int dev, bytes; };
  static thread_local Entry seen[64];
  static thread_local int n_seen = 0;
  int dev = 0;
  (void)cudaGetDevice(&dev);
  for (int i = 0; i < n_seen; ++i)
    if (seen[i].fn == kernel && seen[i].dev == dev && seen[i].bytes >= bytes) return PRISM_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "%s: cannot set %d B of shared memory: %s", what, bytes, cudaGetErrorString(e));
  if (n_seen < 64) seen[n_seen++] = Entry{kernel, dev, bytes};
  return PRISM_OK;
}

// Number of kernels this library has launched in this process (for benchmarks and tests);
// any host thread may launch, so the counter is atomic.
inline std::atomic<long long>& launch_counter() {
  static std::atomic<long long> n{0};
  return n;
}

inline int check_launch(const char* what) {
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(PRISM_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return PRISM_OK;
}

}  // namespace prism
