// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver entry
// point (no link-time dependency on libcuda), the per-device error word and SM count cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#define BB_API extern "C" __attribute__((visibility("default")))

namespace bb {

// Return codes of the C ABI. 0 = ok; >0 = cudaError_t; <0 = argument / setup error.
enum : int { BB_OK = 0, BB_EARG = -1, BB_ETMAP = -2, BB_ESIZE = -3, BB_EDRIVER = -4 };

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn();

// 2-D row-major tensor [outer][inner] with `row_stride_bytes` pitch; box = [box_outer][box_inner],
// 128-byte swizzle (box_inner * elem_size must be 128 bytes), zero fill out of bounds.
int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_size, const void* base,
                 uint64_t inner, uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                 uint32_t box_outer, bool swizzle128 = true);

// 3-D tensor [d2][d1][d0] with byte strides s1 (d1) and s2 (d2); box = [1][box1][box0].
int make_tmap_3d(CUtensorMap* out, CUtensorMapDataType dt, int elem_size, const void* base,
                 uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes, uint64_t s2_bytes,
                 uint32_t box0, uint32_t box1, bool swizzle128 = true);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) belongs to the (function, device) pair, not to
// the process: a launcher keeps one of these per kernel instantiation and sets the attribute the
// first time it runs with each device current.
struct PerDeviceOnce {
  std::atomic<bool> done[64];
  PerDeviceOnce() { for (auto& d : done) d.store(false, std::memory_order_relaxed); }
  // true when the attribute still has to be set on the current device; `dev` receives its index
  bool need(int* dev) {
    *dev = 0;
    cudaGetDevice(dev);
    if (*dev < 0 || *dev >= 64) { *dev = -1; return true; }
    return !done[*dev].load(std::memory_order_acquire);
  }
  void mark(int dev) { if (dev >= 0) done[dev].store(true, std::memory_order_release); }
};

template <typename K>
inline cudaError_t ensure_dyn_smem(PerDeviceOnce& once, K kernel, int bytes) {
  int dev;
  if (!once.need(&dev)) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) once.mark(dev);
  return e;
}

int* device_error_word();  // per-device int, zero-initialised, lives until exit
int sm_count();

}  // namespace bb
