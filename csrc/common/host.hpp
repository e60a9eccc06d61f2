// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver entry
// point (no link-time dependency on libcuda), the per-device error word and SM count cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

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

int* device_error_word();  // per-device int, zero-initialised, lives until exit
int sm_count();

}  // namespace bb
