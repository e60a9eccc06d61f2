// Allocation-free variant of the gradient sum-of-squares reduction: same two-stage, fixed-order
// algorithm as bb_sumsq (adamw.cu), but the per-block partial sums go to an array that is linked
// into the library instead of a caller-supplied scratch buffer.  See sumsq_noalloc.h for the
// contract (who cannot allocate, the size limit, sharing and ordering rules).
#include "sumsq_noalloc.h"

#include <atomic>
#include <cstdio>

#include "../common/host.hpp"
#include "../common/ptx.cuh"

namespace {

// Lives in every GPU's copy of the library image until the process exits (4 KiB).
static __device__ __align__(256) float g_noalloc_partials[BB_SUMSQ_NOALLOC_SCRATCH_FLOATS];

__global__ void noalloc_partial_kernel(const float* __restrict__ g, long n, float* __restrict__ part) {
  __shared__ float sh[32];
  float acc = 0.f;
  const long n4 = n >> 2;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long)gridDim.x * blockDim.x) {
    const float4 x = reinterpret_cast<const float4*>(g)[i];
    acc += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
  }
  if (blockIdx.x == 0) {
    const long t = (n4 << 2) + threadIdx.x;
    if (t < n) acc += g[t] * g[t];
  }
  acc = bb::warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    s = bb::warp_sum(s);
    if (threadIdx.x == 0) part[blockIdx.x] = s;  // every slot the final pass reads is rewritten
  }
}

__global__ void noalloc_final_kernel(const float* __restrict__ part, int np, float* __restrict__ out,
                                     int accumulate) {
  __shared__ float sh[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < np; i += blockDim.x) acc += part[i];
  acc = bb::warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    s = bb::warp_sum(s);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
  }
}

// Device address of the scratch array, looked up once per device with that device current.
// In host code `g_noalloc_partials` is only a stand-in symbol, never a usable pointer.
float* scratch_for_current_device(int* status) {
  // Host threads may make their first call on a device at the same time: the cache entries are
  // atomics (both threads would store the same address, so relaxed ordering is enough).
  static std::atomic<float*> ptrs[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *status = BB_SUMSQ_NOALLOC_ESETUP;
    return nullptr;
  }
  float* cached = ptrs[dev].load(std::memory_order_relaxed);
  if (!cached) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials);
    if (e != cudaSuccess || p == nullptr) {
      std::fprintf(stderr, "bb_sumsq_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
                   cudaGetErrorString(e));
      *status = BB_SUMSQ_NOALLOC_ESETUP;
      return nullptr;
    }
    ptrs[dev].store(p, std::memory_order_relaxed);
    cached = p;
  }
  *status = 0;
  return cached;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int bb_sumsq_noalloc(const float* g, long n,
                                                                        float* out, int accumulate,
                                                                        void* stream) {
  if (n < 0 || n > BB_SUMSQ_NOALLOC_MAX_ELEMS) {
    std::fprintf(stderr,
                 "bb_sumsq_noalloc: n = %ld is outside [0, %ld]; this entry point has a fixed "
                 "built-in scratch and does not take larger inputs (use bb_sumsq with your own "
                 "scratch buffer instead)\n",
                 n, (long)BB_SUMSQ_NOALLOC_MAX_ELEMS);
    return BB_SUMSQ_NOALLOC_ESIZE;
  }
  if (out == nullptr || (n > 0 && g == nullptr) || (reinterpret_cast<uintptr_t>(g) & 15))
    return BB_SUMSQ_NOALLOC_EARG;
  int status = 0;
  float* scratch = scratch_for_current_device(&status);  // first call per device does the set-up
  if (!scratch) return status;
  long blocks = ((n >> 2) + 511) / 512;
  if (blocks > BB_SUMSQ_NOALLOC_SCRATCH_FLOATS) blocks = BB_SUMSQ_NOALLOC_SCRATCH_FLOATS;
  if (blocks < 1) blocks = 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  noalloc_partial_kernel<<<(int)blocks, 512, 0, s>>>(g, n, scratch);
  const cudaError_t first = cudaGetLastError();
  if (first != cudaSuccess) return (int)first;  // never sum stale partials into `out`
  noalloc_final_kernel<<<1, 256, 0, s>>>(scratch, (int)blocks, out, accumulate);
  return (int)cudaGetLastError();
}
