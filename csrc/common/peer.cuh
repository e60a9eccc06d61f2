// Peer-memory helpers shared by the fused compute+collective kernels: tables of per-rank base
// pointers, system-scope acquire/release accessors and the bounded epoch wait.
#pragma once
#include <stdint.h>

namespace bb {

static constexpr int MAX_RANKS = 16;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_s32(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_volatile_f4(const float4* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Wait until (*p >> shift) >= want.  Returns false when `limit` clock cycles pass first.
__device__ __forceinline__ bool wait_epoch(const uint64_t* p, uint32_t want, int shift,
                                           long long limit) {
  const long long t0 = clock64();
  while ((uint32_t)(ld_acquire_sys_u64(p) >> shift) < want) {
    if (clock64() - t0 > limit) return false;
    __nanosleep(64);
  }
  return true;
}
__device__ __forceinline__ bool wait_flag_ge(const int* p, int want, long long limit) {
  const long long t0 = clock64();
  while (ld_acquire_gpu_s32(p) < want) {
    if (clock64() - t0 > limit) return false;
    __nanosleep(32);
  }
  return true;
}

}  // namespace bb
