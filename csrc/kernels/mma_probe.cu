// Roofline probe for the tensor pipe: clocks per tcgen05.mma (M = 128, K = 16, bf16, fp32 accumulate)
// as a function of N and of where the A operand comes from (shared memory or TMEM).  One thread per
// CTA issues a long chain of MMAs over zeroed shared memory (no TMA traffic, no epilogue) and times
// it with clock64; eight MMAs share an accumulator, then the accumulator alternates, as in a real
// k-loop.  The numbers decide tile shapes: on B200 an MMA costs about 68 clocks for every N <= 128 and
// 129 clocks at N = 256, so any tile narrower than 128 wastes the pipe in proportion.
// (Part of the measured-roofline tooling; the reference's probes are crates/gpu-core/src/roof.rs.)
#include "../common/host.hpp"
#include "../common/ptx.cuh"

namespace bb {

template <int N, bool TS, bool BMN>
__global__ void __launch_bounds__(128, 1) mma_probe_kernel(long long* out, int reps, int per) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc(1, 1, 1, 0, BMN ? 1 : 0, 128, N);
    const uint32_t sa = smem_u32(smem), sb = smem_u32(smem + 32 * 1024);
    uint32_t ph = 0;
    long long best = 1LL << 60;
    for (int r = 0; r < reps; ++r) {
      const long long t0 = clock64();
      for (int i = 0; i < per; ++i) {
        const int t = i & 3;            // k-step inside a 64-wide swizzled tile
        const int st = (i >> 2) & 1;    // two stages
        const uint64_t da = umma_smem_desc(sa + st * 16384 + t * 32, 16, 1024);
        const uint64_t db = BMN ? umma_smem_desc(sb + st * 32768 + t * 2048, 128 * 128, 1024)
                                : umma_smem_desc(sb + st * 32768 + t * 32, 16, 1024);
        const uint32_t d = tb + ((i >> 3) & 1) * (N <= 128 ? N : 0);   // switch accumulator every 8 MMAs
        if (TS) umma_f16_ts(d, tb + 448 + t * 8, db, idesc, (i & 7) != 0);
        else umma_f16_ss(d, da, db, idesc, (i & 7) != 0);
      }
      umma_commit(&bar);
      mbar_wait(&bar, ph);
      ph ^= 1;
      const long long dt = clock64() - t0;
      if (dt < best) best = dt;
    }
    out[blockIdx.x] = best;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tb, 512); }
}


}  // namespace bb

// out[grid] (device, int64): best-of-`reps` clocks for a chain of `per` MMAs in every CTA.
// n in {32, 64, 128, 256}; a_from_tmem / b_mn_major as flags.
BB_API int bb_mma_probe(int n, int a_from_tmem, int b_mn_major, int grid, int reps, int per, long long* out,
                        void* stream) {
  using namespace bb;
  if (grid < 1 || grid > 1024 || reps < 1 || per < 8 || per % 8) return BB_EARG;
  // an MN-major B tile of N columns spans N/64 chunks 16 KB apart: beyond N = 128 the second stage
  // would reach past the 96 KB this probe stages
  if (b_mn_major && n > 128) return BB_EARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int smem = 100 * 1024;
#define BB_PROBE(N_, TS_, MN_)                                                                         \
  do {                                                                                                 \
    static PerDeviceOnce once;                                                                         \
    cudaError_t e = ensure_dyn_smem(once, mma_probe_kernel<N_, TS_, MN_>, smem);                       \
    if (e != cudaSuccess) return (int)e;                                                               \
    mma_probe_kernel<N_, TS_, MN_><<<grid, 128, smem, s>>>(out, reps, per);                            \
    return (int)cudaGetLastError();                                                                    \
  } while (0)
#define BB_PROBE_N(N_)                                               \
  do {                                                               \
    if (a_from_tmem && b_mn_major) BB_PROBE(N_, true, true);         \
    if (a_from_tmem) BB_PROBE(N_, true, false);                      \
    if (b_mn_major) BB_PROBE(N_, false, true);                       \
    BB_PROBE(N_, false, false);                                      \
  } while (0)
  switch (n) {
    case 32: BB_PROBE_N(32);
    case 64: BB_PROBE_N(64);
    case 128: BB_PROBE_N(128);
    case 256: BB_PROBE_N(256);
    default: return BB_EARG;
  }
#undef BB_PROBE_N
#undef BB_PROBE
}
