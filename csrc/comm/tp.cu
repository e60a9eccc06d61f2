// Small kernels around the fused tensor-parallel GEMMs:
//   tp_sum_slots   y = sum_r recv[r] (+ residual): the reduction half of GEMM -> reduce-scatter, run
//                  by the owner of the rows over the `world` partial slots its peers filled
//   tp_allreduce   one-shot all-reduce for small serving activations: every rank publishes its
//                  [rows, d] partial in symmetric memory, signals, waits (bounded) for its peers and
//                  sums all partials in a fixed rank order (bit-identical on every rank)
// Peer access is plain ld/st with system-scope release/acquire flags.
#include "../common/host.hpp"
#include "../common/peer.cuh"
#include "../common/ptx.cuh"
#include "../common/vec.cuh"

namespace bb {

__global__ void tp_sum_slots_kernel(const __nv_bfloat16* __restrict__ recv, int world,
                                    long slot_elems, const __nv_bfloat16* __restrict__ residual,
                                    __nv_bfloat16* __restrict__ y) {
  const long nv = slot_elems >> 3;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) {
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(recv + (size_t)r * slot_elems)[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    if (residual) {
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(residual)[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    reinterpret_cast<bf16x8*>(y)[i] = pack8(acc);
  }
}

struct ArArgs {
  PeerPtrs bufs;  // every rank's symmetric [n] bf16 staging buffer
  PeerPtrs sig;   // every rank's uint64[world] flags
  const __nv_bfloat16* x;
  __nv_bfloat16* y;
  long n;
  int rank, world;
  uint32_t epoch;
  long long wait_limit;
  int* err;
  unsigned int* counter;
};

// Phase 1 (all blocks): copy x into my staging buffer.  The last block to finish publishes the
// flag to all peers.  Phase 2: every block waits for all peers' flags, then sums.
__global__ void __launch_bounds__(256) tp_allreduce_kernel(const ArArgs a) {
  __shared__ int s_ok;
  const long nv = a.n >> 3;
  bf16x8* mine = reinterpret_cast<bf16x8*>(a.bufs.p[a.rank]);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long)gridDim.x * blockDim.x)
    mine[i] = reinterpret_cast<const bf16x8*>(a.x)[i];
  // one system-scope fence per block, after the block barrier (it is cumulative over the writes the
  // barrier ordered before it); a fence in every thread made thousands of MEMBAR.SYS queue up
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_ok = 1;
    const unsigned int done = atomicAdd(a.counter, 1u);
    if (done == gridDim.x - 1) {
      *a.counter = 0u;
      for (int r = 0; r < a.world; ++r)
        st_release_sys_u64(reinterpret_cast<uint64_t*>(a.sig.p[r]) + a.rank, (uint64_t)a.epoch);
    }
  }
  __syncthreads();
  if (threadIdx.x < a.world) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(a.sig.p[a.rank]) + threadIdx.x;
    if (!wait_epoch(f, a.epoch, 0, a.wait_limit)) {
      set_error(a.err, ERR_WAIT_PEER);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (!s_ok) return;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < a.world; ++r) {
      const uint4 raw = ld_volatile_u4(reinterpret_cast<const uint4*>(a.bufs.p[r]) + i);
      float f[8];
      unpack8(*reinterpret_cast<const bf16x8*>(&raw), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    reinterpret_cast<bf16x8*>(a.y)[i] = pack8(acc);
  }
}

// Two-shot all-reduce whose epoch lives in device memory, so the launch parameters never change
// and the call can sit inside a captured CUDA graph (decode steps replay one graph).
//   phase 1  copy x into my staging buffer; the last block publishes flag 2e-1 to every peer
//   phase 2  wait for every peer's 2e-1; reduce MY 1/world slice over all staging buffers in rank
//            order (bit-identical everywhere) and store it into every rank's result buffer; the
//            last block publishes flag 2e
//   phase 3  wait for every peer's 2e: my result buffer is complete, and every peer has finished
//            reading my staging buffer, so ONE staging buffer is enough for back-to-back calls.
// A peer writes into my result buffer only after it saw my flag 2(e+1)-1, which my next call
// publishes after everything I launched before it on the stream has consumed the result.
// Each value crosses NVLink (world-1)/world times in each direction instead of world-1 times.
struct Ar2Args {
  PeerPtrs stage, result, sig;
  const __nv_bfloat16* x;
  long n;
  int rank, world;
  unsigned int* epoch_dev;   // [0] epoch of the last finished call
  unsigned int* counters;    // [0..2] zeroed block counters
  long long wait_limit;
  int* err;
};

// W > 0: the world size as a compile-time constant, with 8 / W slices of the loop in flight per
// thread (at W = 2 a thread otherwise has only two 16-byte peer loads outstanding per NVLink round
// trip and the reduce phase is latency-bound); W = 0: any world size up to MAX_RANKS.
template <int W>
__global__ void __launch_bounds__(256) tp_allreduce2_kernel(const Ar2Args a) {
  __shared__ unsigned int s_e;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_e = *reinterpret_cast<volatile unsigned int*>(a.epoch_dev) + 1u;
    s_ok = 1;
  }
  __syncthreads();
  const unsigned int e = s_e;
  const long nv = a.n >> 3;
  const long stride = (long)gridDim.x * blockDim.x;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  bf16x8* mine = reinterpret_cast<bf16x8*>(a.stage.p[a.rank]);
  for (long i = tid; i < nv; i += stride) mine[i] = reinterpret_cast<const bf16x8*>(a.x)[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();   // one per block: cumulative over the block's writes ordered by the barrier
    if (atomicAdd(a.counters, 1u) == gridDim.x - 1) {
      a.counters[0] = 0u;
      for (int r = 0; r < a.world; ++r)
        st_release_sys_u64(reinterpret_cast<uint64_t*>(a.sig.p[r]) + a.rank, (uint64_t)(2u * e - 1u));
    }
  }
  if (threadIdx.x < a.world) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(a.sig.p[a.rank]) + threadIdx.x;
    if (!wait_epoch(f, 2u * e - 1u, 0, a.wait_limit)) {
      set_error(a.err, ERR_WAIT_PEER);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (s_ok) {
    const long per = nv / a.world;  // host guarantees divisibility
    const long lo = (long)a.rank * per;
    if constexpr (W > 0) {
      constexpr int U = 8 / W > 0 ? 8 / W : 1;   // loop slices in flight per thread
      for (long j0 = tid; j0 < per; j0 += stride * U) {
        uint4 raw[U][W];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long j = j0 + (long)u * stride;
          if (j < per) {
#pragma unroll
            for (int r = 0; r < W; ++r)
              raw[u][r] = ld_volatile_u4(reinterpret_cast<const uint4*>(a.stage.p[r]) + lo + j);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long j = j0 + (long)u * stride;
          if (j < per) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int r = 0; r < W; ++r) {   // rank order: the sum is bit-identical on every rank
              float f[8];
              unpack8(*reinterpret_cast<const bf16x8*>(&raw[u][r]), f);
#pragma unroll
              for (int q = 0; q < 8; ++q) acc[q] += f[q];
            }
            const bf16x8 out = pack8(acc);
#pragma unroll
            for (int r = 0; r < W; ++r) reinterpret_cast<bf16x8*>(a.result.p[r])[lo + j] = out;
          }
        }
      }
    } else {
      for (long j = tid; j < per; j += stride) {
        const long i = lo + j;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        uint4 raw[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)   // all peer loads in flight before the first add
          if (r < a.world) raw[r] = ld_volatile_u4(reinterpret_cast<const uint4*>(a.stage.p[r]) + i);
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r) {
          if (r < a.world) {
            float f[8];
            unpack8(*reinterpret_cast<const bf16x8*>(&raw[r]), f);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[q] += f[q];
          }
        }
        const bf16x8 out = pack8(acc);
        for (int r = 0; r < a.world; ++r) reinterpret_cast<bf16x8*>(a.result.p[r])[i] = out;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.counters + 1, 1u) == gridDim.x - 1) {
      a.counters[1] = 0u;
      for (int r = 0; r < a.world; ++r)
        st_release_sys_u64(reinterpret_cast<uint64_t*>(a.sig.p[r]) + a.rank, (uint64_t)(2u * e));
    }
  }
  if (threadIdx.x < a.world && s_ok) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(a.sig.p[a.rank]) + threadIdx.x;
    if (!wait_epoch(f, 2u * e, 0, a.wait_limit)) set_error(a.err, ERR_WAIT_PEER);
  }
  __syncthreads();
  // the epoch advances even after a timeout, so the ranks stay in step for the next call
  if (threadIdx.x == 0) {
    if (atomicAdd(a.counters + 2, 1u) == gridDim.x - 1) {
      a.counters[2] = 0u;
      *reinterpret_cast<volatile unsigned int*>(a.epoch_dev) = e;
      __threadfence();
    }
  }
}

// In-switch variant of the two-shot all-reduce (NVLS): the staging and result buffers are bound to
// NVLink multicast addresses, so phase 2 is ONE multimem.ld_reduce per 16 bytes (the switch adds the
// world's copies in fp32 and returns the sum) and ONE multimem.st (the switch writes the result into
// every rank's buffer).  Each value crosses this GPU's links once in each direction whatever the
// world size, and every rank receives bit-identical sums.  Flags and epoch handling are those of
// tp_allreduce2_kernel; the flag exchange itself stays on plain peer stores.
struct ArMmArgs {
  PeerPtrs sig;
  __nv_bfloat16* stage_local;   // this rank's staging buffer (unicast address)
  const void* stage_mc;         // multicast address of the staging buffers
  void* result_mc;              // multicast address of the result buffers
  const __nv_bfloat16* x;
  long n;
  int rank, world;
  unsigned int* epoch_dev;
  unsigned int* counters;
  long long wait_limit;
  int* err;
};

__global__ void __launch_bounds__(256) tp_allreduce_mm_kernel(const ArMmArgs a) {
  __shared__ unsigned int s_e;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_e = *reinterpret_cast<volatile unsigned int*>(a.epoch_dev) + 1u;
    s_ok = 1;
  }
  __syncthreads();
  const unsigned int e = s_e;
  const long nv = a.n >> 3;
  const long stride = (long)gridDim.x * blockDim.x;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  bf16x8* mine = reinterpret_cast<bf16x8*>(a.stage_local);
  for (long i = tid; i < nv; i += stride) mine[i] = reinterpret_cast<const bf16x8*>(a.x)[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.counters, 1u) == gridDim.x - 1) {
      a.counters[0] = 0u;
      for (int r = 0; r < a.world; ++r)
        st_release_sys_u64(reinterpret_cast<uint64_t*>(a.sig.p[r]) + a.rank, (uint64_t)(2u * e - 1u));
    }
  }
  if (threadIdx.x < a.world) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(a.sig.p[a.rank]) + threadIdx.x;
    if (!wait_epoch(f, 2u * e - 1u, 0, a.wait_limit)) {
      set_error(a.err, ERR_WAIT_PEER);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (s_ok) {
    const long per = nv / a.world;  // host guarantees divisibility
    const long lo = (long)a.rank * per;
    const uint4* src = reinterpret_cast<const uint4*>(a.stage_mc) + lo;
    uint4* dst = reinterpret_cast<uint4*>(a.result_mc) + lo;
    for (long j = tid; j < per; j += stride) {
      uint32_t r0, r1, r2, r3;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                   : "l"(src + j)
                   : "memory");
      asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "r"(r0),
                   "r"(r1), "r"(r2), "r"(r3)
                   : "memory");
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.counters + 1, 1u) == gridDim.x - 1) {
      a.counters[1] = 0u;
      for (int r = 0; r < a.world; ++r)
        st_release_sys_u64(reinterpret_cast<uint64_t*>(a.sig.p[r]) + a.rank, (uint64_t)(2u * e));
    }
  }
  if (threadIdx.x < a.world && s_ok) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(a.sig.p[a.rank]) + threadIdx.x;
    if (!wait_epoch(f, 2u * e, 0, a.wait_limit)) set_error(a.err, ERR_WAIT_PEER);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(a.counters + 2, 1u) == gridDim.x - 1) {
      a.counters[2] = 0u;
      *reinterpret_cast<volatile unsigned int*>(a.epoch_dev) = e;
      __threadfence();
    }
  }
}

// All ranks meet: publish `epoch` to every peer, then wait (bounded) until every peer published it.
// Orders "my earlier kernels' writes to symmetric memory" before "peers' later reads" without NCCL.
__global__ void symm_barrier_kernel(PeerPtrs sig, int rank, int world, uint32_t epoch,
                                    long long wait_limit, int* err) {
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys_u64(reinterpret_cast<uint64_t*>(sig.p[threadIdx.x]) + rank, (uint64_t)epoch);
    if (!wait_epoch(reinterpret_cast<const uint64_t*>(sig.p[rank]) + threadIdx.x, epoch, 0, wait_limit))
      set_error(err, ERR_WAIT_PEER);
  }
}

}  // namespace bb

using namespace bb;

// sig_ptrs[r]: rank r's uint64[world] flag words (zeroed once); epoch must increase on every call.
BB_API int bb_symm_barrier(const uint64_t* sig_ptrs, int rank, int world, unsigned int epoch,
                           double wait_seconds, void* stream) {
  if (world < 1 || world > MAX_RANKS) return BB_EARG;
  PeerPtrs s{};
  for (int r = 0; r < world; ++r) s.p[r] = reinterpret_cast<void*>(sig_ptrs[r]);
  symm_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(s, rank, world, epoch,
                                                          (long long)(wait_seconds * 1.9e9),
                                                          device_error_word());
  return (int)cudaGetLastError();
}

// y[slot_elems] = sum over `world` consecutive slots of recv (+ residual)
BB_API int bb_tp_sum_slots(const void* recv, int world, long slot_elems, const void* residual,
                           void* y, void* stream) {
  if (slot_elems % 8) return BB_EARG;
  long blocks = ((slot_elems >> 3) + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  tp_sum_slots_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)recv, world, slot_elems, (const __nv_bfloat16*)residual,
      (__nv_bfloat16*)y);
  return (int)cudaGetLastError();
}

// One-shot all-reduce of n bf16 values (n % 8 == 0).  buf_ptrs[r]: rank r's symmetric staging
// buffer (>= n elements; two alternating buffers must be used for back-to-back calls so a fast
// rank cannot overwrite data a slow peer is still reading); sig_ptrs[r]: uint64[world] flags;
// counter: zeroed uint32 in local memory.  The grid is at most one wave.
BB_API int bb_tp_allreduce(const uint64_t* buf_ptrs, const uint64_t* sig_ptrs, const void* x,
                           void* y, long n, int rank, int world, unsigned int epoch,
                           unsigned int* counter, double wait_seconds, void* stream) {
  if (world < 1 || world > MAX_RANKS || n % 8) return BB_EARG;
  ArArgs a{};
  for (int r = 0; r < world; ++r) {
    a.bufs.p[r] = reinterpret_cast<void*>(buf_ptrs[r]);
    a.sig.p[r] = reinterpret_cast<void*>(sig_ptrs[r]);
  }
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.n = n;
  a.rank = rank;
  a.world = world;
  a.epoch = epoch;
  a.wait_limit = (long long)(wait_seconds * 1.9e9);
  a.err = device_error_word();
  a.counter = counter;
  long blocks = ((n >> 3) + 255) / 256;
  if (blocks > sm_count()) blocks = sm_count();  // every block waits on peers: keep them co-resident
  if (blocks < 1) blocks = 1;
  tp_allreduce_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// Graph-safe two-shot all-reduce of n bf16 values (n % (8*world) == 0) into this rank's symmetric
// result buffer.  stage/result/sig_ptrs[r]: rank r's buffers (>= n elements; uint64[world] flags
// used by no other protocol); epoch_dev: one zeroed uint32; counters: three zeroed uint32.
BB_API int bb_tp_allreduce2(const uint64_t* stage_ptrs, const uint64_t* result_ptrs,
                            const uint64_t* sig_ptrs, const void* x, long n, int rank, int world,
                            unsigned int* epoch_dev, unsigned int* counters, double wait_seconds,
                            void* stream) {
  using namespace bb;
  if (world < 1 || world > MAX_RANKS || n <= 0 || n % (8L * world)) return BB_EARG;
  Ar2Args a{};
  for (int r = 0; r < world; ++r) {
    a.stage.p[r] = reinterpret_cast<void*>(stage_ptrs[r]);
    a.result.p[r] = reinterpret_cast<void*>(result_ptrs[r]);
    a.sig.p[r] = reinterpret_cast<void*>(sig_ptrs[r]);
  }
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.n = n;
  a.rank = rank;
  a.world = world;
  a.epoch_dev = epoch_dev;
  a.counters = counters;
  a.wait_limit = (long long)(wait_seconds * 1.9e9);
  a.err = device_error_word();
  long blocks = ((n >> 3) + 255) / 256;
  if (blocks > sm_count()) blocks = sm_count();  // every block waits on peers: keep them co-resident
  if (blocks < 1) blocks = 1;
  cudaStream_t s = (cudaStream_t)stream;
  switch (world) {
    case 2: tp_allreduce2_kernel<2><<<(int)blocks, 256, 0, s>>>(a); break;
    case 4: tp_allreduce2_kernel<4><<<(int)blocks, 256, 0, s>>>(a); break;
    case 8: tp_allreduce2_kernel<8><<<(int)blocks, 256, 0, s>>>(a); break;
    default: tp_allreduce2_kernel<0><<<(int)blocks, 256, 0, s>>>(a); break;
  }
  return (int)cudaGetLastError();
}

// NVLS form of bb_tp_allreduce2: `stage_local` is this rank's staging buffer, `stage_mc` /
// `result_mc` the multicast addresses of the symmetric staging and result buffers (the arena must be
// bound to an NVLink multicast object).  Same state words and epoch rules as bb_tp_allreduce2; the
// two must not share signal words.
BB_API int bb_tp_allreduce_mm(void* stage_local, const void* stage_mc, void* result_mc,
                              const uint64_t* sig_ptrs, const void* x, long n, int rank, int world,
                              unsigned int* epoch_dev, unsigned int* counters, double wait_seconds,
                              void* stream) {
  using namespace bb;
  if (world < 2 || world > MAX_RANKS || n <= 0 || n % (8L * world)) return BB_EARG;
  if (!stage_mc || !result_mc) return BB_EARG;
  ArMmArgs a{};
  for (int r = 0; r < world; ++r) a.sig.p[r] = reinterpret_cast<void*>(sig_ptrs[r]);
  a.stage_local = static_cast<__nv_bfloat16*>(stage_local);
  a.stage_mc = stage_mc;
  a.result_mc = result_mc;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.n = n;
  a.rank = rank;
  a.world = world;
  a.epoch_dev = epoch_dev;
  a.counters = counters;
  a.wait_limit = (long long)(wait_seconds * 1.9e9);
  a.err = device_error_word();
  long blocks = ((n >> 3) + 255) / 256;
  if (blocks > sm_count()) blocks = sm_count();  // every block waits on peers: keep them co-resident
  if (blocks < 1) blocks = 1;
  tp_allreduce_mm_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}
