// Fused data-parallel optimiser step over NVLink peer memory (no NCCL call):
//
//   kernel 1  dp_reduce_kernel   every rank announces "my gradient bucket is complete", waits
//                                (bounded) for all peers, then reduces ITS shard of the fp32
//                                gradient bucket by plain peer loads in a fixed rank order
//                                (bit-reproducible), writes the reduced shard locally, and sends
//                                the shard's sum of squares to every peer.
//   kernel 2  dp_adamw_ag_kernel waits (bounded) for all peers' partial norms, forms the global
//                                clip coefficient, applies AdamW to the shard (fp32 master/m/v) and
//                                stores the new bf16 weights straight into EVERY rank's weight
//                                buffer (the all-gather is the kernel's own peer stores); the last
//                                block exchanges "weights landed" flags so the next forward is safe.
//
// Flags are monotonically increasing step numbers (never reset); every spin has a clock limit and
// on expiry records ERR_WAIT_PEER and returns, so a missing peer never hangs the GPU.
// Peer access is plain ld/st (no multimem), which keeps a dying rank from faulting the others.
//
// Replaces the reference's host-staged DP step (crates/model/src/parallel.rs:152-240) and the
// per-tensor AdamW dispatches of crates/optim/src/lib.rs:170-217.
#include "../common/host.hpp"
#include "../common/peer.cuh"
#include "../common/ptx.cuh"

namespace bb {

// Signal area layout inside each rank's symmetric buffer (uint64 slots):
//   [0, R)      ready[r]  : rank r's gradient bucket for step `e` is complete   (value = e)
//   [R, 2R)     norm[r]   : (e << 32) | float bits of rank r's shard sum of squares
//   [2R, 3R)    landed[r] : rank r has stored its weight shard for step e everywhere (value = e)
struct DpReduceArgs {
  PeerPtrs grads;   // fp32 gradient bucket base of every rank
  PeerPtrs sig;     // signal area base of every rank
  float* shard_out; // [n] local, reduced shard
  float* partials;  // [gridDim.x] local scratch
  unsigned int* counter;  // local, zero before launch; reset by the kernel
  long lo, n;       // shard range (elements, multiples of 4)
  int rank, world;
  uint32_t epoch;
  long long wait_limit;
  int* err;
};

__global__ void __launch_bounds__(256) dp_reduce_kernel(const DpReduceArgs a) {
  __shared__ float sh[32];
  __shared__ int s_ok;
  __shared__ bool s_last;
  // 1. announce + wait for every peer's bucket
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    uint64_t* dst = reinterpret_cast<uint64_t*>(a.sig.p[threadIdx.x]) + a.rank;
    st_release_sys_u64(dst, (uint64_t)a.epoch);
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world) {
    const uint64_t* src = reinterpret_cast<const uint64_t*>(a.sig.p[a.rank]) + threadIdx.x;
    if (!wait_epoch(src, a.epoch, 0, a.wait_limit)) {
      set_error(a.err, ERR_WAIT_PEER);
      s_ok = 0;
    }
  }
  __syncthreads();
  float acc = 0.f;
  if (s_ok) {
    const long n4 = a.n >> 2;
    const long lo4 = a.lo >> 2;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (long)gridDim.x * blockDim.x) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
      for (int r = 0; r < a.world; ++r) {
        const float4 v = ld_volatile_f4(reinterpret_cast<const float4*>(a.grads.p[r]) + lo4 + i);
        s.x += v.x;
        s.y += v.y;
        s.z += v.z;
        s.w += v.w;
      }
      reinterpret_cast<float4*>(a.shard_out)[i] = s;
      acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
  }
  // 2. deterministic two-stage sum of squares; the last block publishes it to every peer
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) {
      a.partials[blockIdx.x] = s;
      __threadfence();
      const unsigned int done = atomicAdd(a.counter, 1u);
      s_last = (done == gridDim.x - 1);
    }
  }
  __syncthreads();
  if (s_last) {
    float t = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) t += __ldcg(a.partials + i);
    t = warp_sum(t);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = t;
    __syncthreads();
    if (threadIdx.x < 32) {
      float s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
      s = warp_sum(s);
      s = __shfl_sync(0xffffffffu, s, 0);
      if (threadIdx.x < a.world) {
        uint64_t* dst = reinterpret_cast<uint64_t*>(a.sig.p[threadIdx.x]) + a.world + a.rank;
        st_release_sys_u64(dst, ((uint64_t)a.epoch << 32) | (uint64_t)__float_as_uint(s));
      }
      if (threadIdx.x == 0) *a.counter = 0u;
    }
  }
}

struct DpAdamArgs {
  PeerPtrs weights;  // bf16 weight buffer base of every rank
  PeerPtrs sig;
  float* master;
  float* m;
  float* v;
  const float* g;    // reduced shard
  float* norm_out;   // local: global gradient norm (for logging)
  unsigned int* counter;
  long lo, n;        // shard range, multiples of 8
  int rank, world;
  uint32_t epoch;
  float lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, extra_scale;
  const float* decay_mask;  // null = decay everything; else per-element 0/1 for the shard
  long long wait_limit;
  int* err;
};

__global__ void __launch_bounds__(256) dp_adamw_ag_kernel(const DpAdamArgs a) {
  __shared__ float s_coef;
  __shared__ int s_ok;
  __shared__ bool s_last;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < 32) {
    float ss = 0.f;
    bool ok = true;
    if (threadIdx.x < a.world) {
      const uint64_t* src =
          reinterpret_cast<const uint64_t*>(a.sig.p[a.rank]) + a.world + threadIdx.x;
      ok = wait_epoch(src, a.epoch, 32, a.wait_limit);
      if (ok) ss = __uint_as_float((uint32_t)ld_acquire_sys_u64(src));
    }
    ok = __all_sync(0xffffffffu, ok);
    // fixed-order sum over ranks so every rank derives the identical coefficient
    float total = 0.f;
    for (int r = 0; r < a.world; ++r) total += __shfl_sync(0xffffffffu, ss, r);
    if (threadIdx.x == 0) {
      if (!ok) {
        set_error(a.err, ERR_WAIT_PEER);
        s_ok = 0;
      }
      const float norm = sqrtf(total);
      float c = 1.f;
      if (a.max_norm > 0.f) c = fminf(1.f, a.max_norm / (norm + 1e-6f));
      s_coef = c * a.extra_scale;
      if (blockIdx.x == 0 && a.norm_out) a.norm_out[0] = norm;
    }
  }
  __syncthreads();
  if (s_ok) {
    const float coef = s_coef;
    const long n8 = a.n >> 3;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
         i += (long)gridDim.x * blockDim.x) {
      float P[8], M[8], V[8], G[8], D[8];
      *reinterpret_cast<float4*>(P) = reinterpret_cast<const float4*>(a.master)[2 * i];
      *reinterpret_cast<float4*>(P + 4) = reinterpret_cast<const float4*>(a.master)[2 * i + 1];
      *reinterpret_cast<float4*>(M) = reinterpret_cast<const float4*>(a.m)[2 * i];
      *reinterpret_cast<float4*>(M + 4) = reinterpret_cast<const float4*>(a.m)[2 * i + 1];
      *reinterpret_cast<float4*>(V) = reinterpret_cast<const float4*>(a.v)[2 * i];
      *reinterpret_cast<float4*>(V + 4) = reinterpret_cast<const float4*>(a.v)[2 * i + 1];
      *reinterpret_cast<float4*>(G) = reinterpret_cast<const float4*>(a.g)[2 * i];
      *reinterpret_cast<float4*>(G + 4) = reinterpret_cast<const float4*>(a.g)[2 * i + 1];
      if (a.decay_mask) {
        *reinterpret_cast<float4*>(D) = reinterpret_cast<const float4*>(a.decay_mask)[2 * i];
        *reinterpret_cast<float4*>(D + 4) = reinterpret_cast<const float4*>(a.decay_mask)[2 * i + 1];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gr = G[j] * coef;
        M[j] = a.beta1 * M[j] + (1.f - a.beta1) * gr;
        V[j] = a.beta2 * V[j] + (1.f - a.beta2) * gr * gr;
        const float wd = a.decay_mask ? a.wd * D[j] : a.wd;
        P[j] = P[j] - a.lr * ((M[j] / a.bc1) / (sqrtf(V[j] / a.bc2) + a.eps) + wd * P[j]);
      }
      reinterpret_cast<float4*>(a.master)[2 * i] = *reinterpret_cast<float4*>(P);
      reinterpret_cast<float4*>(a.master)[2 * i + 1] = *reinterpret_cast<float4*>(P + 4);
      reinterpret_cast<float4*>(a.m)[2 * i] = *reinterpret_cast<float4*>(M);
      reinterpret_cast<float4*>(a.m)[2 * i + 1] = *reinterpret_cast<float4*>(M + 4);
      reinterpret_cast<float4*>(a.v)[2 * i] = *reinterpret_cast<float4*>(V);
      reinterpret_cast<float4*>(a.v)[2 * i + 1] = *reinterpret_cast<float4*>(V + 4);
      uint4 w;
      w.x = pack_bf16x2(P[0], P[1]);
      w.y = pack_bf16x2(P[2], P[3]);
      w.z = pack_bf16x2(P[4], P[5]);
      w.w = pack_bf16x2(P[6], P[7]);
      const long e = (a.lo >> 3) + i;
      // all-gather: push the shard to every rank, starting with the next neighbour so the eight
      // ranks do not all hit the same destination at once
#pragma unroll 1
      for (int k = 0; k < a.world; ++k) {
        const int r = (a.rank + 1 + k) % a.world;
        reinterpret_cast<uint4*>(a.weights.p[r])[e] = w;
      }
    }
  }
  // "weights landed" handshake by the last block to finish
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(a.counter, 1u);
    s_last = (done == gridDim.x - 1);
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < a.world) {
      uint64_t* dst = reinterpret_cast<uint64_t*>(a.sig.p[threadIdx.x]) + 2 * a.world + a.rank;
      st_release_sys_u64(dst, (uint64_t)a.epoch);
      const uint64_t* src =
          reinterpret_cast<const uint64_t*>(a.sig.p[a.rank]) + 2 * a.world + threadIdx.x;
      if (!wait_epoch(src, a.epoch, 0, a.wait_limit)) set_error(a.err, ERR_WAIT_PEER);
    }
    if (threadIdx.x == 0) *a.counter = 0u;
  }
}

}  // namespace bb

using namespace bb;

BB_API int bb_dp_signal_bytes(int world) { return 3 * world * 8; }

// scratch: >= (1024 + 2) floats of local device memory, zeroed once at allocation
//   [0,1024) partial sums, [1024] counter for kernel 1, [1025] counter for kernel 2.
BB_API int bb_dp_scratch_floats() { return 1026; }

// grad_ptrs / sig_ptrs / weight_ptrs: host arrays of `world` device pointers (every rank's buffer).
BB_API int bb_dp_reduce(const uint64_t* grad_ptrs, const uint64_t* sig_ptrs, float* shard_out,
                        float* scratch, long lo, long n, int rank, int world, unsigned int epoch,
                        double wait_seconds, void* stream) {
  if (world < 1 || world > MAX_RANKS || (lo & 3) || (n & 3)) return BB_EARG;
  DpReduceArgs a{};
  for (int r = 0; r < world; ++r) {
    a.grads.p[r] = reinterpret_cast<void*>(grad_ptrs[r]);
    a.sig.p[r] = reinterpret_cast<void*>(sig_ptrs[r]);
  }
  a.shard_out = shard_out;
  a.partials = scratch;
  a.counter = reinterpret_cast<unsigned int*>(scratch + 1024);
  a.lo = lo;
  a.n = n;
  a.rank = rank;
  a.world = world;
  a.epoch = epoch;
  a.wait_limit = (long long)(wait_seconds * 1.9e9);
  a.err = device_error_word();
  long blocks = ((n >> 2) + 255) / 256;
  const long cap = (long)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks > 1024) blocks = 1024;
  if (blocks < 1) blocks = 1;
  dp_reduce_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

BB_API int bb_dp_adamw_allgather(const uint64_t* weight_ptrs, const uint64_t* sig_ptrs,
                                 float* master, float* m, float* v, const float* g,
                                 const float* decay_mask, float* norm_out, float* scratch, long lo,
                                 long n, int rank, int world, unsigned int epoch, float lr,
                                 float beta1, float beta2, float eps, float wd, int step,
                                 float max_norm, float extra_scale, double wait_seconds,
                                 void* stream) {
  if (world < 1 || world > MAX_RANKS || (lo & 7) || (n & 7)) return BB_EARG;
  DpAdamArgs a{};
  for (int r = 0; r < world; ++r) {
    a.weights.p[r] = reinterpret_cast<void*>(weight_ptrs[r]);
    a.sig.p[r] = reinterpret_cast<void*>(sig_ptrs[r]);
  }
  a.master = master;
  a.m = m;
  a.v = v;
  a.g = g;
  a.norm_out = norm_out;
  a.counter = reinterpret_cast<unsigned int*>(scratch + 1025);
  a.lo = lo;
  a.n = n;
  a.rank = rank;
  a.world = world;
  a.epoch = epoch;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.wd = wd;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.max_norm = max_norm;
  a.extra_scale = extra_scale;
  a.decay_mask = decay_mask;
  a.wait_limit = (long long)(wait_seconds * 1.9e9);
  a.err = device_error_word();
  long blocks = ((n >> 3) + 255) / 256;
  const long cap = (long)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  dp_adamw_ag_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}
