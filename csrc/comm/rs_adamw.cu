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

// ------------------------------------------------------------------------------------------------
// Bucketed reduce-scatter with bf16 on the wire, launched per bucket while backward still runs.
//
// The flat gradient range is cut into buckets that never cross a rank's shard, so every bucket has
// one OWNER (the rank whose optimiser shard contains it).  All ranks launch this kernel for every
// bucket in the same order on a side stream, as soon as the last micro-batch's backward has
// finished the parameters of the bucket:
//   every other rank  casts its fp32 gradients of the bucket to bf16 into its own symmetric staging
//                     buffer (local traffic only) and bumps its "staged" sequence word at the owner
//   the owner         waits (bounded) until every peer's sequence word reached this bucket, then
//                     sums, in rank order, its own fp32 values and the peers' bf16 values (plain
//                     peer loads, half the NVLink bytes of an fp32 exchange), writes the reduced
//                     fp32 shard slice and the bucket's sum of squares (two-stage, fixed order)
// Signal words [3R, 4R) of the owner hold the peers' sequence numbers (monotonic, never reset).
struct DpBucketArgs {
  const float* grads;         // this rank's fp32 gradient bucket array (whole flat range)
  PeerPtrs stage;             // bf16 staging array of every rank (whole flat range)
  PeerPtrs sig;
  float* shard_out;           // owner: reduced shard (indexed from the shard start)
  float* partials;            // owner: [gridDim.x] scratch
  float* bucket_sumsq;        // owner: where this bucket's sum of squares goes
  unsigned int* counter;      // zeroed; reset by the kernel
  long start, n;              // bucket range in elements (multiples of 8)
  long shard_lo;              // first element of the owner's shard
  int rank, world, owner;
  unsigned long long seq;     // sequence number of this bucket (grows by one per bucket launch)
  long long wait_limit;
  int* err;
};

__global__ void __launch_bounds__(256) dp_bucket_kernel(const DpBucketArgs a) {
  __shared__ float sh[32];
  __shared__ int s_ok;
  __shared__ bool s_last;
  const long n8 = a.n >> 3;
  const long s8 = a.start >> 3;
  const long stride = (long)gridDim.x * blockDim.x;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (a.rank != a.owner) {
    // ---- stage my contribution as bf16 and tell the owner
    uint4* dst = reinterpret_cast<uint4*>(a.stage.p[a.rank]) + s8;
    const float4* src = reinterpret_cast<const float4*>(a.grads) + 2 * s8;
    for (long i = tid; i < n8; i += stride) {
      const float4 x = src[2 * i], y = src[2 * i + 1];
      uint4 w;
      w.x = pack_bf16x2(x.x, x.y);
      w.y = pack_bf16x2(x.z, x.w);
      w.z = pack_bf16x2(y.x, y.y);
      w.w = pack_bf16x2(y.z, y.w);
      dst[i] = w;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();  // one per block: cumulative over the block's writes ordered by the barrier
      if (atomicAdd(a.counter, 1u) == gridDim.x - 1) {
        *a.counter = 0u;
        st_release_sys_u64(reinterpret_cast<uint64_t*>(a.sig.p[a.owner]) + 3 * a.world + a.rank,
                           (uint64_t)a.seq);
      }
    }
    return;
  }
  // ---- owner: wait for every peer's staged copy, reduce in rank order
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(a.sig.p[a.rank]) + 3 * a.world + threadIdx.x;
    const long long t0 = clock64();
    while (ld_acquire_sys_u64(f) < (uint64_t)a.seq) {
      if (clock64() - t0 > a.wait_limit) {
        set_error(a.err, ERR_WAIT_PEER);
        s_ok = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  float acc = 0.f;
  if (s_ok) {
    const float4* own = reinterpret_cast<const float4*>(a.grads) + 2 * s8;
    float4* out = reinterpret_cast<float4*>(a.shard_out) + 2 * ((a.start - a.shard_lo) >> 3);
    for (long i = tid; i < n8; i += stride) {
      uint4 raw[MAX_RANKS];
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)   // every peer load in flight before the first add
        if (r < a.world && r != a.rank)
          raw[r] = ld_volatile_u4(reinterpret_cast<const uint4*>(a.stage.p[r]) + s8 + i);
      const float4 x = own[2 * i], y = own[2 * i + 1];
      float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r) {
        if (r >= a.world) continue;
        if (r == a.rank) {
          s[0] += x.x; s[1] += x.y; s[2] += x.z; s[3] += x.w;
          s[4] += y.x; s[5] += y.y; s[6] += y.z; s[7] += y.w;
        } else {
          const uint32_t w[4] = {raw[r].x, raw[r].y, raw[r].z, raw[r].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            s[2 * q] += __uint_as_float(w[q] << 16);
            s[2 * q + 1] += __uint_as_float(w[q] & 0xFFFF0000u);
          }
        }
      }
      out[2 * i] = make_float4(s[0], s[1], s[2], s[3]);
      out[2 * i + 1] = make_float4(s[4], s[5], s[6], s[7]);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc += s[q] * s[q];
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) {
      a.partials[blockIdx.x] = v;
      __threadfence();
      s_last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
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
      float v = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
      v = warp_sum(v);
      if (threadIdx.x == 0) {
        *a.bucket_sumsq = v;
        *a.counter = 0u;
      }
    }
  }
}

// Sum this rank's bucket sums of squares in bucket order and send the total to every peer (the
// AdamW kernel that follows waits for all ranks' totals and forms the clip coefficient).
__global__ void dp_publish_norm_kernel(PeerPtrs sig, const float* bucket_sumsq, int n_owned, int rank,
                                       int world, uint32_t epoch) {
  if (threadIdx.x < world) {
    float t = 0.f;
    for (int i = 0; i < n_owned; ++i) t += bucket_sumsq[i];
    uint64_t* dst = reinterpret_cast<uint64_t*>(sig.p[threadIdx.x]) + world + rank;
    st_release_sys_u64(dst, ((uint64_t)epoch << 32) | (uint64_t)__float_as_uint(t));
  }
}

}  // namespace bb

using namespace bb;

BB_API int bb_dp_signal_bytes(int world) { return 4 * world * 8; }

// scratch: >= (1024 + 2) floats of local device memory, zeroed once at allocation
//   [0,1024) partial sums, [1024] counter for kernel 1, [1025] counter for kernel 2,
//   [1026] counter of the bucket kernel.
BB_API int bb_dp_scratch_floats() { return 1028; }

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

// One bucket of the overlapped reduce-scatter (see dp_bucket_kernel).  grads: this rank's fp32 flat
// gradients; stage_ptrs[r]: rank r's bf16 staging array (flat, symmetric); scratch as in
// bb_dp_reduce plus one more counter word: >= 1028 floats, zeroed once.  `seq` must grow by one with
// every call on every rank (all ranks make the same calls in the same order).  max_ctas bounds the
// grid so the kernel can share the GPU with the backward pass (0 = 4 CTAs per SM).
BB_API int bb_dp_bucket_reduce(const float* grads, const uint64_t* stage_ptrs, const uint64_t* sig_ptrs,
                               float* shard_out, float* bucket_sumsq, float* scratch, long start, long n,
                               long shard_lo, int rank, int world, int owner, unsigned long long seq,
                               int max_ctas, double wait_seconds, void* stream) {
  if (world < 1 || world > MAX_RANKS || (start & 7) || (n & 7) || n <= 0 || owner < 0 || owner >= world)
    return BB_EARG;
  DpBucketArgs a{};
  a.grads = grads;
  for (int r = 0; r < world; ++r) {
    a.stage.p[r] = reinterpret_cast<void*>(stage_ptrs[r]);
    a.sig.p[r] = reinterpret_cast<void*>(sig_ptrs[r]);
  }
  a.shard_out = shard_out;
  a.partials = scratch;
  a.counter = reinterpret_cast<unsigned int*>(scratch + 1026);
  a.bucket_sumsq = bucket_sumsq;
  a.start = start;
  a.n = n;
  a.shard_lo = shard_lo;
  a.rank = rank;
  a.world = world;
  a.owner = owner;
  a.seq = seq;
  a.wait_limit = (long long)(wait_seconds * 1.9e9);
  a.err = device_error_word();
  long blocks = ((n >> 3) + 255) / 256;
  long cap = max_ctas > 0 ? max_ctas : (long)sm_count() * 4;
  if (cap > 1024) cap = 1024;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  dp_bucket_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

BB_API int bb_dp_publish_norm(const uint64_t* sig_ptrs, const float* bucket_sumsq, int n_owned, int rank,
                              int world, unsigned int epoch, void* stream) {
  if (world < 1 || world > MAX_RANKS || n_owned < 0) return BB_EARG;
  PeerPtrs s{};
  for (int r = 0; r < world; ++r) s.p[r] = reinterpret_cast<void*>(sig_ptrs[r]);
  dp_publish_norm_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(s, bucket_sumsq, n_owned, rank, world, epoch);
  return (int)cudaGetLastError();
}
