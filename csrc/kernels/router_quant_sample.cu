// Small-row kernels: MoE router (softmax over experts + greedy top-k, ties to the lowest index),
// per-row symmetric int8 quantisation (W8A8 activations / weights), and greedy argmax sampling.
// Reference contracts: crates/kernels/wgsl/{router_gate_train,router_topk_compact,expert_counts,
// max_abs_row,quant_pack,argmax_part,argmax_final}.wgsl and crates/model/src/int8.rs:33-59.
#include "../common/host.hpp"
#include "../common/ptx.cuh"
#include "../common/vec.cuh"

namespace bb {

// One warp per token; E <= 256 (E % 32 == 0 not required).
// logits fp32 [n, E] -> probs fp32 [n, E] (optional), lse [n] (optional),
// topk_idx int32 [n, k], topk_w fp32 [n, k] (renormalised when norm != 0, then * scale),
// counts int32 [E] (+= number of tokens routed to e).
__global__ void router_topk_kernel(const float* __restrict__ logits, float* __restrict__ probs,
                                   float* __restrict__ lse_out, int* __restrict__ topk_idx,
                                   float* __restrict__ topk_w, int* __restrict__ counts, int n,
                                   int E, int k, int norm, float scale) {
  const int tok = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tok >= n) return;
  constexpr int MAXP = 8;
  float v[MAXP];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAXP; ++j) {
    const int e = j * 32 + lane;
    v[j] = e < E ? logits[(size_t)tok * E + e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < MAXP; ++j) {
    v[j] = (j * 32 + lane < E) ? __expf(v[j] - mx) : 0.f;
    s += v[j];
  }
  s = warp_sum(s);
  const float inv = 1.f / s;
#pragma unroll
  for (int j = 0; j < MAXP; ++j) {
    v[j] *= inv;
    const int e = j * 32 + lane;
    if (probs && e < E) probs[(size_t)tok * E + e] = v[j];
  }
  if (lane == 0 && lse_out) lse_out[tok] = mx + __logf(s);
  float wsum = 0.f;
  float my_w = 0.f;
  int my_i = 0;
  for (int t = 0; t < k; ++t) {
    float best = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
      const int e = j * 32 + lane;
      if (e < E && v[j] > best) {  // strict > keeps the lowest index inside a lane
        best = v[j];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
      const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
      if (b2 > best || (b2 == best && i2 < bi)) {
        best = b2;
        bi = i2;
      }
    }
#pragma unroll
    for (int j = 0; j < MAXP; ++j)
      if (j * 32 + lane == bi) v[j] = -2.f;  // remove the winner
    wsum += best;
    if (lane == t) {
      my_w = best;
      my_i = bi;
    }
  }
  if (lane < k) {
    const float w = (norm ? my_w / wsum : my_w) * scale;
    topk_idx[(size_t)tok * k + lane] = my_i;
    topk_w[(size_t)tok * k + lane] = w;
    if (counts) atomicAdd(counts + my_i, 1);
  }
}

// Per-row symmetric int8: s = max|x| / 127 (>= 1e-8), q = clamp(rint(x / s), +-127). Warp per row.
template <typename T>
__global__ void quant_rows_kernel(const T* __restrict__ x, int8_t* __restrict__ q,
                                  float* __restrict__ scale, int rows, int k) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + (size_t)row * k;
  float mx = 0.f;
  for (int i = lane; i < k; i += 32) mx = fmaxf(mx, fabsf((float)xr[i]));
  mx = warp_max(mx);
  const float s = fmaxf(mx / 127.f, 1e-8f);
  if (lane == 0) scale[row] = s;
  const float inv = 1.f / s;
  int8_t* qr = q + (size_t)row * k;
  for (int i = lane; i < k; i += 32) {
    float r = rintf((float)xr[i] * inv);
    r = fminf(127.f, fmaxf(-127.f, r));
    qr[i] = (int8_t)r;
  }
}

// bf16 rows with k % 8 == 0 and a 16-byte aligned base: 16-byte loads, 8-byte packed stores (the
// scalar form above moved 2 bytes per lane per load and was several times off the copy roofline).
__global__ void quant_rows_bf16_vec_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q,
                                           float* __restrict__ scale, int rows, int k) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nv = k >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)row * k);
  float mx = 0.f;
  for (int i = lane; i < nv; i += 32) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(f[j]));
  }
  mx = warp_max(mx);
  const float s = fmaxf(mx / 127.f, 1e-8f);
  if (lane == 0) scale[row] = s;
  const float inv = 1.f / s;
  uint2* qr = reinterpret_cast<uint2*>(q + (size_t)row * k);
  for (int i = lane; i < nv; i += 32) {
    float f[8];
    unpack8(xr[i], f);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float r = fminf(127.f, fmaxf(-127.f, rintf(f[j] * inv)));
      w[j >> 2] |= ((uint32_t)(int)r & 0xffu) << (8 * (j & 3));
    }
    qr[i] = make_uint2(w[0], w[1]);
  }
}

// Greedy head: out[r] = argmax_c logits[r, c] (lowest index on ties).  One block per row.
__global__ void argmax_rows_kernel(const __nv_bfloat16* __restrict__ logits, long ld, int V,
                                   int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const __nv_bfloat16* row = logits + (size_t)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float f = __bfloat162float(row[i]);
    if (f > best) {
      best = f;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
    if (b2 > best || (b2 == best && i2 < bi)) {
      best = b2;
      bi = i2;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
      const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
      if (b2 > best || (b2 == best && i2 < bi)) {
        best = b2;
        bi = i2;
      }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

// Top-K per row by K rounds of "largest remaining" (value descending, lowest index first on ties —
// the order of crates/kernels/wgsl/topk_extract_step.wgsl).  One block per row; every round is one
// pass over the row (it stays in L2), "remaining" = lexicographically after the previous pick.
__global__ void topk_rows_kernel(const __nv_bfloat16* __restrict__ logits, long ld, int V, int K,
                                 int* __restrict__ out_idx, float* __restrict__ out_val) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float s_last_v;
  __shared__ int s_last_i;
  const __nv_bfloat16* row = logits + (size_t)blockIdx.x * ld;
  if (threadIdx.x == 0) {
    s_last_v = INFINITY;
    s_last_i = -1;
  }
  __syncthreads();
  for (int k = 0; k < K; ++k) {
    const float lv = s_last_v;
    const int li = s_last_i;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float f = __bfloat162float(row[i]);
      const bool remaining = f < lv || (f == lv && i > li);
      if (remaining && (f > best || (f == best && i < bi))) {
        best = f;
        bi = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
      const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
      if (b2 > best || (b2 == best && i2 < bi)) {
        best = b2;
        bi = i2;
      }
    }
    if ((threadIdx.x & 31) == 0) {
      sv[threadIdx.x >> 5] = best;
      si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      const int nw = blockDim.x >> 5;
      best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
      bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
        if (b2 > best || (b2 == best && i2 < bi)) {
          best = b2;
          bi = i2;
        }
      }
      if (threadIdx.x == 0) {
        const bool found = bi != 0x7fffffff;
        out_idx[(size_t)blockIdx.x * K + k] = found ? bi : 0;
        out_val[(size_t)blockIdx.x * K + k] = found ? best : -INFINITY;
        s_last_v = found ? best : -INFINITY;
        s_last_i = found ? bi : 0x7fffffff;
      }
    }
    __syncthreads();
  }
}

}  // namespace bb

using namespace bb;

BB_API int bb_router_topk(const float* logits, float* probs, float* lse, int* topk_idx,
                          float* topk_w, int* counts, int n, int E, int k, int norm, float scale,
                          void* stream) {
  if (n <= 0) return BB_OK;
  if (E > 256 || k > 32 || k > E || k < 1) return BB_EARG;
  router_topk_kernel<<<(n + 7) / 8, 256, 0, (cudaStream_t)stream>>>(logits, probs, lse, topk_idx,
                                                                   topk_w, counts, n, E, k, norm,
                                                                   scale);
  return (int)cudaGetLastError();
}

// dtype: 0 = bf16 input, 1 = fp32 input.
BB_API int bb_quant_rows(const void* x, void* q, float* scale, int rows, int k, int dtype,
                         void* stream) {
  if (rows <= 0) return BB_OK;
  const int grid = (rows + 7) / 8;
  if (dtype == 0 && k % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q)) & 15) == 0)
    quant_rows_bf16_vec_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x,
                                                                       (int8_t*)q, scale, rows, k);
  else if (dtype == 0)
    quant_rows_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (int8_t*)q, scale, rows, k);
  else
    quant_rows_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)x, (int8_t*)q,
                                                                    scale, rows, k);
  return (int)cudaGetLastError();
}

// idx[rows, K] int32, val[rows, K] fp32: the K largest logits of every row, descending.
BB_API int bb_topk_rows(const void* logits, long ld, int rows, int V, int K, int* idx, float* val,
                        void* stream) {
  if (rows <= 0) return BB_OK;
  if (K < 1 || K > V) return BB_EARG;
  topk_rows_kernel<<<rows, 512, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, V, K,
                                                          idx, val);
  return (int)cudaGetLastError();
}

BB_API int bb_argmax_rows(const void* logits, long ld, int rows, int V, int* out, void* stream) {
  if (rows <= 0) return BB_OK;
  argmax_rows_kernel<<<rows, 512, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, V,
                                                            out);
  return (int)cudaGetLastError();
}
