// Masked cross-entropy over bf16 logits [n, V] (V ~ 152k): one block per row.
//   forward : loss[r] = lse(r) - logit[r, tgt]      (0 for ignored rows), lse saved
//   fused   : same, and logits are overwritten IN PLACE with the gradient
//             (softmax - onehot) * scale            (0 for ignored rows)
// so the LM-head backward GEMMs can consume the buffer directly.  target < 0 means "ignore"
// (the reference's IGNORE sentinel 0xFFFFFFFF reinterpreted as int32 is -1).
// Reference contracts: crates/kernels/wgsl/{ce_value_masked,ce_stats,ce_grad_stats}.wgsl.
#include "../common/host.hpp"
#include "../common/ptx.cuh"
#include "../common/vec.cuh"

namespace bb {

__device__ __forceinline__ void block_reduce_max_sum(float& m, float& s, float* sh) {
  // online-softmax merge across the block: (m, s) pairs with s = sum exp(x - m)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mm = fmaxf(m, m2);
    const float e1 = (m == -INFINITY) ? 0.f : __expf(m - mm);
    const float e2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mm);
    s = s * e1 + s2 * e2;
    m = mm;
  }
  if (lane == 0) {
    sh[warp * 2] = m;
    sh[warp * 2 + 1] = s;
  }
  __syncthreads();
  if (warp == 0) {
    float mw = lane < nw ? sh[lane * 2] : -INFINITY;
    float sw = lane < nw ? sh[lane * 2 + 1] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, mw, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, sw, o);
      const float mm = fmaxf(mw, m2);
      const float e1 = (mw == -INFINITY) ? 0.f : __expf(mw - mm);
      const float e2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mm);
      sw = sw * e1 + s2 * e2;
      mw = mm;
    }
    if (lane == 0) {
      sh[64] = mw;
      sh[65] = sw;
    }
  }
  __syncthreads();
  m = sh[64];
  s = sh[65];
}

template <bool GRAD>
__global__ void __launch_bounds__(512)
ce_kernel(__nv_bfloat16* __restrict__ logits, long ld, const int* __restrict__ tgt,
          float* __restrict__ loss, float* __restrict__ lse_out, int V, const float* scale_ptr,
          float scale_mul BB_ERR_PARAM) {
  __shared__ float sh[66];
  const int r = blockIdx.x;
  __nv_bfloat16* row = logits + (size_t)r * ld;
  const int t = tgt[r];
  // a negative target is the ignore mark; one past the vocabulary is a caller error that production
  // builds treat as ignored and bounds-checking builds also record
  if (t >= 0 && threadIdx.x == 0) (void)BB_INDEX_OK(t, V);
  const int nv = V >> 3;  // V % 8 == 0 enforced by the launcher
  if (t < 0 || t >= V) {
    if (threadIdx.x == 0) {
      loss[r] = 0.f;
      if (lse_out) lse_out[r] = 0.f;
    }
    if (GRAD) {
      bf16x8 z;
#pragma unroll
      for (int i = 0; i < 4; ++i) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
      for (int i = threadIdx.x; i < nv; i += blockDim.x) reinterpret_cast<bf16x8*>(row)[i] = z;
    }
    return;
  }
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(row)[i], f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    const float mm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - mm);
    s = s * __expf(m - mm) + acc;
    m = mm;
  }
  if (m == -INFINITY) s = 0.f;
  block_reduce_max_sum(m, s, sh);
  const float lse = m + __logf(s);
  if (threadIdx.x == 0) {
    loss[r] = lse - __bfloat162float(row[t]);
    if (lse_out) lse_out[r] = lse;
  }
  if (GRAD) {
    __syncthreads();  // row[t] read above must precede the overwrite
    const float scale = (scale_ptr ? *scale_ptr : 1.f) * scale_mul;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(row)[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float p = __expf(f[j] - lse);
        if (i * 8 + j == t) p -= 1.f;
        f[j] = p * scale;
      }
      reinterpret_cast<bf16x8*>(row)[i] = pack8(f);
    }
  }
}

}  // namespace bb

using namespace bb;

// logits: bf16 [n, ld] (first V columns used, V % 8 == 0); tgt: int32[n] (<0 ignored);
// loss, lse: fp32[n].  grad != 0 overwrites logits with dlogits * (*scale_ptr) * scale_mul.
BB_API int bb_cross_entropy(void* logits, long ld, const int* tgt, float* loss, float* lse, int n,
                            int V, int grad, const float* scale_ptr, float scale_mul,
                            void* stream) {
  if (n <= 0) return BB_OK;
  if (V % 8 || ld % 8) return BB_EARG;
  const int threads = V >= 8192 ? 512 : 128;
  if (grad)
    ce_kernel<true><<<n, threads, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, ld, tgt, loss,
                                                            lse, V, scale_ptr, scale_mul BB_ERR_ARG);
  else
    ce_kernel<false><<<n, threads, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, ld, tgt,
                                                             loss, lse, V, scale_ptr, scale_mul BB_ERR_ARG);
  return (int)cudaGetLastError();
}
