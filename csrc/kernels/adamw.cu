// Optimiser kernels over flat fp32 buffers: AdamW (decoupled weight decay, bias correction, eps
// outside the sqrt) writing bf16 working weights, the two-stage deterministic global gradient
// norm, and the clip coefficient  coef = min(1, max_norm / (||g|| + 1e-6)) * extra_scale.
// Reference contracts: crates/kernels/wgsl/{adamw,gradnorm_part,clip_coef_wg,grad_scale_buf}.wgsl.
#include "../common/host.hpp"
#include "../common/ptx.cuh"

namespace bb {

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2;  // bc = 1 - beta^t
};

// p,m,v: fp32 master / moments; g: fp32 gradient (scaled by *coef); w16: bf16 copy of p (or null).
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ g, __nv_bfloat16* __restrict__ w16, long n,
                             AdamArgs a, const float* __restrict__ coef_ptr) {
  const float coef = coef_ptr ? *coef_ptr : 1.f;
  const long n4 = n >> 2;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float* P = &pp.x;
    float* M = &mm.x;
    float* V = &vv.x;
    const float* G = &gg.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gr = G[j] * coef;
      M[j] = a.beta1 * M[j] + (1.f - a.beta1) * gr;
      V[j] = a.beta2 * V[j] + (1.f - a.beta2) * gr * gr;
      const float mh = M[j] / a.bc1, vh = V[j] / a.bc2;
      P[j] = P[j] - a.lr * (mh / (sqrtf(vh) + a.eps) + a.wd * P[j]);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (w16) {
      uint2 o;
      o.x = pack_bf16x2(P[0], P[1]);
      o.y = pack_bf16x2(P[2], P[3]);
      reinterpret_cast<uint2*>(w16)[i] = o;
    }
  }
  // tail (n % 4)
  const long base = n4 << 2;
  const long t = base + (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n && blockIdx.x == 0) {
    const float gr = g[t] * coef;
    const float mj = a.beta1 * m[t] + (1.f - a.beta1) * gr;
    const float vj = a.beta2 * v[t] + (1.f - a.beta2) * gr * gr;
    m[t] = mj;
    v[t] = vj;
    const float pj = p[t] - a.lr * ((mj / a.bc1) / (sqrtf(vj / a.bc2) + a.eps) + a.wd * p[t]);
    p[t] = pj;
    if (w16) w16[t] = __float2bfloat16(pj);
  }
}

// Stage 1: per-block partial sums of squares (fixed grid => deterministic reduction order).
__global__ void sumsq_partial_kernel(const float* __restrict__ g, long n, float* __restrict__ part) {
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
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) part[blockIdx.x] = s;
  }
}

// Stage 2: out[0] (+)= sum(part[0..np))
__global__ void sumsq_final_kernel(const float* __restrict__ part, int np, float* __restrict__ out,
                                   int accumulate) {
  __shared__ float sh[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < np; i += blockDim.x) acc += part[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
  }
}

__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float extra,
                                 float* __restrict__ coef, float* __restrict__ norm_out) {
  const float norm = sqrtf(sumsq[0]);
  if (norm_out) norm_out[0] = norm;
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (norm + 1e-6f));
  coef[0] = c * extra;
}

__global__ void scale_f32_kernel(float* __restrict__ x, long n, const float* __restrict__ coef_ptr,
                                 float mul) {
  const float c = (coef_ptr ? *coef_ptr : 1.f) * mul;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long)gridDim.x * blockDim.x)
    x[i] *= c;
}

}  // namespace bb

using namespace bb;

BB_API int bb_adamw(float* p, float* m, float* v, const float* g, void* w16, long n, float lr,
                    float beta1, float beta2, float eps, float wd, int step, const float* coef_ptr,
                    void* stream) {
  if (n <= 0) return BB_OK;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(g)) & 15)
    return BB_EARG;
  if (w16 && (reinterpret_cast<uintptr_t>(w16) & 7)) return BB_EARG;
  AdamArgs a{lr, beta1, beta2, eps, wd, 1.f - powf(beta1, (float)step),
             1.f - powf(beta2, (float)step)};
  long blocks = ((n >> 2) + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  adamw_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(p, m, v, g, (__nv_bfloat16*)w16, n, a,
                                                             coef_ptr);
  return (int)cudaGetLastError();
}

// out[0] (+)= sum g^2.  `scratch` must hold bb_sumsq_scratch_floats() floats.
BB_API int bb_sumsq_scratch_floats() { return 1024; }

BB_API int bb_sumsq(const float* g, long n, float* scratch, float* out, int accumulate,
                    void* stream) {
  if (n < 0) return BB_EARG;
  if (reinterpret_cast<uintptr_t>(g) & 15) return BB_EARG;
  long blocks = ((n >> 2) + 511) / 512;
  if (blocks > 1024) blocks = 1024;
  if (blocks < 1) blocks = 1;
  sumsq_partial_kernel<<<(int)blocks, 512, 0, (cudaStream_t)stream>>>(g, n, scratch);
  sumsq_final_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(scratch, (int)blocks, out, accumulate);
  return (int)cudaGetLastError();
}

BB_API int bb_clip_coef(const float* sumsq, float max_norm, float extra, float* coef,
                        float* norm_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(sumsq, max_norm, extra, coef, norm_out);
  return (int)cudaGetLastError();
}

BB_API int bb_scale_f32(float* x, long n, const float* coef_ptr, float mul, void* stream) {
  if (n <= 0) return BB_OK;
  long blocks = (n + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  scale_f32_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(x, n, coef_ptr, mul);
  return (int)cudaGetLastError();
}
