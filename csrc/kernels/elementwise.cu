// Vectorised elementwise kernels: SwiGLU fwd/bwd (on the fused [n, 2*ff] gate|up layout the
// gate/up GEMM writes), tanh-GELU fwd/bwd, residual add, embedding gather / scatter-add, casts.
// Reference contracts: crates/kernels/wgsl/{silu_mul,silu_bwd_da,silu_bwd_db,gelu,gelu_bwd,add2,
// embed,emb_bwd,pos_add,pos_bwd}.wgsl.
#include "../common/host.hpp"
#include "../common/ptx.cuh"
#include "../common/vec.cuh"

namespace bb {


// h[r, c] = silu(gu[r, c]) * gu[r, ff + c];  gu pitch = 2*ff, ff % 8 == 0.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h,
                                  long n_vec, int ffv) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (long)gridDim.x * blockDim.x) {
    const long r = i / ffv;
    const int c = (int)(i % ffv);
    const bf16x8* row = reinterpret_cast<const bf16x8*>(gu) + r * 2 * ffv;
    float g[8], u[8], o[8];
    unpack8(row[c], g);
    unpack8(row[ffv + c], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<bf16x8*>(h)[i] = pack8(o);
  }
}

// dgu[r, c] = dh * u * s*(1 + g*(1-s)),  dgu[r, ff+c] = dh * g*s   (s = sigmoid(g))
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh,
                                  const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long n_vec, int ffv) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (long)gridDim.x * blockDim.x) {
    const long r = i / ffv;
    const int c = (int)(i % ffv);
    const bf16x8* row = reinterpret_cast<const bf16x8*>(gu) + r * 2 * ffv;
    bf16x8* drow = reinterpret_cast<bf16x8*>(dgu) + r * 2 * ffv;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[c], g);
    unpack8(row[ffv + c], u);
    unpack8(reinterpret_cast<const bf16x8*>(dh)[i], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
      du[j] = d[j] * g[j] * s;
    }
    drow[c] = pack8(dg);
    drow[ffv + c] = pack8(du);
  }
}

__device__ __forceinline__ float gelu_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (x + k1 * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
}

__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                long n_vec) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (long)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = gelu_f(f[j]);
    reinterpret_cast<bf16x8*>(y)[i] = pack8(f);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                __nv_bfloat16* __restrict__ dx, long n_vec) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (long)gridDim.x * blockDim.x) {
    float f[8], g[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], f);
    unpack8(reinterpret_cast<const bf16x8*>(dy)[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = g[j] * gelu_grad_f(f[j]);
    reinterpret_cast<bf16x8*>(dx)[i] = pack8(f);
  }
}

__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ y, long n_vec) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (long)gridDim.x * blockDim.x) {
    float f[8], g[8];
    unpack8(reinterpret_cast<const bf16x8*>(a)[i], f);
    unpack8(reinterpret_cast<const bf16x8*>(b)[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] += g[j];
    reinterpret_cast<bf16x8*>(y)[i] = pack8(f);
  }
}

// out[t, :] = emb[tok[t], :] (+ pos_emb[t % T, :])
__global__ void embed_fwd_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ emb,
                                 const __nv_bfloat16* __restrict__ pos_emb, int T,
                                 __nv_bfloat16* __restrict__ out, long n_tok, int dv, int vocab BB_ERR_PARAM) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n_tok * dv;
       i += (long)gridDim.x * blockDim.x) {
    const long t = i / dv;
    const int c = (int)(i % dv);
    int id = tok[t];
    if (!BB_INDEX_OK(id, vocab)) continue;   // bounds-checking builds: recorded, row left untouched
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    bf16x8 v = reinterpret_cast<const bf16x8*>(emb)[(size_t)id * dv + c];
    if (pos_emb) {
      float f[8], g[8];
      unpack8(v, f);
      unpack8(reinterpret_cast<const bf16x8*>(pos_emb)[(size_t)(t % T) * dv + c], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      v = pack8(f);
    }
    reinterpret_cast<bf16x8*>(out)[i] = v;
  }
}

// demb[tok[t], :] += dout[t, :]  (fp32 main-grad, red.global.add) ; dpos[t % T, :] += dout[t, :]
__global__ void embed_bwd_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ dout,
                                 float* __restrict__ demb, float* __restrict__ dpos, int T,
                                 long n_tok, int d, int vocab BB_ERR_PARAM) {
  const int dp = d >> 1;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n_tok * dp;
       i += (long)gridDim.x * blockDim.x) {
    const long t = i / dp;
    const int c = (int)(i % dp) * 2;
    int id = tok[t];
    if (!BB_INDEX_OK(id, vocab)) continue;
    if (id < 0 || id >= vocab) continue;
    const float2 g =
        __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dout + (size_t)t * d + c));
    if (demb) {
      atomicAdd(demb + (size_t)id * d + c, g.x);
      atomicAdd(demb + (size_t)id * d + c + 1, g.y);
    }
    if (dpos) {
      atomicAdd(dpos + (size_t)(t % T) * d + c, g.x);
      atomicAdd(dpos + (size_t)(t % T) * d + c + 1, g.y);
    }
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                     long n) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16(x[i]);
}

}  // namespace bb

using namespace bb;

static inline int ew_grid(long n, int threads = 256) {
  long g = (n + threads - 1) / threads;
  const long cap = (long)sm_count() * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

BB_API int bb_swiglu_fwd(const void* gu, void* h, long rows, int ff, void* stream) {
  if (ff % 8) return BB_EARG;
  const long nv = rows * (ff / 8);
  if (nv <= 0) return BB_OK;
  swiglu_fwd_kernel<<<ew_grid(nv), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)h, nv, ff / 8);
  return (int)cudaGetLastError();
}
BB_API int bb_swiglu_bwd(const void* dh, const void* gu, void* dgu, long rows, int ff,
                         void* stream) {
  if (ff % 8) return BB_EARG;
  const long nv = rows * (ff / 8);
  if (nv <= 0) return BB_OK;
  swiglu_bwd_kernel<<<ew_grid(nv), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dh, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, nv, ff / 8);
  return (int)cudaGetLastError();
}
BB_API int bb_gelu_fwd(const void* x, void* y, long n, void* stream) {
  if (n % 8) return BB_EARG;
  if (n <= 0) return BB_OK;
  gelu_fwd_kernel<<<ew_grid(n / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x,
                                                                   (__nv_bfloat16*)y, n / 8);
  return (int)cudaGetLastError();
}
BB_API int bb_gelu_bwd(const void* dy, const void* x, void* dx, long n, void* stream) {
  if (n % 8) return BB_EARG;
  if (n <= 0) return BB_OK;
  gelu_bwd_kernel<<<ew_grid(n / 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (__nv_bfloat16*)dx, n / 8);
  return (int)cudaGetLastError();
}
BB_API int bb_add(const void* a, const void* b, void* y, long n, void* stream) {
  if (n % 8) return BB_EARG;
  if (n <= 0) return BB_OK;
  add_kernel<<<ew_grid(n / 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n / 8);
  return (int)cudaGetLastError();
}
BB_API int bb_embed_fwd(const int* tok, const void* emb, const void* pos_emb, int T, void* out,
                        long n_tok, int d, int vocab, void* stream) {
  if (d % 8) return BB_EARG;
  if (n_tok <= 0) return BB_OK;
  embed_fwd_kernel<<<ew_grid(n_tok * (d / 8)), 256, 0, (cudaStream_t)stream>>>(
      tok, (const __nv_bfloat16*)emb, (const __nv_bfloat16*)pos_emb, T, (__nv_bfloat16*)out, n_tok,
      d / 8, vocab BB_ERR_ARG);
  return (int)cudaGetLastError();
}
BB_API int bb_embed_bwd(const int* tok, const void* dout, float* demb, float* dpos, int T,
                        long n_tok, int d, int vocab, void* stream) {
  if (d % 2) return BB_EARG;
  if (n_tok <= 0) return BB_OK;
  embed_bwd_kernel<<<ew_grid(n_tok * (d / 2)), 256, 0, (cudaStream_t)stream>>>(
      tok, (const __nv_bfloat16*)dout, demb, dpos, T, n_tok, d, vocab BB_ERR_ARG);
  return (int)cudaGetLastError();
}
BB_API int bb_cast_f32_bf16(const float* x, void* y, long n, void* stream) {
  if (n <= 0) return BB_OK;
  cast_f32_bf16_kernel<<<ew_grid(n), 256, 0, (cudaStream_t)stream>>>(x, (__nv_bfloat16*)y, n);
  return (int)cudaGetLastError();
}
