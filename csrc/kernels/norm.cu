// Row-normalisation kernels (warp per row, 16-byte vector accesses, fp32 math, bf16 storage):
//   RMSNorm fwd (optionally fused with a residual add) / bwd-dx, LayerNorm fwd / bwd-dx,
//   and the column reductions that produce gain / bias gradients.
// Contracts follow crates/kernels/wgsl/{rmsnorm_rows,rmsnorm_dx,rmsnorm_dw,layernorm_rows,
// layernorm_dx_rows,layernorm_dgamma,layernorm_dbeta,bias_grad}.wgsl of the reference.
#include "../common/host.hpp"
#include "../common/ptx.cuh"
#include "../common/vec.cuh"

namespace bb {


// y = w * (x [+ res]) * rstd ; optionally writes h = x + res (the new residual stream).
// d must be a multiple of 8.  One warp per row.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out,
                                   int rows, int d, float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const int nv = d >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)warp * d);
  const bf16x8* rr = res ? reinterpret_cast<const bf16x8*>(res + (size_t)warp * d) : nullptr;
  bf16x8* hr = h_out ? reinterpret_cast<bf16x8*>(h_out + (size_t)warp * d) : nullptr;
  float ss = 0.f;
  for (int i = lane; i < nv; i += 32) {
    float f[8];
    unpack8(xr[i], f);
    if (rr) {
      float g[8];
      unpack8(rr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      if (hr) {
        bf16x8 hp = pack8(f);
        hr[i] = hp;
        unpack8(hp, f);  // normalise exactly what the residual stream stores
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)d + eps);
  if (lane == 0 && rstd_out) rstd_out[warp] = rstd;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + (size_t)warp * d);
  const bf16x8* src = (rr && hr) ? reinterpret_cast<const bf16x8*>(hr) : xr;
  for (int i = lane; i < nv; i += 32) {
    float f[8], g[8];
    unpack8(src[i], f);
    if (rr && !hr) {
      unpack8(rr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
    }
    unpack8(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
    yr[i] = pack8(f);
  }
}

// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) [+ dres]  with xhat = x*rstd.
__global__ void rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy,
                                      const __nv_bfloat16* __restrict__ x,
                                      const __nv_bfloat16* __restrict__ w,
                                      const float* __restrict__ rstd_in,
                                      const __nv_bfloat16* __restrict__ dres,
                                      __nv_bfloat16* __restrict__ dx, int rows, int d) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const int nv = d >> 3;
  const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + (size_t)warp * d);
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)warp * d);
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  const float rstd = rstd_in[warp];
  float dot = 0.f;
  for (int i = lane; i < nv; i += 32) {
    float a[8], b[8], c[8];
    unpack8(dyr[i], a);
    unpack8(xr[i], b);
    unpack8(wr[i], c);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += a[j] * c[j] * b[j] * rstd;
  }
  dot = warp_sum(dot) / (float)d;
  const bf16x8* rr = dres ? reinterpret_cast<const bf16x8*>(dres + (size_t)warp * d) : nullptr;
  bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + (size_t)warp * d);
  for (int i = lane; i < nv; i += 32) {
    float a[8], b[8], c[8], o[8];
    unpack8(dyr[i], a);
    unpack8(xr[i], b);
    unpack8(wr[i], c);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = rstd * (a[j] * c[j] - b[j] * rstd * dot);
    if (rr) {
      float r[8];
      unpack8(rr[i], r);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] += r[j];
    }
    dxr[i] = pack8(o);
  }
}

// Register-resident forms (d <= 256 * MAXV): every load of the row is issued before the first
// use, the row is read from memory once, and the second pass runs out of registers.  The looped
// kernels above keep one 16-byte load per lane in flight and re-read the row; they measured
// 0.53-0.58 of the copy bandwidth.  Arithmetic and rounding are identical.
template <int MAXV>
__global__ void rmsnorm_fwd_reg_kernel(const __nv_bfloat16* __restrict__ x,
                                       const __nv_bfloat16* __restrict__ res,
                                       const __nv_bfloat16* __restrict__ w,
                                       __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
                                       float* __restrict__ rstd_out, int rows, int d, float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const int nv = d >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)warp * d);
  const bf16x8* rr = res ? reinterpret_cast<const bf16x8*>(res + (size_t)warp * d) : nullptr;
  bf16x8* hr = h_out ? reinterpret_cast<bf16x8*>(h_out + (size_t)warp * d) : nullptr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8 xv[MAXV], rv[MAXV], wv[MAXV];
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      xv[t] = xr[i];
      if (rr) rv[t] = rr[i];
      wv[t] = wr[i];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      float f[8];
      unpack8(xv[t], f);
      if (rr) {
        float g[8];
        unpack8(rv[t], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
        xv[t] = pack8(f);      // the residual stream value (callers of this form always store it)
        hr[i] = xv[t];
        unpack8(xv[t], f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)d + eps);
  if (lane == 0 && rstd_out) rstd_out[warp] = rstd;
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + (size_t)warp * d);
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      float f[8], g[8];
      unpack8(xv[t], f);
      unpack8(wv[t], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
      yr[i] = pack8(f);
    }
  }
}

template <int MAXV>
__global__ void rmsnorm_bwd_dx_reg_kernel(const __nv_bfloat16* __restrict__ dy,
                                          const __nv_bfloat16* __restrict__ x,
                                          const __nv_bfloat16* __restrict__ w,
                                          const float* __restrict__ rstd_in,
                                          const __nv_bfloat16* __restrict__ dres,
                                          __nv_bfloat16* __restrict__ dx, int rows, int d) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const int nv = d >> 3;
  const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + (size_t)warp * d);
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)warp * d);
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  const bf16x8* rr = dres ? reinterpret_cast<const bf16x8*>(dres + (size_t)warp * d) : nullptr;
  bf16x8 av[MAXV], bv[MAXV], cv[MAXV], rv[MAXV];
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      av[t] = dyr[i];
      bv[t] = xr[i];
      cv[t] = wr[i];
      if (rr) rv[t] = rr[i];
    }
  }
  const float rstd = rstd_in[warp];
  float dot = 0.f;
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      float a[8], b[8], c[8];
      unpack8(av[t], a);
      unpack8(bv[t], b);
      unpack8(cv[t], c);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += a[j] * c[j] * b[j] * rstd;
    }
  }
  dot = warp_sum(dot) / (float)d;
  bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + (size_t)warp * d);
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      float a[8], b[8], c[8], o[8];
      unpack8(av[t], a);
      unpack8(bv[t], b);
      unpack8(cv[t], c);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * (a[j] * c[j] - b[j] * rstd * dot);
      if (rr) {
        float r[8];
        unpack8(rv[t], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      dxr[i] = pack8(o);
    }
  }
}

// LayerNorm forward: y = (x-mean)*rstd*g + b ; saves mean and rstd.
__global__ void layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                     const __nv_bfloat16* __restrict__ g,
                                     const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                     float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                     int rows, int d, float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const int nv = d >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)warp * d);
  float s = 0.f;
  for (int i = lane; i < nv; i += 32) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j];
  }
  const float mean = warp_sum(s) / (float)d;
  float ss = 0.f;
  for (int i = lane; i < nv; i += 32) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += (f[j] - mean) * (f[j] - mean);
  }
  const float rstd = rsqrtf(warp_sum(ss) / (float)d + eps);
  if (lane == 0) {
    if (mean_out) mean_out[warp] = mean;
    if (rstd_out) rstd_out[warp] = rstd;
  }
  const bf16x8* gr = reinterpret_cast<const bf16x8*>(g);
  const bf16x8* br = reinterpret_cast<const bf16x8*>(b);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + (size_t)warp * d);
  for (int i = lane; i < nv; i += 32) {
    float f[8], gg[8], bb_[8];
    unpack8(xr[i], f);
    unpack8(gr[i], gg);
    unpack8(br[i], bb_);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * rstd * gg[j] + bb_[j];
    yr[i] = pack8(f);
  }
}

// LayerNorm backward wrt x: dx = rstd*(g*dy - mean(g*dy) - xhat*mean(g*dy*xhat)) [+ dres].
__global__ void layernorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy,
                                        const __nv_bfloat16* __restrict__ x,
                                        const __nv_bfloat16* __restrict__ g,
                                        const float* __restrict__ mean_in,
                                        const float* __restrict__ rstd_in,
                                        const __nv_bfloat16* __restrict__ dres,
                                        __nv_bfloat16* __restrict__ dx, int rows, int d) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const int nv = d >> 3;
  const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + (size_t)warp * d);
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)warp * d);
  const bf16x8* gr = reinterpret_cast<const bf16x8*>(g);
  const float mean = mean_in[warp], rstd = rstd_in[warp];
  float s1 = 0.f, s2 = 0.f;
  for (int i = lane; i < nv; i += 32) {
    float a[8], b[8], c[8];
    unpack8(dyr[i], a);
    unpack8(xr[i], b);
    unpack8(gr[i], c);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gd = a[j] * c[j];
      s1 += gd;
      s2 += gd * (b[j] - mean) * rstd;
    }
  }
  s1 = warp_sum(s1) / (float)d;
  s2 = warp_sum(s2) / (float)d;
  const bf16x8* rr = dres ? reinterpret_cast<const bf16x8*>(dres + (size_t)warp * d) : nullptr;
  bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + (size_t)warp * d);
  for (int i = lane; i < nv; i += 32) {
    float a[8], b[8], c[8], o[8];
    unpack8(dyr[i], a);
    unpack8(xr[i], b);
    unpack8(gr[i], c);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      o[j] = rstd * (a[j] * c[j] - s1 - (b[j] - mean) * rstd * s2);
    if (rr) {
      float r[8];
      unpack8(rr[i], r);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] += r[j];
    }
    dxr[i] = pack8(o);
  }
}

// Column reduction: out[c] += sum_r dy[r,c] * f(x[r,c]) where
//   mode 0: f = 1                       (bias / beta gradient)
//   mode 1: f = x * rstd[r]             (RMSNorm gain gradient)
//   mode 2: f = (x - mean[r]) * rstd[r] (LayerNorm gamma gradient)
// Each block owns 64 columns and a slice of rows; partial sums are added to fp32 `out` with one
// atomic per (block, column).  blockDim = 256 (8 warps x 32 lanes x 2 columns).
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                              const float* __restrict__ mean, const float* __restrict__ rstd,
                              float* __restrict__ out, int rows, int d, int ld, int mode,
                              int rows_per_block) {
  __shared__ float2 part[8][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 64 + lane * 2;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float2 acc = make_float2(0.f, 0.f);
  if (c < d) {
    for (int r = r0 + warp; r < r1; r += 8) {
      const float2 g = __bfloat1622float2(
          *reinterpret_cast<const __nv_bfloat162*>(dy + (size_t)r * ld + c));
      if (mode == 0) {
        acc.x += g.x;
        acc.y += g.y;
      } else {
        float2 xv = __bfloat1622float2(
            *reinterpret_cast<const __nv_bfloat162*>(x + (size_t)r * ld + c));
        const float rs = rstd[r];
        if (mode == 2) {
          const float m = mean[r];
          xv.x -= m;
          xv.y -= m;
        }
        acc.x += g.x * xv.x * rs;
        acc.y += g.y * xv.y * rs;
      }
    }
  }
  part[warp][lane] = acc;
  __syncthreads();
  if (warp == 0 && c < d) {
    float2 s = part[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) {
      s.x += part[w][lane].x;
      s.y += part[w][lane].y;
    }
    atomicAdd(out + c, s.x);
    if (c + 1 < d) atomicAdd(out + c + 1, s.y);
  }
}

}  // namespace bb

using namespace bb;

static inline int warp_rows_grid(int rows, int threads) {
  const int rows_per_block = threads / 32;
  return (rows + rows_per_block - 1) / rows_per_block;
}

BB_API int bb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out,
                          float* rstd, int rows, int d, float eps, void* stream) {
  if (rows <= 0) return BB_OK;
  if (d % 8) return BB_EARG;
  const int grid = warp_rows_grid(rows, 256);
  cudaStream_t s = (cudaStream_t)stream;
#define BB_RF(MAXV_)                                                                              \
  rmsnorm_fwd_reg_kernel<MAXV_><<<grid, 256, 0, s>>>(                                             \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,                \
      (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, rows, d, eps)
  if (res && !h_out) {   // sum not stored: the looped kernel normalises the unrounded fp32 sum
    rmsnorm_fwd_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res,
                                            (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
                                            (__nv_bfloat16*)h_out, rstd, rows, d, eps);
  } else if (d <= 256 * 2) {
    BB_RF(2);
  } else if (d <= 256 * 4) {
    BB_RF(4);
  } else if (d <= 256 * 8) {
    BB_RF(8);
  } else if (d <= 256 * 16) {
    BB_RF(16);
  } else {
    rmsnorm_fwd_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res,
                                            (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
                                            (__nv_bfloat16*)h_out, rstd, rows, d, eps);
  }
#undef BB_RF
  return (int)cudaGetLastError();
}

BB_API int bb_rmsnorm_bwd_dx(const void* dy, const void* x, const void* w, const float* rstd,
                             const void* dres, void* dx, int rows, int d, void* stream) {
  if (rows <= 0) return BB_OK;
  if (d % 8) return BB_EARG;
  const int grid = warp_rows_grid(rows, 256);
  cudaStream_t s = (cudaStream_t)stream;
#define BB_RB(MAXV_)                                                                              \
  rmsnorm_bwd_dx_reg_kernel<MAXV_><<<grid, 256, 0, s>>>(                                          \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,           \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, rows, d)
  if (d <= 256 * 2) {
    BB_RB(2);
  } else if (d <= 256 * 4) {
    BB_RB(4);
  } else if (d <= 256 * 8) {
    BB_RB(8);
  } else {
    rmsnorm_bwd_dx_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                               (const __nv_bfloat16*)w, rstd,
                                               (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, rows, d);
  }
#undef BB_RB
  return (int)cudaGetLastError();
}

BB_API int bb_layernorm_fwd(const void* x, const void* g, const void* b, void* y, float* mean,
                            float* rstd, int rows, int d, float eps, void* stream) {
  if (rows <= 0) return BB_OK;
  if (d % 8) return BB_EARG;
  layernorm_fwd_kernel<<<warp_rows_grid(rows, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, (const __nv_bfloat16*)b,
      (__nv_bfloat16*)y, mean, rstd, rows, d, eps);
  return (int)cudaGetLastError();
}

BB_API int bb_layernorm_bwd_dx(const void* dy, const void* x, const void* g, const float* mean,
                               const float* rstd, const void* dres, void* dx, int rows, int d,
                               void* stream) {
  if (rows <= 0) return BB_OK;
  if (d % 8) return BB_EARG;
  layernorm_bwd_dx_kernel<<<warp_rows_grid(rows, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, mean, rstd,
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, rows, d);
  return (int)cudaGetLastError();
}

// out (fp32, [d]) += column sums; see colsum_kernel for `mode`.  ld = row pitch in elements.
BB_API int bb_colsum(const void* dy, const void* x, const float* mean, const float* rstd,
                     float* out, int rows, int d, int ld, int mode, void* stream) {
  if (rows <= 0) return BB_OK;
  if ((d % 2) || (ld % 2)) return BB_EARG;
  const int col_blocks = (d + 63) / 64;
  int row_blocks = (4 * sm_count() + col_blocks - 1) / col_blocks;
  if (row_blocks < 1) row_blocks = 1;
  int rpb = (rows + row_blocks - 1) / row_blocks;
  if (rpb < 64) rpb = 64;
  row_blocks = (rows + rpb - 1) / rpb;
  dim3 grid(col_blocks, row_blocks);
  colsum_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy,
                                                         (const __nv_bfloat16*)x, mean, rstd, out,
                                                         rows, d, ld, mode, rpb);
  return (int)cudaGetLastError();
}
