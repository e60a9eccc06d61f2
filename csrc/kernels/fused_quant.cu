// Producer kernels of the W8A8 serving path that emit int8 rows + per-row scales directly, so the
// activation never makes a bf16 round trip through memory before its GEMM:
//   rmsnorm_q8   q, s = quant_rows(RMSNorm(x [+ res]) * w)      (also writes the residual sum)
//   swiglu_q8    q, s = quant_rows(silu(gate) * up)
// Both keep one row per warp in registers (bf16-rounded, exactly what the unfused pair stores), take
// the row maximum with a warp reduction and quantise from registers: results are bit-identical to
// rmsnorm_fwd / swiglu_fwd followed by quant_rows.  Rows wider than the register budget are refused
// (BB_ESIZE) and the caller runs the two kernels separately.
// Contracts: crates/kernels/wgsl/{rmsnorm_rows,swiglu,max_abs_row,quant_pack}.wgsl of the reference
// (crates/model/src/int8.rs:221-235 quant_rows_steps).
#include "../common/host.hpp"
#include "../common/ptx.cuh"
#include "../common/vec.cuh"

namespace bb {

__device__ __forceinline__ uint2 quant8(const float (&f)[8], float inv) {
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float r = fminf(127.f, fmaxf(-127.f, rintf(f[j] * inv)));
    w[j >> 2] |= ((uint32_t)(int)r & 0xffu) << (8 * (j & 3));
  }
  return make_uint2(w[0], w[1]);
}

// One warp per row; MAXV 16-byte vectors per lane (d <= 256 * MAXV).
template <int MAXV>
__global__ void rmsnorm_q8_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                  const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h_out,
                                  int8_t* __restrict__ q, float* __restrict__ scale, int rows, int d,
                                  float eps) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nv = d >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)row * d);
  const bf16x8* rr = res ? reinterpret_cast<const bf16x8*>(res + (size_t)row * d) : nullptr;
  bf16x8* hr = h_out ? reinterpret_cast<bf16x8*>(h_out + (size_t)row * d) : nullptr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  // every load of the row is issued before the first use (a load inside the compute loop waits
  // for the previous iteration's store to the residual stream and serialises the row)
  bf16x8 hv[MAXV], rv[MAXV], wv[MAXV];
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      hv[t] = xr[i];
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
      unpack8(hv[t], f);
      if (rr) {
        float g[8];
        unpack8(rv[t], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
        hv[t] = pack8(f);      // the residual stream value: normalise exactly what is stored
        hr[i] = hv[t];
        unpack8(hv[t], f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)d + eps);
  float mx = 0.f;
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      float f[8], g[8];
      unpack8(hv[t], f);
      unpack8(wv[t], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
      hv[t] = pack8(f);          // the bf16 value the unfused norm would have stored
      unpack8(hv[t], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(f[j]));
    }
  }
  mx = warp_max(mx);
  const float s = fmaxf(mx / 127.f, 1e-8f);
  if (lane == 0) scale[row] = s;
  const float inv = 1.f / s;
  uint2* qr = reinterpret_cast<uint2*>(q + (size_t)row * d);
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      float f[8];
      unpack8(hv[t], f);
      qr[i] = quant8(f, inv);
    }
  }
}

// gu: [rows, 2*ff] (gate | up); one warp per row; MAXV vectors per lane (ff <= 256 * MAXV).
template <int MAXV>
__global__ void swiglu_q8_kernel(const __nv_bfloat16* __restrict__ gu, int8_t* __restrict__ q,
                                 float* __restrict__ scale, int rows, int ff) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nv = ff >> 3;
  const bf16x8* gr = reinterpret_cast<const bf16x8*>(gu + (size_t)row * 2 * ff);
  bf16x8 hv[MAXV], uv[MAXV];
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      hv[t] = gr[i];
      uv[t] = gr[nv + i];
    }
  }
  float mx = 0.f;
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      float g[8], u[8], o[8];
      unpack8(hv[t], g);
      unpack8(uv[t], u);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
      hv[t] = pack8(o);
      unpack8(hv[t], o);
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(o[j]));
    }
  }
  mx = warp_max(mx);
  const float s = fmaxf(mx / 127.f, 1e-8f);
  if (lane == 0) scale[row] = s;
  const float inv = 1.f / s;
  uint2* qr = reinterpret_cast<uint2*>(q + (size_t)row * ff);
#pragma unroll
  for (int t = 0; t < MAXV; ++t) {
    const int i = lane + 32 * t;
    if (i < nv) {
      float f[8];
      unpack8(hv[t], f);
      qr[i] = quant8(f, inv);
    }
  }
}

}  // namespace bb

using namespace bb;

// q[rows, d] int8, scale[rows] = quant_rows(RMSNorm(x [+ res]) * w); h_out (required when res is
// given) receives x + res.  d % 8 == 0, d <= 4096 (BB_ESIZE beyond).
BB_API int bb_rmsnorm_q8(const void* x, const void* res, const void* w, void* h_out, void* q,
                         float* scale, int rows, int d, float eps, void* stream) {
  if (rows <= 0) return BB_OK;
  if (d % 8 || (res && !h_out)) return BB_EARG;
  const int grid = (rows + 7) / 8;
  cudaStream_t s = (cudaStream_t)stream;
#define BB_RQ(MAXV_)                                                                              \
  rmsnorm_q8_kernel<MAXV_><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, \
                                                (const __nv_bfloat16*)w, (__nv_bfloat16*)h_out,   \
                                                (int8_t*)q, scale, rows, d, eps)
  if (d <= 256 * 4) BB_RQ(4);
  else if (d <= 256 * 8) BB_RQ(8);
  else if (d <= 256 * 16) BB_RQ(16);
  else return BB_ESIZE;   // wider rows do not fit the register file: run the norm and the quant apart
#undef BB_RQ
  return (int)cudaGetLastError();
}

namespace bb {
// 4-bit weight storage -> int8 operand of the kind::i8 GEMM (W4A8): every 32-bit word holds eight
// two's-complement nibbles, element b of the group in bits 4b..4b+3.  One thread expands one word
// into eight int8 values (one 8-byte store), so a layer's weights live in HBM at half a byte per
// parameter and are expanded into a scratch buffer right before the GEMM that consumes them.
// Reference: crates/model/src/int4.rs:46-73 (storage format), crates/kernels/wgsl/matmul_q4_dyn.wgsl.
__global__ void unpack_q4_kernel(const int* __restrict__ words, int2* __restrict__ out, long n_words) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_words) return;
  const int w = __ldg(words + i);
  int lo = 0, hi = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int v0 = (w << (28 - 4 * b)) >> 28;        // sign-extended nibble b
    const int v1 = (w << (12 - 4 * b)) >> 28;        // nibble b + 4
    lo |= (v0 & 0xFF) << (8 * b);
    hi |= (v1 & 0xFF) << (8 * b);
  }
  out[i] = make_int2(lo, hi);
}

}  // namespace bb

// out[8 * n_words] int8 = the sign-extended nibbles of words[n_words]; out must be 8-byte aligned.
BB_API int bb_unpack_q4(const void* words, void* out, long n_words, void* stream) {
  if (n_words <= 0) return bb::BB_OK;
  if (reinterpret_cast<uintptr_t>(out) & 7) return bb::BB_EARG;
  const long blocks = (n_words + 255) / 256;
  bb::unpack_q4_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const int*)words, (int2*)out, n_words);
  return (int)cudaGetLastError();
}

// q[rows, ff] int8, scale[rows] = quant_rows(silu(gu[:, :ff]) * gu[:, ff:]).  ff % 8 == 0, ff <= 4096 (BB_ESIZE beyond).
BB_API int bb_swiglu_q8(const void* gu, void* q, float* scale, int rows, int ff, void* stream) {
  if (rows <= 0) return BB_OK;
  if (ff % 8) return BB_EARG;
  const int grid = (rows + 7) / 8;
  cudaStream_t s = (cudaStream_t)stream;
#define BB_SQ(MAXV_) \
  swiglu_q8_kernel<MAXV_><<<grid, 256, 0, s>>>((const __nv_bfloat16*)gu, (int8_t*)q, scale, rows, ff)
  if (ff <= 256 * 4) BB_SQ(4);
  else if (ff <= 256 * 8) BB_SQ(8);
  else if (ff <= 256 * 16) BB_SQ(16);
  else return BB_ESIZE;
#undef BB_SQ
  return (int)cudaGetLastError();
}
