// Fused per-head RMSNorm (Qwen3 "QK-norm") + half-split (NeoX) rotary embedding, forward and
// backward.  One warp per (token, head).  Head dim 64 or 128.
//   xn  = x * rsqrt(mean(x^2)+eps) * w          (skipped when w == null: plain RoPE)
//   out[m]      = xn[m]*cos - xn[m+hd/2]*sin
//   out[m+hd/2] = xn[m+hd/2]*cos + xn[m]*sin    angle = pos * theta^(-2m/hd)
// cos/sin come from a precomputed fp32 table [max_pos][hd/2].
// Reference contracts: crates/kernels/wgsl/{rmsnorm_rows,rope_base,rope_base_bwd,rope_paged}.wgsl.
#include "../common/host.hpp"
#include "../common/ptx.cuh"

namespace bb {

template <int HD>
__global__ void qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                       const __nv_bfloat16* __restrict__ w_q,
                                       const __nv_bfloat16* __restrict__ w_k,
                                       const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t,
                                       const int* __restrict__ pos, __nv_bfloat16* __restrict__ out,
                                       int ldo, float* __restrict__ rstd_out, int n_tok, int hq,
                                       int hk, float eps) {
  constexpr int HALF = HD / 2;
  constexpr int PER = HALF / 32;  // elements per lane per half: 1 (hd 64) or 2 (hd 128)
  const int heads = hq + hk;
  const long gw = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= (long)n_tok * heads) return;
  const int tok = (int)(gw / heads), head = (int)(gw % heads);
  const __nv_bfloat16* xr = x + (size_t)tok * ldx + head * HD;
  const __nv_bfloat16* w = head < hq ? w_q : w_k;
  float a[PER], b[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    a[j] = __bfloat162float(xr[lane * PER + j]);
    b[j] = __bfloat162float(xr[HALF + lane * PER + j]);
  }
  float rstd = 1.f;
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) ss += a[j] * a[j] + b[j] * b[j];
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)HD + eps);
    if (lane == 0 && rstd_out) rstd_out[gw] = rstd;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      a[j] *= rstd * __bfloat162float(w[lane * PER + j]);
      b[j] *= rstd * __bfloat162float(w[HALF + lane * PER + j]);
    }
  }
  const int p = pos[tok];
  __nv_bfloat16* orow = out + (size_t)tok * ldo + head * HD;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int m = lane * PER + j;
    const float c = cos_t[(size_t)p * HALF + m], s = sin_t[(size_t)p * HALF + m];
    orow[m] = __float2bfloat16(a[j] * c - b[j] * s);
    orow[HALF + m] = __float2bfloat16(b[j] * c + a[j] * s);
  }
}

// Backward: given d(out), produce d(x) and accumulate d(w_q), d(w_k) (fp32, [HD] each).
// Persistent grid-stride over (token, head) pairs so the gain gradient is reduced in registers and
// hits global memory with one atomic per lane per block-warp.
template <int HD>
__global__ void qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout, int ldo,
                                       const __nv_bfloat16* __restrict__ x, int ldx,
                                       const __nv_bfloat16* __restrict__ w_q,
                                       const __nv_bfloat16* __restrict__ w_k,
                                       const float* __restrict__ rstd_in,
                                       const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t,
                                       const int* __restrict__ pos, __nv_bfloat16* __restrict__ dx,
                                       int ldd, float* __restrict__ dw_q, float* __restrict__ dw_k,
                                       int n_tok, int hq, int hk) {
  constexpr int HALF = HD / 2;
  constexpr int PER = HALF / 32;
  const int heads = hq + hk;
  const int lane = threadIdx.x & 31;
  const long nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  const long total = (long)n_tok * heads;
  float gq_a[PER] = {0}, gq_b[PER] = {0}, gk_a[PER] = {0}, gk_b[PER] = {0};
  for (long gw = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; gw < total; gw += nwarps) {
    const int tok = (int)(gw / heads), head = (int)(gw % heads);
    const bool is_q = head < hq;
    const __nv_bfloat16* w = is_q ? w_q : w_k;
    const __nv_bfloat16* dor = dout + (size_t)tok * ldo + head * HD;
    const int p = pos[tok];
    float da[PER], db[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int m = lane * PER + j;
      const float c = cos_t[(size_t)p * HALF + m], s = sin_t[(size_t)p * HALF + m];
      const float g0 = __bfloat162float(dor[m]), g1 = __bfloat162float(dor[HALF + m]);
      da[j] = g0 * c + g1 * s;   // d xn[m]
      db[j] = g1 * c - g0 * s;   // d xn[m+half]
    }
    __nv_bfloat16* dxr = dx + (size_t)tok * ldd + head * HD;
    if (!w) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        dxr[lane * PER + j] = __float2bfloat16(da[j]);
        dxr[HALF + lane * PER + j] = __float2bfloat16(db[j]);
      }
      continue;
    }
    const __nv_bfloat16* xr = x + (size_t)tok * ldx + head * HD;
    const float rstd = rstd_in[gw];
    float xa[PER], xb[PER], wa[PER], wb[PER];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      xa[j] = __bfloat162float(xr[lane * PER + j]) * rstd;
      xb[j] = __bfloat162float(xr[HALF + lane * PER + j]) * rstd;
      wa[j] = __bfloat162float(w[lane * PER + j]);
      wb[j] = __bfloat162float(w[HALF + lane * PER + j]);
      if (is_q) {
        gq_a[j] += da[j] * xa[j];
        gq_b[j] += db[j] * xb[j];
      } else {
        gk_a[j] += da[j] * xa[j];
        gk_b[j] += db[j] * xb[j];
      }
      dot += da[j] * wa[j] * xa[j] + db[j] * wb[j] * xb[j];
    }
    dot = warp_sum(dot) / (float)HD;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      dxr[lane * PER + j] = __float2bfloat16(rstd * (da[j] * wa[j] - xa[j] * dot));
      dxr[HALF + lane * PER + j] = __float2bfloat16(rstd * (db[j] * wb[j] - xb[j] * dot));
    }
  }
  // block-level reduction in shared memory, then one atomic per element per block
  __shared__ float red[2][8][HD];
  const int wib = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    red[0][wib][lane * PER + j] = gq_a[j];
    red[0][wib][HALF + lane * PER + j] = gq_b[j];
    red[1][wib][lane * PER + j] = gk_a[j];
    red[1][wib][HALF + lane * PER + j] = gk_b[j];
  }
  __syncthreads();
  const int nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < 2 * HD; i += blockDim.x) {
    const int which = i / HD, c = i % HD;
    float sum = 0.f;
    for (int w2 = 0; w2 < nw; ++w2) sum += red[which][w2][c];
    if (which == 0) {
      if (w_q && dw_q) atomicAdd(dw_q + c, sum);
    } else {
      if (w_k && dw_k && hk > 0) atomicAdd(dw_k + c, sum);
    }
  }
}

}  // namespace bb

using namespace bb;

// x: [n_tok, ldx] holding hq+hk heads of `hd` (q heads first); out: [n_tok, ldo]; pos: int32[n_tok].
// w_q/w_k: bf16[hd] gains or null for plain RoPE; rstd: fp32[n_tok*(hq+hk)] saved for backward.
BB_API int bb_qknorm_rope_fwd(const void* x, int ldx, const void* w_q, const void* w_k,
                              const float* cos_t, const float* sin_t, const int* pos, void* out,
                              int ldo, float* rstd, int n_tok, int hq, int hk, int hd, float eps,
                              void* stream) {
  const long total = (long)n_tok * (hq + hk);
  if (total <= 0) return BB_OK;
  const int grid = (int)((total + 7) / 8);
  if (hd == 128)
    qknorm_rope_fwd_kernel<128><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w_q, (const __nv_bfloat16*)w_k, cos_t,
        sin_t, pos, (__nv_bfloat16*)out, ldo, rstd, n_tok, hq, hk, eps);
  else if (hd == 64)
    qknorm_rope_fwd_kernel<64><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w_q, (const __nv_bfloat16*)w_k, cos_t,
        sin_t, pos, (__nv_bfloat16*)out, ldo, rstd, n_tok, hq, hk, eps);
  else
    return BB_EARG;
  return (int)cudaGetLastError();
}

BB_API int bb_qknorm_rope_bwd(const void* dout, int ldo, const void* x, int ldx, const void* w_q,
                              const void* w_k, const float* rstd, const float* cos_t,
                              const float* sin_t, const int* pos, void* dx, int ldd, float* dw_q,
                              float* dw_k, int n_tok, int hq, int hk, int hd, void* stream) {
  const long total = (long)n_tok * (hq + hk);
  if (total <= 0) return BB_OK;
  long want = (total + 7) / 8;
  const long cap = (long)sm_count() * 4;
  const int grid = (int)(want < cap ? want : cap);
  if (hd == 128)
    qknorm_rope_bwd_kernel<128><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)dout, ldo, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w_q,
        (const __nv_bfloat16*)w_k, rstd, cos_t, sin_t, pos, (__nv_bfloat16*)dx, ldd, dw_q, dw_k,
        n_tok, hq, hk);
  else if (hd == 64)
    qknorm_rope_bwd_kernel<64><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)dout, ldo, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w_q,
        (const __nv_bfloat16*)w_k, rstd, cos_t, sin_t, pos, (__nv_bfloat16*)dx, ldd, dw_q, dw_k,
        n_tok, hq, hk);
  else
    return BB_EARG;
  return (int)cudaGetLastError();
}
