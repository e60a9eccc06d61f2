// Fused per-head RMSNorm (Qwen3 "QK-norm") + half-split (NeoX) rotary embedding, forward and
// backward.  One warp per (token, head).  Head dim 64 or 128.
//   xn  = x * rsqrt(mean(x^2)+eps) * w          (skipped when w == null: plain RoPE)
//   out[m]      = xn[m]*cos - xn[m+hd/2]*sin
//   out[m+hd/2] = xn[m+hd/2]*cos + xn[m]*sin    angle = pos * theta^(-2m/hd)
// cos/sin come from a precomputed fp32 table [max_pos][hd/2].
// Reference contracts: crates/kernels/wgsl/{rmsnorm_rows,rope_base,rope_base_bwd,rope_paged}.wgsl.
#include "../common/host.hpp"
#include "../common/ptx.cuh"

#include <type_traits>

namespace bb {

// One warp per TOKEN (grid-stride): position, cos and sin are fetched once per token and reused
// for all of its heads; heads are processed ROPE_UNR at a time (8: 44 / 75 us forward / backward on
// 16384 tokens x 24 heads x 128 against 48 / 81 us with 4) with every load of the group issued
// before the first dependent instruction.  No integer division anywhere on the hot path (an
// earlier (token, head)-per-warp form spent more instructions on 64-bit div/mod than on the math).
static constexpr int ROPE_UNR = 8;

template <int HD>
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                       const __nv_bfloat16* __restrict__ w_q, const __nv_bfloat16* __restrict__ w_k,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                       const int* __restrict__ pos, __nv_bfloat16* __restrict__ out, int ldo,
                       float* __restrict__ rstd_out, int n_tok, int hq, int hk, float eps) {
  constexpr int HALF = HD / 2;
  constexpr int PER = HALF / 32;  // elements per lane per half: 1 (hd 64) or 2 (hd 128)
  constexpr int U = ROPE_UNR;
  using Vec = typename std::conditional<PER == 2, __nv_bfloat162, __nv_bfloat16>::type;
  const int heads = hq + hk;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const bool norm = w_q != nullptr;
  float wqa[PER], wqb[PER], wka[PER], wkb[PER];
  if (norm) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      wqa[j] = __bfloat162float(w_q[lane * PER + j]);
      wqb[j] = __bfloat162float(w_q[HALF + lane * PER + j]);
      wka[j] = __bfloat162float(w_k[lane * PER + j]);
      wkb[j] = __bfloat162float(w_k[HALF + lane * PER + j]);
    }
  }
  auto unpack = [](const Vec v, float (&o)[PER]) {
    if constexpr (PER == 2) { o[0] = __low2float(v); o[1] = __high2float(v); }
    else { o[0] = __bfloat162float(v); }
  };
  for (int tok = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; tok < n_tok; tok += nwarps) {
    const int p = pos[tok];
    float c[PER], sn[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      c[j] = cos_t[(size_t)p * HALF + lane * PER + j];
      sn[j] = sin_t[(size_t)p * HALF + lane * PER + j];
    }
    const __nv_bfloat16* xt = x + (size_t)tok * ldx;
    __nv_bfloat16* ot = out + (size_t)tok * ldo;
    for (int h0 = 0; h0 < heads; h0 += U) {
      float a[U][PER], b[U][PER];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = min(h0 + u, heads - 1);
        unpack(*reinterpret_cast<const Vec*>(xt + h * HD + lane * PER), a[u]);
        unpack(*reinterpret_cast<const Vec*>(xt + h * HD + HALF + lane * PER), b[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = h0 + u;
        if (norm) {
          float ss = 0.f;
#pragma unroll
          for (int j = 0; j < PER; ++j) ss += a[u][j] * a[u][j] + b[u][j] * b[u][j];
          ss = warp_sum(ss);
          const float rstd = rsqrtf(ss / (float)HD + eps);
          if (lane == 0 && rstd_out && h < heads) rstd_out[(size_t)tok * heads + h] = rstd;
          const bool is_q = h < hq;
#pragma unroll
          for (int j = 0; j < PER; ++j) {
            a[u][j] *= rstd * (is_q ? wqa[j] : wka[j]);
            b[u][j] *= rstd * (is_q ? wqb[j] : wkb[j]);
          }
        }
        if (h >= heads) continue;
        float o0[PER], o1[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          o0[j] = a[u][j] * c[j] - b[u][j] * sn[j];
          o1[j] = b[u][j] * c[j] + a[u][j] * sn[j];
        }
        __nv_bfloat16* orow = ot + h * HD;
        if constexpr (PER == 2) {
          *reinterpret_cast<__nv_bfloat162*>(orow + lane * 2) = __floats2bfloat162_rn(o0[0], o0[1]);
          *reinterpret_cast<__nv_bfloat162*>(orow + HALF + lane * 2) = __floats2bfloat162_rn(o1[0], o1[1]);
        } else {
          orow[lane] = __float2bfloat16(o0[0]);
          orow[HALF + lane] = __float2bfloat16(o1[0]);
        }
      }
    }
  }
}

// Backward: given d(out), produce d(x) and accumulate d(w_q), d(w_k) (fp32, [HD] each).  The gain
// gradient is reduced in registers over the warp's tokens, then across the block in shared memory,
// and reaches global memory with one atomic per element per block.
template <int HD>
__global__ void __launch_bounds__(256)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout, int ldo,
                       const __nv_bfloat16* __restrict__ x, int ldx,
                       const __nv_bfloat16* __restrict__ w_q, const __nv_bfloat16* __restrict__ w_k,
                       const float* __restrict__ rstd_in, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, const int* __restrict__ pos,
                       __nv_bfloat16* __restrict__ dx, int ldd, float* __restrict__ dw_q,
                       float* __restrict__ dw_k, int n_tok, int hq, int hk) {
  constexpr int HALF = HD / 2;
  constexpr int PER = HALF / 32;
  constexpr int U = ROPE_UNR;
  using Vec = typename std::conditional<PER == 2, __nv_bfloat162, __nv_bfloat16>::type;
  const int heads = hq + hk;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const bool norm = w_q != nullptr;
  float gq_a[PER] = {0}, gq_b[PER] = {0}, gk_a[PER] = {0}, gk_b[PER] = {0};
  float wqa[PER], wqb[PER], wka[PER], wkb[PER];
  if (norm) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      wqa[j] = __bfloat162float(w_q[lane * PER + j]);
      wqb[j] = __bfloat162float(w_q[HALF + lane * PER + j]);
      wka[j] = __bfloat162float(w_k[lane * PER + j]);
      wkb[j] = __bfloat162float(w_k[HALF + lane * PER + j]);
    }
  }
  auto unpack = [](const Vec v, float (&o)[PER]) {
    if constexpr (PER == 2) { o[0] = __low2float(v); o[1] = __high2float(v); }
    else { o[0] = __bfloat162float(v); }
  };
  for (int tok = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; tok < n_tok; tok += nwarps) {
    const int p = pos[tok];
    float c[PER], sn[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      c[j] = cos_t[(size_t)p * HALF + lane * PER + j];
      sn[j] = sin_t[(size_t)p * HALF + lane * PER + j];
    }
    const __nv_bfloat16* dot_ = dout + (size_t)tok * ldo;
    const __nv_bfloat16* xt = x + (size_t)tok * ldx;
    __nv_bfloat16* dxt = dx + (size_t)tok * ldd;
    for (int h0 = 0; h0 < heads; h0 += U) {
      float g0[U][PER], g1[U][PER], xa[U][PER], xb[U][PER], rstd[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = min(h0 + u, heads - 1);
        unpack(*reinterpret_cast<const Vec*>(dot_ + h * HD + lane * PER), g0[u]);
        unpack(*reinterpret_cast<const Vec*>(dot_ + h * HD + HALF + lane * PER), g1[u]);
        if (norm) {
          unpack(*reinterpret_cast<const Vec*>(xt + h * HD + lane * PER), xa[u]);
          unpack(*reinterpret_cast<const Vec*>(xt + h * HD + HALF + lane * PER), xb[u]);
          rstd[u] = rstd_in[(size_t)tok * heads + h];
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = h0 + u;
        const bool live = h < heads;
        float da[PER], db[PER], ra[PER], rb[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          da[j] = g0[u][j] * c[j] + g1[u][j] * sn[j];   // d xn[m]
          db[j] = g1[u][j] * c[j] - g0[u][j] * sn[j];   // d xn[m+half]
        }
        if (!norm) {
#pragma unroll
          for (int j = 0; j < PER; ++j) { ra[j] = da[j]; rb[j] = db[j]; }
        } else {
          const bool is_q = h < hq;
          float dot = 0.f;
          float wa[PER], wb[PER];
#pragma unroll
          for (int j = 0; j < PER; ++j) {
            xa[u][j] *= rstd[u];
            xb[u][j] *= rstd[u];
            wa[j] = is_q ? wqa[j] : wka[j];
            wb[j] = is_q ? wqb[j] : wkb[j];
            const float pa = live ? da[j] * xa[u][j] : 0.f, pb = live ? db[j] * xb[u][j] : 0.f;
            if (is_q) { gq_a[j] += pa; gq_b[j] += pb; }
            else { gk_a[j] += pa; gk_b[j] += pb; }
            dot += da[j] * wa[j] * xa[u][j] + db[j] * wb[j] * xb[u][j];
          }
          dot = warp_sum(dot) / (float)HD;
#pragma unroll
          for (int j = 0; j < PER; ++j) {
            ra[j] = rstd[u] * (da[j] * wa[j] - xa[u][j] * dot);
            rb[j] = rstd[u] * (db[j] * wb[j] - xb[u][j] * dot);
          }
        }
        if (!live) continue;
        __nv_bfloat16* dxr = dxt + h * HD;
        if constexpr (PER == 2) {
          *reinterpret_cast<__nv_bfloat162*>(dxr + lane * 2) = __floats2bfloat162_rn(ra[0], ra[1]);
          *reinterpret_cast<__nv_bfloat162*>(dxr + HALF + lane * 2) = __floats2bfloat162_rn(rb[0], rb[1]);
        } else {
          dxr[lane] = __float2bfloat16(ra[0]);
          dxr[HALF + lane] = __float2bfloat16(rb[0]);
        }
      }
    }
  }
  if (!norm) return;
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
    const int which = i / HD, cc = i % HD;
    float sum = 0.f;
    for (int w2 = 0; w2 < nw; ++w2) sum += red[which][w2][cc];
    if (which == 0) {
      if (dw_q) atomicAdd(dw_q + cc, sum);
    } else {
      if (dw_k && hk > 0) atomicAdd(dw_k + cc, sum);
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
  long want = ((long)n_tok + 7) / 8;
  const long cap = (long)sm_count() * 8;
  const int grid = (int)(want < cap ? want : cap);
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
  long want = ((long)n_tok + 7) / 8;
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
