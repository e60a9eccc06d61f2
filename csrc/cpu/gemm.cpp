// CPU backend, native part: fp32 GEMM for the three products a linear layer needs, written for
// x86-64-v3 (AVX2 + FMA, which the build's -march guarantees), threaded over row panels.
//
//   bbh_cpu_gemm(ta, tb)   C[M,N] = alpha * op(A) * op(B) + beta * C
//                          op(A) = A[M,K] (ta = 0) or A[K,M]^T (ta = 1); op(B) = B[K,N] (tb = 0) or
//                          B[N,K]^T (tb = 1).  forward y = x W^T is (0,1); dX = dY W is (0,0);
//                          dW = dY^T X is (1,0).
//
// Method: both operands are packed into K-major panels (MR rows of A, NR columns of B, zero padded),
// so the micro-kernel is the same for every layout: MR x NR = 6 x 16 accumulators held in twelve
// ymm registers, one broadcast of A and two loads of B per k.  Panels of B are packed once per call
// and shared by all threads; every thread packs the A rows it owns.  K is cut into KC-deep slabs so
// a B slab (KC x NC) stays in L2.
//
// The CPU backend exists for the CPU-only configuration (GPT-2 small, two data-parallel thread
// workers) and as an independent check of the PyTorch oracle; replaces crates/backend-cpu/src/fast_ops.rs
// (AVX2 GEMM) and par.rs:27-83 (the worker pool).
#include <immintrin.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int MR = 6, NR = 16, KC = 256, NC = 1024;

template <typename F>
void parallel_for(int n, int threads, F fn) {
  threads = std::max(1, std::min(threads, n));
  if (threads == 1) {
    for (int i = 0; i < n; ++i) fn(i);
    return;
  }
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([=] {
      for (int i = t; i < n; i += threads) fn(i);
    });
  for (auto& th : pool) th.join();
}

// element (r, k) of op(A) / (k, c) of op(B) from the stored matrix
inline float a_at(const float* A, int lda, int ta, int r, int k) { return ta ? A[(size_t)k * lda + r] : A[(size_t)r * lda + k]; }
inline float b_at(const float* B, int ldb, int tb, int k, int c) { return tb ? B[(size_t)c * ldb + k] : B[(size_t)k * ldb + c]; }

// C tile [mr x nr] (+)= alpha * Ap[kc][MR] * Bp[kc][NR]
inline void micro(const float* Ap, const float* Bp, int kc, float* C, int ldc, int mr, int nr, float alpha,
                  bool accumulate, float beta) {
  __m256 acc[MR][2];
  for (int i = 0; i < MR; ++i) acc[i][0] = acc[i][1] = _mm256_setzero_ps();
  for (int k = 0; k < kc; ++k) {
    const __m256 b0 = _mm256_loadu_ps(Bp + (size_t)k * NR), b1 = _mm256_loadu_ps(Bp + (size_t)k * NR + 8);
    const float* a = Ap + (size_t)k * MR;
#pragma GCC unroll 6
    for (int i = 0; i < MR; ++i) {
      const __m256 av = _mm256_broadcast_ss(a + i);
      acc[i][0] = _mm256_fmadd_ps(av, b0, acc[i][0]);
      acc[i][1] = _mm256_fmadd_ps(av, b1, acc[i][1]);
    }
  }
  alignas(32) float tmp[MR][NR];
  for (int i = 0; i < MR; ++i) {
    _mm256_store_ps(tmp[i], acc[i][0]);
    _mm256_store_ps(tmp[i] + 8, acc[i][1]);
  }
  for (int i = 0; i < mr; ++i) {
    float* c = C + (size_t)i * ldc;
    for (int j = 0; j < nr; ++j) {
      const float v = alpha * tmp[i][j];
      c[j] = accumulate ? c[j] + v : (beta != 0.f ? beta * c[j] + v : v);
    }
  }
}

}  // namespace

BBH_API int bbh_cpu_gemm(const float* A, const float* B, float* C, int M, int N, int K, int lda, int ldb,
                         int ldc, int ta, int tb, float alpha, float beta, int threads) {
  if (M < 0 || N < 0 || K < 0) return -1;
  if (M == 0 || N == 0) return 0;
  if (K == 0) {
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) C[(size_t)i * ldc + j] = beta != 0.f ? beta * C[(size_t)i * ldc + j] : 0.f;
    return 0;
  }
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  const int m_panels = (M + MR - 1) / MR;
  std::vector<float> Bp((size_t)((std::min(N, NC) + NR - 1) / NR) * NR * KC);
  for (int k0 = 0; k0 < K; k0 += KC) {
    const int kc = std::min(KC, K - k0);
    const bool first_k = k0 == 0;
    for (int n0 = 0; n0 < N; n0 += NC) {
      const int nc = std::min(NC, N - n0);
      const int n_panels = (nc + NR - 1) / NR;
      // pack the B slab: panel p holds columns [n0 + p*NR, +NR) as [kc][NR]
      parallel_for(n_panels, threads, [&](int p) {
        float* dst = Bp.data() + (size_t)p * NR * KC;
        const int c0 = n0 + p * NR, nr = std::min(NR, N - c0);
        for (int k = 0; k < kc; ++k) {
          for (int j = 0; j < nr; ++j) dst[(size_t)k * NR + j] = b_at(B, ldb, tb, k0 + k, c0 + j);
          for (int j = nr; j < NR; ++j) dst[(size_t)k * NR + j] = 0.f;
        }
      });
      // every thread packs the A panels it owns and sweeps them over the shared B slab
      parallel_for(m_panels, threads, [&](int mp) {
        alignas(32) float Ap[MR * KC];
        const int r0 = mp * MR, mr = std::min(MR, M - r0);
        for (int k = 0; k < kc; ++k) {
          for (int i = 0; i < mr; ++i) Ap[k * MR + i] = a_at(A, lda, ta, r0 + i, k0 + k);
          for (int i = mr; i < MR; ++i) Ap[k * MR + i] = 0.f;
        }
        for (int p = 0; p < n_panels; ++p) {
          const int c0 = n0 + p * NR, nr = std::min(NR, N - c0);
          micro(Ap, Bp.data() + (size_t)p * NR * KC, kc, C + (size_t)r0 * ldc + c0, ldc, mr, nr, alpha,
                /*accumulate=*/!first_k, beta);
        }
      });
    }
  }
  return 0;
}

// y[rows, d] = x / sqrt(mean(x^2) + eps) * w      (row-parallel, AVX2)
BBH_API int bbh_cpu_rmsnorm(const float* x, const float* w, float* y, int rows, int d, float eps, int threads) {
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  const int chunk = 64;
  parallel_for((rows + chunk - 1) / chunk, threads, [&](int c) {
    for (int r = c * chunk; r < std::min(rows, (c + 1) * chunk); ++r) {
      const float* xr = x + (size_t)r * d;
      float* yr = y + (size_t)r * d;
      __m256 s = _mm256_setzero_ps();
      int i = 0;
      for (; i + 8 <= d; i += 8) {
        const __m256 v = _mm256_loadu_ps(xr + i);
        s = _mm256_fmadd_ps(v, v, s);
      }
      alignas(32) float t[8];
      _mm256_store_ps(t, s);
      double ss = (double)t[0] + t[1] + t[2] + t[3] + t[4] + t[5] + t[6] + t[7];
      for (; i < d; ++i) ss += (double)xr[i] * xr[i];
      const float inv = 1.0f / std::sqrt((float)(ss / d) + eps);
      for (int j = 0; j < d; ++j) yr[j] = xr[j] * inv * w[j];
    }
  });
  return 0;
}
