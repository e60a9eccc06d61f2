// CPU backend, native part: fp32 GEMM for the three products a linear layer needs.  The file is built
// for x86-64-v3 (AVX2 + FMA); on CPUs with AVX-512 a wider micro-kernel is chosen at run time.
//
//   bbh_cpu_gemm(ta, tb)   C[M,N] = alpha * op(A) * op(B) + beta * C
//                          op(A) = A[M,K] (ta = 0) or A[K,M]^T (ta = 1); op(B) = B[K,N] (tb = 0) or
//                          B[N,K]^T (tb = 1).  forward y = x W^T is (0,1); dX = dY W is (0,0);
//                          dW = dY^T X is (1,0).
//
// Method: both operands are packed into K-major panels (MR rows of A, NR columns of B, zero padded),
// so the micro-kernel is the same for every layout: MR x NR = 6 x 16 accumulators in twelve ymm
// registers (AVX2) or 12 x 32 in twenty-four zmm registers (AVX-512), one broadcast of A per row and two
// loads of B per k.  Panels of B are packed once per call
// and shared by all threads; every thread packs the A rows it owns.  K is cut into KC-deep slabs so
// a B slab (KC x NC) stays in L2.  A task owns a block of up to MC rows: it packs them once per slab and
// sweeps them over the slab one B panel at a time, so a B panel is pulled into L1 once per block instead
// of once per 6-row panel.  Worker threads are persistent (one pool per calling thread).
//
// The CPU backend exists for the CPU-only configuration (GPT-2 small, two data-parallel thread
// workers) and as an independent check of the PyTorch oracle; replaces crates/backend-cpu/src/fast_ops.rs
// (AVX2 GEMM) and par.rs:27-83 (the worker pool).
#include <immintrin.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int KC = 256, NC = 1024, MC = 96;   // MC: rows of A one task keeps hot in L2
// MR (rows of an A panel): 6 with AVX2, 12 with AVX-512 (24 of the 32 zmm registers hold the tile)
// NR (columns of a B panel): 16 with AVX2 (two ymm per row), 32 with AVX-512 (two zmm per row)

// Persistent workers, one pool per CALLING thread (the thread data-parallel workers of the CPU
// configuration each drive their own).  A call publishes a job (index range + function), the
// workers and the caller pull indices from one atomic counter, the caller returns when all are done.
// Threads are started on first use and parked on a condition variable between jobs; starting eight
// threads per parallel region cost more than small layers' GEMMs take.
class Pool {
 public:
  explicit Pool(int workers) {
    for (int t = 0; t < workers; ++t) th_.emplace_back([this] { loop(); });
  }
  ~Pool() {
    {
      std::lock_guard<std::mutex> g(m_);
      stop_ = true;
      ++gen_;
      gen_pub_.store(gen_, std::memory_order_release);
    }
    cv_.notify_all();
    for (auto& t : th_) t.join();
  }
  int workers() const { return (int)th_.size(); }

  template <typename F>
  void run(int n, F&& fn) {
    if (n <= 0) return;
    if (th_.empty() || n == 1) {
      for (int i = 0; i < n; ++i) fn(i);
      return;
    }
    std::function<void(int)> f = std::ref(fn);
    {
      std::lock_guard<std::mutex> g(m_);
      job_ = &f;
      n_ = n;
      next_.store(0, std::memory_order_relaxed);
      pending_ = (int)th_.size();
      left_.store(pending_, std::memory_order_relaxed);
      ++gen_;
      gen_pub_.store(gen_, std::memory_order_release);
    }
    cv_.notify_all();
    for (int i; (i = next_.fetch_add(1, std::memory_order_relaxed)) < n;) fn(i);
    for (int spin = 0; spin < 20000 && left_.load(std::memory_order_acquire) != 0; ++spin) _mm_pause();
    std::unique_lock<std::mutex> g(m_);
    done_.wait(g, [this] { return pending_ == 0; });
    job_ = nullptr;
  }

 private:
  void loop() {
    unsigned long seen = 0;
    for (;;) {
      std::function<void(int)>* f;
      int n;
      // a GEMM is several short parallel regions back to back: spin for the next one for a while
      // before parking (a condition-variable wake-up costs tens of microseconds per region)
      for (int spin = 0; spin < 20000 && gen_pub_.load(std::memory_order_acquire) == seen; ++spin) _mm_pause();
      {
        std::unique_lock<std::mutex> g(m_);
        cv_.wait(g, [&] { return gen_ != seen; });
        seen = gen_;
        if (stop_) return;
        f = job_;
        n = n_;
      }
      for (int i; (i = next_.fetch_add(1, std::memory_order_relaxed)) < n;) (*f)(i);
      {
        std::lock_guard<std::mutex> g(m_);
        left_.store(pending_ - 1, std::memory_order_release);
        if (--pending_ == 0) done_.notify_one();
      }
    }
  }
  std::vector<std::thread> th_;
  std::mutex m_;
  std::condition_variable cv_, done_;
  std::function<void(int)>* job_ = nullptr;
  std::atomic<int> next_{0};
  std::atomic<int> left_{0};
  std::atomic<unsigned long> gen_pub_{0};   // copy of gen_ the spinning workers poll without the lock
  int n_ = 0, pending_ = 0;
  unsigned long gen_ = 0;
  bool stop_ = false;
};

Pool& pool_for(int threads) {
  thread_local std::unique_ptr<Pool> pool;
  if (!pool || pool->workers() != threads - 1) pool.reset(new Pool(threads - 1));
  return *pool;
}

template <typename F>
void parallel_for(int n, int threads, F fn) {
  threads = std::max(1, std::min(threads, n));
  if (threads == 1) {
    for (int i = 0; i < n; ++i) fn(i);
    return;
  }
  pool_for(threads).run(n, fn);
}

// element (r, k) of op(A) / (k, c) of op(B) from the stored matrix
inline float a_at(const float* A, int lda, int ta, int r, int k) { return ta ? A[(size_t)k * lda + r] : A[(size_t)r * lda + k]; }
inline float b_at(const float* B, int ldb, int tb, int k, int c) { return tb ? B[(size_t)c * ldb + k] : B[(size_t)k * ldb + c]; }

// C tile [mr x nr] = (first k-slab ? beta * C : C) + alpha * Ap[kc][MR] * Bp[kc][NR]: the ragged-edge
// write-back shared by both micro-kernels
template <int NR>
inline void store_edge(const float (*tmp)[NR], float* C, int ldc, int mr, int nr, float alpha, bool accumulate,
                       float beta) {   // tmp: [MR][NR] accumulators
  for (int i = 0; i < mr; ++i) {
    float* c = C + (size_t)i * ldc;
    for (int j = 0; j < nr; ++j) {
      const float v = alpha * tmp[i][j];
      c[j] = accumulate ? c[j] + v : (beta != 0.f ? beta * c[j] + v : v);
    }
  }
}

// AVX2: 6 x 16 accumulators in twelve ymm registers, one broadcast of A and two loads of B per k
struct MicroAvx2 {
  static constexpr int MR = 6, NR = 16;
  static inline void run(const float* Ap, const float* Bp, int kc, float* C, int ldc, int mr, int nr, float alpha,
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
    if (mr == MR && nr == NR) {   // whole tile: vector read-modify-write of C
      const __m256 va = _mm256_set1_ps(alpha), vb = _mm256_set1_ps(accumulate ? 1.f : beta);
      const bool keep = accumulate || beta != 0.f;
#pragma GCC unroll 6
      for (int i = 0; i < MR; ++i) {
        float* c = C + (size_t)i * ldc;
        __m256 r0 = _mm256_mul_ps(va, acc[i][0]), r1 = _mm256_mul_ps(va, acc[i][1]);
        if (keep) {
          r0 = _mm256_fmadd_ps(vb, _mm256_loadu_ps(c), r0);
          r1 = _mm256_fmadd_ps(vb, _mm256_loadu_ps(c + 8), r1);
        }
        _mm256_storeu_ps(c, r0);
        _mm256_storeu_ps(c + 8, r1);
      }
      return;
    }
    alignas(32) float tmp[MR][NR];
    for (int i = 0; i < MR; ++i) {
      _mm256_store_ps(tmp[i], acc[i][0]);
      _mm256_store_ps(tmp[i] + 8, acc[i][1]);
    }
    store_edge<NR>(tmp, C, ldc, mr, nr, alpha, accumulate, beta);
  }
};

// AVX-512 (chosen at run time where the CPU has it; the rest of the file is built for AVX2):
// 12 x 32 accumulators in twenty-four zmm registers
struct MicroAvx512 {
  static constexpr int MR = 12, NR = 32;
  __attribute__((target("avx512f"))) static inline void run(const float* Ap, const float* Bp, int kc, float* C,
                                                            int ldc, int mr, int nr, float alpha, bool accumulate,
                                                            float beta) {
    __m512 acc[MR][2];
    for (int i = 0; i < MR; ++i) acc[i][0] = acc[i][1] = _mm512_setzero_ps();
    for (int k = 0; k < kc; ++k) {
      const __m512 b0 = _mm512_loadu_ps(Bp + (size_t)k * NR), b1 = _mm512_loadu_ps(Bp + (size_t)k * NR + 16);
      const float* a = Ap + (size_t)k * MR;
#pragma GCC unroll 12
      for (int i = 0; i < MR; ++i) {
        const __m512 av = _mm512_set1_ps(a[i]);
        acc[i][0] = _mm512_fmadd_ps(av, b0, acc[i][0]);
        acc[i][1] = _mm512_fmadd_ps(av, b1, acc[i][1]);
      }
    }
    if (mr == MR && nr == NR) {
      const __m512 va = _mm512_set1_ps(alpha), vb = _mm512_set1_ps(accumulate ? 1.f : beta);
      const bool keep = accumulate || beta != 0.f;
#pragma GCC unroll 12
      for (int i = 0; i < MR; ++i) {
        float* c = C + (size_t)i * ldc;
        __m512 r0 = _mm512_mul_ps(va, acc[i][0]), r1 = _mm512_mul_ps(va, acc[i][1]);
        if (keep) {
          r0 = _mm512_fmadd_ps(vb, _mm512_loadu_ps(c), r0);
          r1 = _mm512_fmadd_ps(vb, _mm512_loadu_ps(c + 16), r1);
        }
        _mm512_storeu_ps(c, r0);
        _mm512_storeu_ps(c + 16, r1);
      }
      return;
    }
    alignas(64) float tmp[MR][NR];
    for (int i = 0; i < MR; ++i) {
      _mm512_store_ps(tmp[i], acc[i][0]);
      _mm512_store_ps(tmp[i] + 16, acc[i][1]);
    }
    store_edge<NR>(tmp, C, ldc, mr, nr, alpha, accumulate, beta);
  }
};

}  // namespace

template <typename Micro>
static int gemm_impl(const float* A, const float* B, float* C, int M, int N, int K, int lda, int ldb, int ldc,
                     int ta, int tb, float alpha, float beta, int threads) {
  constexpr int NR = Micro::NR, MR = Micro::MR;
  if (M < 0 || N < 0 || K < 0) return -1;
  if (M == 0 || N == 0) return 0;
  if (K == 0) {
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) C[(size_t)i * ldc + j] = beta != 0.f ? beta * C[(size_t)i * ldc + j] : 0.f;
    return 0;
  }
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  // tasks: MC-row blocks of A (their packed panels stay in the owner's L2 while it sweeps the B slab);
  // small M is cut finer so that every thread gets work
  int mc = MC;
  while (mc > MR && (M + mc - 1) / mc < 2 * threads) mc -= MR;
  const int m_blocks = (M + mc - 1) / mc;
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
        if (tb && nr == NR) {           // B stored [N][K]: 16 rows of the source, transposed on the way
          for (int j = 0; j < NR; ++j) {
            const float* src = B + (size_t)(c0 + j) * ldb + k0;
            for (int k = 0; k < kc; ++k) dst[(size_t)k * NR + j] = src[k];
          }
        } else if (!tb && nr == NR) {   // B stored [K][N]: contiguous 16-float rows
          for (int k = 0; k < kc; ++k) std::memcpy(dst + (size_t)k * NR, B + (size_t)(k0 + k) * ldb + c0, NR * sizeof(float));
        } else {
          for (int k = 0; k < kc; ++k) {
            for (int j = 0; j < nr; ++j) dst[(size_t)k * NR + j] = b_at(B, ldb, tb, k0 + k, c0 + j);
            for (int j = nr; j < NR; ++j) dst[(size_t)k * NR + j] = 0.f;
          }
        }
      });
      // every task packs its block of A once and sweeps it over the B slab panel by panel: a B panel
      // (16 KB) is read into L1 once per block and reused by all of the block's row panels
      parallel_for(m_blocks, threads, [&](int mb) {
        const int r_lo = mb * mc, rows = std::min(mc, M - r_lo);
        const int panels = (rows + MR - 1) / MR;
        std::vector<float> Ap((size_t)panels * MR * kc);
        for (int pi = 0; pi < panels; ++pi) {
          float* ap = Ap.data() + (size_t)pi * MR * kc;
          const int r0 = r_lo + pi * MR, mr = std::min(MR, M - r0);
          if (!ta) {
            for (int i = 0; i < mr; ++i) {
              const float* src = A + (size_t)(r0 + i) * lda + k0;
              for (int k = 0; k < kc; ++k) ap[(size_t)k * MR + i] = src[k];
            }
          } else {
            for (int k = 0; k < kc; ++k)
              for (int i = 0; i < mr; ++i) ap[(size_t)k * MR + i] = A[(size_t)(k0 + k) * lda + r0 + i];
          }
          for (int i = mr; i < MR; ++i)
            for (int k = 0; k < kc; ++k) ap[(size_t)k * MR + i] = 0.f;
        }
        for (int p = 0; p < n_panels; ++p) {
          const int c0 = n0 + p * NR, nr = std::min(NR, N - c0);
          const float* bp = Bp.data() + (size_t)p * NR * KC;
          for (int pi = 0; pi < panels; ++pi) {
            const int r0 = r_lo + pi * MR, mr = std::min(MR, M - r0);
            Micro::run(Ap.data() + (size_t)pi * MR * kc, bp, kc, C + (size_t)r0 * ldc + c0, ldc, mr, nr, alpha,
                       /*accumulate=*/!first_k, beta);
          }
        }
      });
    }
  }
  return 0;
}

BBH_API int bbh_cpu_gemm(const float* A, const float* B, float* C, int M, int N, int K, int lda, int ldb,
                         int ldc, int ta, int tb, float alpha, float beta, int threads) {
  // BRAIN_CPU_ISA=avx2 keeps the 6 x 16 AVX2 micro-kernel on CPUs that have AVX-512 (tests cover both)
  static const bool wide = [] {
    const char* e = std::getenv("BRAIN_CPU_ISA");
    if (e && std::strcmp(e, "avx2") == 0) return false;
    return (bool)__builtin_cpu_supports("avx512f");
  }();
  return wide ? gemm_impl<MicroAvx512>(A, B, C, M, N, K, lda, ldb, ldc, ta, tb, alpha, beta, threads)
              : gemm_impl<MicroAvx2>(A, B, C, M, N, K, lda, ldb, ldc, ta, tb, alpha, beta, threads);
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
