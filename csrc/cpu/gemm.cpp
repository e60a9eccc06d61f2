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
// loads of B per k.  A slab of B (KC x NC) is packed by all threads together and shared; every thread
// packs the A rows it owns.  Packs that transpose go through registers in 8 x 8 blocks.  Column slabs
// are the outer loop and K slabs the inner one, so a task's part of C stays in cache while K is summed.  A task owns a block of up to MC rows: it packs them once per slab and
// sweeps them over the slab one B panel at a time, so a B panel is pulled into L1 once per block instead
// of once per 6-row panel.  Worker threads are persistent (one pool per calling thread).
// Products with few rows of A (a batch of tokens against a weight matrix) take another route: all of A
// is packed once, then every task owns a run of columns and packs its own piece of B (one barrier per
// call).  Scratch buffers are per thread and grow-only; the workers park when a call ends.
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
    unsigned long g1;
    {
      std::lock_guard<std::mutex> g(m_);
      stop_.store(true, std::memory_order_release);
      g1 = ++gen_;
    }
    gen_pub_.store(g1, std::memory_order_release);
    cv_.notify_all();
    for (auto& t : th_) t.join();
  }
  int workers() const { return (int)th_.size(); }
  void quiet() { quiet_.store(true, std::memory_order_release); }

  template <typename F>
  void run(int n, F&& fn) {
    if (n <= 0) return;
    if (th_.empty() || n == 1) {
      for (int i = 0; i < n; ++i) fn(i);
      return;
    }
    std::function<void(int)> f = std::ref(fn);
    // The job is written first and published by the release store of the generation: workers that
    // spin pick it up without the mutex.  (Publishing inside the critical section sent every spinning
    // worker straight into a blocked lock, a sleep and a wake-up per parallel region.)
    job_ = &f;
    n_ = n;
    quiet_.store(false, std::memory_order_relaxed);
    next_.store(0, std::memory_order_relaxed);
    left_.store((int)th_.size(), std::memory_order_relaxed);
    unsigned long g1;
    {
      std::lock_guard<std::mutex> g(m_);
      g1 = ++gen_;
    }
    gen_pub_.store(g1, std::memory_order_release);
    if (parked_.load(std::memory_order_acquire) != 0) cv_.notify_all();
    for (int i; (i = next_.fetch_add(1, std::memory_order_relaxed)) < n;) fn(i);
    for (int spin = 0; spin < 200000 && left_.load(std::memory_order_acquire) != 0; ++spin) _mm_pause();
    if (left_.load(std::memory_order_acquire) != 0) {
      std::unique_lock<std::mutex> g(m_);
      done_.wait(g, [this] { return left_.load(std::memory_order_acquire) == 0; });
    }
    job_ = nullptr;
  }

 private:
  void loop() {
    unsigned long seen = 0;
    for (;;) {
      // a GEMM is several short parallel regions back to back: spin for the next one for a while
      // before parking (a condition-variable wake-up costs tens of microseconds per region)
      // generations only grow; "newer than seen" (not "different") because a worker that was woken
      // through gen_ can be one step ahead of gen_pub_ for a moment
      auto newer = [&](unsigned long g) { return (long)(g - seen) > 0; };
      for (int spin = 0; spin < 20000 && !newer(gen_pub_.load(std::memory_order_acquire)) &&
                         !quiet_.load(std::memory_order_acquire);
           ++spin)
        _mm_pause();
      unsigned long cur = gen_pub_.load(std::memory_order_acquire);
      if (!newer(cur)) {
        std::unique_lock<std::mutex> g(m_);
        parked_.fetch_add(1, std::memory_order_acq_rel);
        cv_.wait(g, [&] { return newer(gen_); });
        parked_.fetch_sub(1, std::memory_order_acq_rel);
        cur = gen_;
      }
      // run() starts the next generation only after every worker has finished this one, so the
      // job fields are stable from here to the decrement below
      seen = cur;
      if (stop_.load(std::memory_order_acquire)) return;
      std::function<void(int)>* f = job_;
      const int n = n_;
      for (int i; (i = next_.fetch_add(1, std::memory_order_relaxed)) < n;) (*f)(i);
      if (left_.fetch_sub(1, std::memory_order_acq_rel) == 1) {
        std::lock_guard<std::mutex> g(m_);   // the caller may be asleep on done_: wake it under the lock
        done_.notify_one();
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
  std::atomic<bool> quiet_{false};          // set at the end of a GEMM call: park without spinning
  std::atomic<int> parked_{0};              // workers asleep on cv_ (run() skips the notify when none are)
  int n_ = 0;
  unsigned long gen_ = 0;
  std::atomic<bool> stop_{false};
};

thread_local std::unique_ptr<Pool> tl_pool;

Pool& pool_for(int threads) {
  if (!tl_pool || tl_pool->workers() != threads - 1) tl_pool.reset(new Pool(threads - 1));
  return *tl_pool;
}

// End of a GEMM call: the workers stop spinning for the next region and park at once.  What follows
// a GEMM in a training step is other libraries' thread teams on the same cores (bias, activation,
// normalisation), which spinning workers would be time-sliced against.
void quiesce_pool() {
  if (tl_pool) tl_pool->quiet();
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

// dst[k * W + j] = src[j * ld + k] for j < rows, k < kc; columns rows..W-1 of dst are zero.  The
// source rows are contiguous in k, so the copy is a transpose: 8 x 8 blocks go through registers
// (eight loads, three rounds of shuffles, eight stores), 4 x 4 blocks likewise with SSE, the rest
// element by element.  Element-wise strided stores made the two transposing packs a quarter of a
// layer-sized GEMM's time.
inline void pack_transposed(const float* src, size_t ld, int rows, int kc, float* dst, int W) {
  int j = 0;
  for (; j + 8 <= rows; j += 8) {
    const float* s = src + (size_t)j * ld;
    int k = 0;
    for (; k + 8 <= kc; k += 8) {
      __m256 r0 = _mm256_loadu_ps(s + 0 * ld + k), r1 = _mm256_loadu_ps(s + 1 * ld + k);
      __m256 r2 = _mm256_loadu_ps(s + 2 * ld + k), r3 = _mm256_loadu_ps(s + 3 * ld + k);
      __m256 r4 = _mm256_loadu_ps(s + 4 * ld + k), r5 = _mm256_loadu_ps(s + 5 * ld + k);
      __m256 r6 = _mm256_loadu_ps(s + 6 * ld + k), r7 = _mm256_loadu_ps(s + 7 * ld + k);
      const __m256 t0 = _mm256_unpacklo_ps(r0, r1), t1 = _mm256_unpackhi_ps(r0, r1);
      const __m256 t2 = _mm256_unpacklo_ps(r2, r3), t3 = _mm256_unpackhi_ps(r2, r3);
      const __m256 t4 = _mm256_unpacklo_ps(r4, r5), t5 = _mm256_unpackhi_ps(r4, r5);
      const __m256 t6 = _mm256_unpacklo_ps(r6, r7), t7 = _mm256_unpackhi_ps(r6, r7);
      r0 = _mm256_shuffle_ps(t0, t2, 0x44); r1 = _mm256_shuffle_ps(t0, t2, 0xEE);
      r2 = _mm256_shuffle_ps(t1, t3, 0x44); r3 = _mm256_shuffle_ps(t1, t3, 0xEE);
      r4 = _mm256_shuffle_ps(t4, t6, 0x44); r5 = _mm256_shuffle_ps(t4, t6, 0xEE);
      r6 = _mm256_shuffle_ps(t5, t7, 0x44); r7 = _mm256_shuffle_ps(t5, t7, 0xEE);
      float* d = dst + (size_t)k * W + j;
      _mm256_storeu_ps(d + 0 * (size_t)W, _mm256_permute2f128_ps(r0, r4, 0x20));
      _mm256_storeu_ps(d + 1 * (size_t)W, _mm256_permute2f128_ps(r1, r5, 0x20));
      _mm256_storeu_ps(d + 2 * (size_t)W, _mm256_permute2f128_ps(r2, r6, 0x20));
      _mm256_storeu_ps(d + 3 * (size_t)W, _mm256_permute2f128_ps(r3, r7, 0x20));
      _mm256_storeu_ps(d + 4 * (size_t)W, _mm256_permute2f128_ps(r0, r4, 0x31));
      _mm256_storeu_ps(d + 5 * (size_t)W, _mm256_permute2f128_ps(r1, r5, 0x31));
      _mm256_storeu_ps(d + 6 * (size_t)W, _mm256_permute2f128_ps(r2, r6, 0x31));
      _mm256_storeu_ps(d + 7 * (size_t)W, _mm256_permute2f128_ps(r3, r7, 0x31));
    }
    for (; k < kc; ++k)
      for (int jj = 0; jj < 8; ++jj) dst[(size_t)k * W + j + jj] = s[(size_t)jj * ld + k];
  }
  for (; j + 4 <= rows; j += 4) {
    const float* s = src + (size_t)j * ld;
    int k = 0;
    for (; k + 4 <= kc; k += 4) {
      __m128 r0 = _mm_loadu_ps(s + 0 * ld + k), r1 = _mm_loadu_ps(s + 1 * ld + k);
      __m128 r2 = _mm_loadu_ps(s + 2 * ld + k), r3 = _mm_loadu_ps(s + 3 * ld + k);
      _MM_TRANSPOSE4_PS(r0, r1, r2, r3);
      float* d = dst + (size_t)k * W + j;
      _mm_storeu_ps(d + 0 * (size_t)W, r0);
      _mm_storeu_ps(d + 1 * (size_t)W, r1);
      _mm_storeu_ps(d + 2 * (size_t)W, r2);
      _mm_storeu_ps(d + 3 * (size_t)W, r3);
    }
    for (; k < kc; ++k)
      for (int jj = 0; jj < 4; ++jj) dst[(size_t)k * W + j + jj] = s[(size_t)jj * ld + k];
  }
  for (; j < rows; ++j) {
    const float* s = src + (size_t)j * ld;
    for (int k = 0; k < kc; ++k) dst[(size_t)k * W + j] = s[k];
  }
  if (rows < W)
    for (int k = 0; k < kc; ++k)
      for (int jj = rows; jj < W; ++jj) dst[(size_t)k * W + jj] = 0.f;
}

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
  // Few rows (a batch of tokens against a weight matrix: forward, dX, the LM head): the whole of A is
  // packed once, by all threads together, and after that single barrier every task owns a run of
  // columns: it packs its own piece of B (which stays in its core's L2 and is read by nobody else) and
  // takes all rows of A over it, K slab by K slab, so its piece of C stays in cache too.  The row-block
  // scheme below packs a B slab together, waits, computes, waits, eighteen times for a layer-sized
  // product, and every core reads the whole slab out of the others' caches.
  const int total_panels = (N + NR - 1) / NR;
  if ((size_t)M * KC * sizeof(float) <= (1u << 20) && (size_t)M * K * sizeof(float) <= (8u << 20) &&
      total_panels >= threads) {
    const int m_panels = (M + MR - 1) / MR, k_slabs = (K + KC - 1) / KC;
    // scratch that outlives the call (grow-only, one per calling / worker thread): a fresh megabyte-sized
    // vector per call is a new mapping whose pages fault in one by one
    static thread_local std::vector<float> Apack_tl;
    if (Apack_tl.size() < (size_t)m_panels * MR * K) Apack_tl.resize((size_t)m_panels * MR * K);
    float* const Apack = Apack_tl.data();   // slab s at m_panels*MR*(s*KC), panel pi at + pi*MR*kc
    parallel_for(k_slabs * m_panels, threads, [&](int t) {
      const int sl = t / m_panels, pi = t % m_panels;
      const int k0 = sl * KC, kc = std::min(KC, K - k0);
      const int r0 = pi * MR, mr = std::min(MR, M - r0);
      float* ap = Apack + (size_t)m_panels * MR * k0 + (size_t)pi * MR * kc;
      if (!ta) {
        pack_transposed(A + (size_t)r0 * lda + k0, (size_t)lda, mr, kc, ap, MR);
      } else {
        for (int k = 0; k < kc; ++k) {
          const float* src = A + (size_t)(k0 + k) * lda + r0;
          for (int i = 0; i < mr; ++i) ap[(size_t)k * MR + i] = src[i];
          for (int i = mr; i < MR; ++i) ap[(size_t)k * MR + i] = 0.f;
        }
      }
    });
    // panels per task: at most 8 (a 256 KB piece of B), and a task count that is a multiple of the
    // thread count so that the last round is not one straggler
    const int rounds = std::max(total_panels >= 4 * threads ? 2 : 1, (total_panels + 8 * threads - 1) / (8 * threads));
    const int cw = (total_panels + rounds * threads - 1) / (rounds * threads);
    parallel_for((total_panels + cw - 1) / cw, threads, [&](int t) {
      const int p_lo = t * cw, p_hi = std::min(total_panels, p_lo + cw);
      static thread_local std::vector<float> Bq;
      if (Bq.size() < (size_t)cw * NR * KC) Bq.resize((size_t)cw * NR * KC);
      for (int k0 = 0; k0 < K; k0 += KC) {
        const int kc = std::min(KC, K - k0);
        for (int p = p_lo; p < p_hi; ++p) {
          float* dst = Bq.data() + (size_t)(p - p_lo) * NR * KC;
          const int c0 = p * NR, nr = std::min(NR, N - c0);
          if (tb) {
            pack_transposed(B + (size_t)c0 * ldb + k0, (size_t)ldb, nr, kc, dst, NR);
          } else {
            for (int k = 0; k < kc; ++k) {
              const float* src = B + (size_t)(k0 + k) * ldb + c0;
              if (nr == NR) {
                std::memcpy(dst + (size_t)k * NR, src, NR * sizeof(float));
              } else {
                for (int j = 0; j < nr; ++j) dst[(size_t)k * NR + j] = src[j];
                for (int j = nr; j < NR; ++j) dst[(size_t)k * NR + j] = 0.f;
              }
            }
          }
        }
        const float* aslab = Apack + (size_t)m_panels * MR * k0;
        for (int p = p_lo; p < p_hi; ++p) {
          const float* bp = Bq.data() + (size_t)(p - p_lo) * NR * KC;
          const int c0 = p * NR, nr = std::min(NR, N - c0);
          for (int pi = 0; pi < m_panels; ++pi) {
            const int r0 = pi * MR, mr = std::min(MR, M - r0);
            Micro::run(aslab + (size_t)pi * MR * kc, bp, kc, C + (size_t)r0 * ldc + c0, ldc, mr, nr, alpha,
                       /*accumulate=*/k0 != 0, beta);
          }
        }
      }
    });
    return 0;
  }
  // tasks: MC-row blocks of A (their packed panels stay in the owner's L2 while it sweeps the B slab);
  // small M is cut finer so that every thread gets work
  int mc = MC;
  while (mc > MR && (M + mc - 1) / mc < 2 * threads) mc -= MR;
  const int m_blocks = (M + mc - 1) / mc;
  static thread_local std::vector<float> Bp;   // grow-only scratch, see above
  if (Bp.size() < (size_t)((std::min(N, NC) + NR - 1) / NR) * NR * KC) Bp.resize((size_t)((std::min(N, NC) + NR - 1) / NR) * NR * KC);
  float* const Bp_data = Bp.data();            // workers use the caller's buffer through this pointer
  // column slabs outside, K slabs inside: a task's part of C (its rows x NC columns) is accumulated
  // over all of K while it is still in cache; with K outside, a wide C (the LM head's) went to
  // memory and back once per K slab
  for (int n0 = 0; n0 < N; n0 += NC) {
    const int nc = std::min(NC, N - n0);
    const int n_panels = (nc + NR - 1) / NR;
    for (int k0 = 0; k0 < K; k0 += KC) {
      const int kc = std::min(KC, K - k0);
      const bool first_k = k0 == 0;
      // pack the B slab: panel p holds columns [n0 + p*NR, +NR) as [kc][NR]
      if (!tb) {
        // B stored [K][N]: tasks own runs of k rows and read each row of the slab front to back (one
        // sequential stream), dealing it out NR floats at a time to the panels; copying panel by
        // panel instead touched two cache lines per row of a panel, a page apart each
        constexpr int KR = 16;
        const int full = nc / NR, rem = nc - full * NR;
        parallel_for((kc + KR - 1) / KR, threads, [&](int t) {
          for (int k = t * KR; k < std::min(kc, (t + 1) * KR); ++k) {
            const float* src = B + (size_t)(k0 + k) * ldb + n0;
            float* dst = Bp_data + (size_t)k * NR;
            for (int q = 0; q < full; ++q) std::memcpy(dst + (size_t)q * NR * KC, src + (size_t)q * NR, NR * sizeof(float));
            if (rem) {
              float* d = dst + (size_t)full * NR * KC;
              for (int j = 0; j < rem; ++j) d[j] = src[(size_t)full * NR + j];
              for (int j = rem; j < NR; ++j) d[j] = 0.f;
            }
          }
        });
      } else {
        parallel_for(n_panels, threads, [&](int p) {   // B stored [N][K]: NR source rows, transposed on the way
          const int c0 = n0 + p * NR, nr = std::min(NR, N - c0);
          pack_transposed(B + (size_t)c0 * ldb + k0, (size_t)ldb, nr, kc, Bp_data + (size_t)p * NR * KC, NR);
        });
      }
      // every task packs its block of A once and sweeps it over the B slab panel by panel: a B panel
      // (16 KB) is read into L1 once per block and reused by all of the block's row panels
      parallel_for(m_blocks, threads, [&](int mb) {
        const int r_lo = mb * mc, rows = std::min(mc, M - r_lo);
        const int panels = (rows + MR - 1) / MR;
        static thread_local std::vector<float> Ap;
        if (Ap.size() < (size_t)panels * MR * kc) Ap.resize((size_t)panels * MR * kc);
        for (int pi = 0; pi < panels; ++pi) {
          float* ap = Ap.data() + (size_t)pi * MR * kc;
          const int r0 = r_lo + pi * MR, mr = std::min(MR, M - r0);
          if (!ta) {
            pack_transposed(A + (size_t)r0 * lda + k0, (size_t)lda, mr, kc, ap, MR);
          } else {
            for (int k = 0; k < kc; ++k) {
              const float* src = A + (size_t)(k0 + k) * lda + r0;
              for (int i = 0; i < mr; ++i) ap[(size_t)k * MR + i] = src[i];
              for (int i = mr; i < MR; ++i) ap[(size_t)k * MR + i] = 0.f;
            }
          }
        }
        for (int p = 0; p < n_panels; ++p) {
          const int c0 = n0 + p * NR, nr = std::min(NR, N - c0);
          const float* bp = Bp_data + (size_t)p * NR * KC;
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
  const int rc = wide ? gemm_impl<MicroAvx512>(A, B, C, M, N, K, lda, ldb, ldc, ta, tb, alpha, beta, threads)
                      : gemm_impl<MicroAvx2>(A, B, C, M, N, K, lda, ldb, ldc, ta, tb, alpha, beta, threads);
  quiesce_pool();
  return rc;
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
