// CPU backend, native part: causal / full softmax attention with grouped KV heads, forward and
// backward, fp32.  Rows are tokens: q [B*T, hq*hd], k and v [B*S, hk*hd] (row strides given), head h
// at columns [h*hd, (h+1)*hd).  Query row i of a sequence sees keys 0 .. i + (S - T) when causal.
//
// Forward, per (sequence, query head) and block of 32 query rows: tiles of 64 keys; each tile is used by
// every row of the block (scores, running maximum and sum, rescale, weighted sum of the tile's V rows)
// before the next tile is touched, so K and V are read once per block of rows, not once per row.  The
// log-sum-exp of every row is kept for backward.  No T x S matrix exists at any point.
// Backward in two passes that both recompute the probabilities from the saved log-sum-exp: dQ per block
// of query rows over key tiles, then dK / dV per block of keys over query-row tiles (scores with the
// roles swapped), so every output row belongs to exactly one task and nothing is shared between threads.
// Dot products and row updates go eight rows at a time (one set of horizontal sums, one load and store
// of the updated row per eight multiply-adds).
//
// Replaces the attention half of crates/backend-cpu/src/fast_ops.rs; the PyTorch restatement with
// materialised scores (ops/reference.py) stays the oracle.
#include <immintrin.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

// e^x for x <= 0 (and moderately positive x): x = n ln2 + r, |r| <= ln2 / 2, degree-6 polynomial for
// e^r, 2^n through the exponent field.  Relative error about 2e-7; inputs below -87 give 0.
inline __m256 exp256(__m256 x) {
  const __m256 lo = _mm256_set1_ps(-87.0f);
  const __m256 under = _mm256_cmp_ps(x, lo, _CMP_LT_OQ);
  x = _mm256_max_ps(x, lo);
  x = _mm256_min_ps(x, _mm256_set1_ps(88.0f));
  const __m256 n = _mm256_round_ps(_mm256_mul_ps(x, _mm256_set1_ps(1.44269504088896341f)),
                                   _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
  __m256 r = _mm256_fnmadd_ps(n, _mm256_set1_ps(0.693359375f), x);
  r = _mm256_fnmadd_ps(n, _mm256_set1_ps(-2.12194440e-4f), r);
  __m256 p = _mm256_set1_ps(1.9875691500e-4f);
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.3981999507e-3f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(8.3334519073e-3f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(4.1665795894e-2f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.6666665459e-1f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(5.0000001201e-1f));
  p = _mm256_fmadd_ps(p, _mm256_mul_ps(r, r), _mm256_add_ps(r, _mm256_set1_ps(1.0f)));
  const __m256i e = _mm256_slli_epi32(_mm256_add_epi32(_mm256_cvtps_epi32(n), _mm256_set1_epi32(127)), 23);
  p = _mm256_mul_ps(p, _mm256_castsi256_ps(e));
  return _mm256_andnot_ps(under, p);
}

inline float hsum(__m256 v) {
  __m128 s = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
  s = _mm_add_ps(s, _mm_movehl_ps(s, s));
  s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 1));
  return _mm_cvtss_f32(s);
}

inline float dot(const float* a, const float* b, int hd) {
  __m256 s0 = _mm256_setzero_ps(), s1 = _mm256_setzero_ps();
  int d = 0;
  for (; d + 16 <= hd; d += 16) {
    s0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + d), _mm256_loadu_ps(b + d), s0);
    s1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + d + 8), _mm256_loadu_ps(b + d + 8), s1);
  }
  for (; d < hd; d += 8) s0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + d), _mm256_loadu_ps(b + d), s0);
  return hsum(_mm256_add_ps(s0, s1));
}

// eight dot products at once: a . b_t for rows b_t = b + t * ldb, t = 0..7, as one vector.  Eight
// accumulators share every load of a, and the horizontal sums are done for all eight together
// (three rounds of pairwise adds) instead of once per product.
inline __m256 dot8(const float* a, const float* b, int64_t ldb, int hd) {
  __m256 s0 = _mm256_setzero_ps(), s1 = s0, s2 = s0, s3 = s0, s4 = s0, s5 = s0, s6 = s0, s7 = s0;
  for (int d = 0; d < hd; d += 8) {
    const __m256 av = _mm256_loadu_ps(a + d);
    s0 = _mm256_fmadd_ps(av, _mm256_loadu_ps(b + 0 * ldb + d), s0);
    s1 = _mm256_fmadd_ps(av, _mm256_loadu_ps(b + 1 * ldb + d), s1);
    s2 = _mm256_fmadd_ps(av, _mm256_loadu_ps(b + 2 * ldb + d), s2);
    s3 = _mm256_fmadd_ps(av, _mm256_loadu_ps(b + 3 * ldb + d), s3);
    s4 = _mm256_fmadd_ps(av, _mm256_loadu_ps(b + 4 * ldb + d), s4);
    s5 = _mm256_fmadd_ps(av, _mm256_loadu_ps(b + 5 * ldb + d), s5);
    s6 = _mm256_fmadd_ps(av, _mm256_loadu_ps(b + 6 * ldb + d), s6);
    s7 = _mm256_fmadd_ps(av, _mm256_loadu_ps(b + 7 * ldb + d), s7);
  }
  const __m256 a0123 = _mm256_hadd_ps(_mm256_hadd_ps(s0, s1), _mm256_hadd_ps(s2, s3));
  const __m256 a4567 = _mm256_hadd_ps(_mm256_hadd_ps(s4, s5), _mm256_hadd_ps(s6, s7));
  const __m128 lo = _mm_add_ps(_mm256_castps256_ps128(a0123), _mm256_extractf128_ps(a0123, 1));
  const __m128 hi = _mm_add_ps(_mm256_castps256_ps128(a4567), _mm256_extractf128_ps(a4567, 1));
  return _mm256_insertf128_ps(_mm256_castps128_ps256(lo), hi, 1);
}

// y[0..hd) += a * x[0..hd)
inline void axpy(float a, const float* x, float* y, int hd) {
  const __m256 va = _mm256_set1_ps(a);
  for (int d = 0; d < hd; d += 8) _mm256_storeu_ps(y + d, _mm256_fmadd_ps(va, _mm256_loadu_ps(x + d), _mm256_loadu_ps(y + d)));
}

// y[0..hd) += sum over t < 8 of a[t] * x_t[0..hd), rows x_t = x + t * ldx: one load and one store of y
// per eight multiply-adds instead of per one
inline void axpy8(const float* a, const float* x, int64_t ldx, float* y, int hd) {
  const __m256 a0 = _mm256_broadcast_ss(a + 0), a1 = _mm256_broadcast_ss(a + 1), a2 = _mm256_broadcast_ss(a + 2),
               a3 = _mm256_broadcast_ss(a + 3), a4 = _mm256_broadcast_ss(a + 4), a5 = _mm256_broadcast_ss(a + 5),
               a6 = _mm256_broadcast_ss(a + 6), a7 = _mm256_broadcast_ss(a + 7);
  for (int d = 0; d < hd; d += 8) {
    __m256 acc = _mm256_loadu_ps(y + d);
    __m256 acc2 = _mm256_mul_ps(a1, _mm256_loadu_ps(x + 1 * ldx + d));
    acc = _mm256_fmadd_ps(a0, _mm256_loadu_ps(x + 0 * ldx + d), acc);
    acc2 = _mm256_fmadd_ps(a3, _mm256_loadu_ps(x + 3 * ldx + d), acc2);
    acc = _mm256_fmadd_ps(a2, _mm256_loadu_ps(x + 2 * ldx + d), acc);
    acc2 = _mm256_fmadd_ps(a5, _mm256_loadu_ps(x + 5 * ldx + d), acc2);
    acc = _mm256_fmadd_ps(a4, _mm256_loadu_ps(x + 4 * ldx + d), acc);
    acc2 = _mm256_fmadd_ps(a7, _mm256_loadu_ps(x + 7 * ldx + d), acc2);
    acc = _mm256_fmadd_ps(a6, _mm256_loadu_ps(x + 6 * ldx + d), acc);
    _mm256_storeu_ps(y + d, _mm256_add_ps(acc, acc2));
  }
}

// exp(s[j] * 1 - m) in place over [0, n), returns the sum; n need not be a multiple of 8 (the buffer is)
inline float exp_rows(float* s, int n, float m) {
  const __m256 vm = _mm256_set1_ps(m);
  __m256 acc = _mm256_setzero_ps();
  int j = 0;
  for (; j + 8 <= n; j += 8) {
    const __m256 e = exp256(_mm256_sub_ps(_mm256_loadu_ps(s + j), vm));
    _mm256_storeu_ps(s + j, e);
    acc = _mm256_add_ps(acc, e);
  }
  float sum = hsum(acc);
  if (j < n) {
    alignas(32) float t[8];
    for (int q = 0; q < 8; ++q) t[q] = j + q < n ? s[j + q] - m : -100.0f;
    _mm256_store_ps(t, exp256(_mm256_load_ps(t)));
    for (int q = 0; j + q < n; ++q) {
      s[j + q] = t[q];
      sum += t[q];
    }
  }
  return sum;
}

template <typename F>
void parallel_tasks(int n, int threads, F fn) {
  threads = std::max(1, std::min(threads, n));
  if (threads == 1) {
    for (int i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<int> next{0};
  auto work = [&] {
    for (int i; (i = next.fetch_add(1, std::memory_order_relaxed)) < n;) fn(i);
  };
  std::vector<std::thread> pool;
  for (int t = 1; t < threads; ++t) pool.emplace_back(work);
  work();
  for (auto& th : pool) th.join();
}

struct Shape {
  int B, T, S, hq, hk, hd;
  float scale;
  int causal;
  int visible(int i) const { return causal ? std::min(S, i + (S - T) + 1) : S; }
};

constexpr int ROWS_PER_TASK = 32;   // query rows (dQ, forward) or keys (dK / dV) one task owns
constexpr int TILE = 64;            // rows of the other operand taken at a time: 64 x 128 floats are 32 KB

// scores of one query row against n (<= TILE) keys starting at kb, times scale; returns their maximum
inline float tile_scores(const float* qi, const float* kb, int64_t ldk, int n, int hd, float scale, float* sc) {
  const __m256 vscale = _mm256_set1_ps(scale);
  __m256 vmax = _mm256_set1_ps(-INFINITY);
  float m = -INFINITY;
  int j = 0;
  for (; j + 8 <= n; j += 8) {
    const __m256 s8 = _mm256_mul_ps(vscale, dot8(qi, kb + (int64_t)j * ldk, ldk, hd));
    _mm256_storeu_ps(sc + j, s8);
    vmax = _mm256_max_ps(vmax, s8);
  }
  if (j) {
    alignas(32) float t[8];
    _mm256_store_ps(t, vmax);
    for (int q8 = 0; q8 < 8; ++q8) m = std::max(m, t[q8]);
  }
  for (; j < n; ++j) {
    const float s = scale * dot(qi, kb + (int64_t)j * ldk, hd);
    sc[j] = s;
    m = std::max(m, s);
  }
  return m;
}

// y += sum_j a[j] * x_j over n rows
inline void rows_axpy(const float* a, const float* x, int64_t ldx, int n, float* y, int hd) {
  int j = 0;
  for (; j + 8 <= n; j += 8) axpy8(a + j, x + (int64_t)j * ldx, ldx, y, hd);
  for (; j < n; ++j) axpy(a[j], x + (int64_t)j * ldx, y, hd);
}

}  // namespace

// o [B*T, hq*hd], lse [B, hq, T].  Returns 0, or -1 for a head dimension this code does not take.
BBH_API int bbh_cpu_attn_fwd(const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv,
                             float* o, int64_t ldo, float* lse, int B, int T, int S, int hq, int hk, int hd,
                             float scale, int causal, int threads) {
  if (hd % 8 != 0 || hd <= 0 || hq % hk != 0) return -1;
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  const Shape sh{B, T, S, hq, hk, hd, scale, causal};
  const int g = hq / hk, blocks = (T + ROWS_PER_TASK - 1) / ROWS_PER_TASK;
  parallel_tasks(B * hq * blocks, threads, [&](int task) {
    const int blk = task % blocks, h = (task / blocks) % hq, b = task / (blocks * hq);
    const int hkv = h / g;
    const int i0 = blk * ROWS_PER_TASK, i1 = std::min(T, i0 + ROWS_PER_TASK);
    float m[ROWS_PER_TASK], l[ROWS_PER_TASK];
    for (int i = i0; i < i1; ++i) {
      m[i - i0] = -INFINITY;
      l[i - i0] = 0.f;
      std::memset(o + ((int64_t)b * T + i) * ldo + (int64_t)h * hd, 0, sizeof(float) * hd);
    }
    alignas(32) float sc[TILE];
    const int n_max = sh.visible(i1 - 1);   // the block's last row sees the most keys
    // a tile of keys (and of V rows) is used by every row of the block before the next one is
    // touched; the running maximum and sum of each row rescale what it has accumulated so far
    for (int j0 = 0; j0 < n_max; j0 += TILE) {
      const float* kb = k + ((int64_t)b * S + j0) * ldk + (int64_t)hkv * hd;
      const float* vb = v + ((int64_t)b * S + j0) * ldv + (int64_t)hkv * hd;
      for (int i = i0; i < i1; ++i) {
        const int n = std::min(sh.visible(i), j0 + TILE) - j0;
        if (n <= 0) continue;
        const int r = i - i0;
        const float* qi = q + ((int64_t)b * T + i) * ldq + (int64_t)h * hd;
        float* oi = o + ((int64_t)b * T + i) * ldo + (int64_t)h * hd;
        const float mt = tile_scores(qi, kb, ldk, n, hd, scale, sc);
        const float m_new = std::max(m[r], mt);
        const float alpha = m[r] == -INFINITY ? 0.f : std::exp(m[r] - m_new);
        l[r] = l[r] * alpha + exp_rows(sc, n, m_new);
        m[r] = m_new;
        if (alpha != 1.f) {
          const __m256 va = _mm256_set1_ps(alpha);
          for (int d = 0; d < hd; d += 8) _mm256_storeu_ps(oi + d, _mm256_mul_ps(va, _mm256_loadu_ps(oi + d)));
        }
        rows_axpy(sc, vb, ldv, n, oi, hd);
      }
    }
    for (int i = i0; i < i1; ++i) {
      const int r = i - i0;
      float* oi = o + ((int64_t)b * T + i) * ldo + (int64_t)h * hd;
      if (l[r] > 0.f) {
        const __m256 inv = _mm256_set1_ps(1.0f / l[r]);
        for (int d = 0; d < hd; d += 8) _mm256_storeu_ps(oi + d, _mm256_mul_ps(inv, _mm256_loadu_ps(oi + d)));
        lse[((int64_t)b * hq + h) * T + i] = m[r] + std::log(l[r]);
      } else {   // a query that sees no key: zero output, lse -inf
        lse[((int64_t)b * hq + h) * T + i] = -INFINITY;
      }
    }
  });
  return 0;
}

// dq [B*T, hq*hd], dk and dv [B*S, hk*hd]: all three are overwritten.
BBH_API int bbh_cpu_attn_bwd(const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv,
                             const float* o, int64_t ldo, const float* dout, int64_t lddo, const float* lse,
                             float* dq, int64_t lddq, float* dk, int64_t lddk, float* dv, int64_t lddv, int B, int T,
                             int S, int hq, int hk, int hd, float scale, int causal, int threads) {
  if (hd % 8 != 0 || hd <= 0 || hq % hk != 0) return -1;
  if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
  const Shape sh{B, T, S, hq, hk, hd, scale, causal};
  const int g = hq / hk;
  const __m256 vscale = _mm256_set1_ps(scale);
  // delta_i = dO_i . O_i, kept in a [B, hq, T] table both passes read
  std::vector<float> delta((size_t)B * hq * T);
  const int blocks = (T + ROWS_PER_TASK - 1) / ROWS_PER_TASK;
  // pass 1, one task per (sequence, query head, block of query rows): dQ.  Key tile by key tile, every
  // row of the block: scores and dO.V, probabilities from the saved log-sum-exp, dS, dQ_i += dS_ij K_j.
  parallel_tasks(B * hq * blocks, threads, [&](int task) {
    const int blk = task % blocks, h = (task / blocks) % hq, b = task / (blocks * hq);
    const int hkv = h / g;
    const int i0 = blk * ROWS_PER_TASK, i1 = std::min(T, i0 + ROWS_PER_TASK);
    for (int i = i0; i < i1; ++i) {
      const int64_t row = (int64_t)b * T + i;
      std::memset(dq + row * lddq + (int64_t)h * hd, 0, sizeof(float) * hd);
      delta[((size_t)b * hq + h) * T + i] = dot(dout + row * lddo + (int64_t)h * hd, o + row * ldo + (int64_t)h * hd, hd);
    }
    alignas(32) float p[TILE], dp[TILE];
    const int n_max = sh.visible(i1 - 1);
    for (int j0 = 0; j0 < n_max; j0 += TILE) {
      const float* kb = k + ((int64_t)b * S + j0) * ldk + (int64_t)hkv * hd;
      const float* vb = v + ((int64_t)b * S + j0) * ldv + (int64_t)hkv * hd;
      for (int i = i0; i < i1; ++i) {
        const int n = std::min(sh.visible(i), j0 + TILE) - j0;
        if (n <= 0) continue;
        const int64_t row = (int64_t)b * T + i;
        const float* qi = q + row * ldq + (int64_t)h * hd;
        const float* doi = dout + row * lddo + (int64_t)h * hd;
        const float l = lse[((int64_t)b * hq + h) * T + i];
        const float dl = delta[((size_t)b * hq + h) * T + i];
        tile_scores(qi, kb, ldk, n, hd, scale, p);
        int j = 0;
        for (; j + 8 <= n; j += 8) _mm256_storeu_ps(dp + j, dot8(doi, vb + (int64_t)j * ldv, ldv, hd));
        for (; j < n; ++j) dp[j] = dot(doi, vb + (int64_t)j * ldv, hd);
        exp_rows(p, n, l);   // probabilities: exp(score - lse)
        for (j = 0; j < n; ++j) p[j] = p[j] * (dp[j] - dl) * scale;   // dS
        rows_axpy(p, kb, ldk, n, dq + row * lddq + (int64_t)h * hd, hd);
      }
    }
  });
  // pass 2, one task per (sequence, KV head, block of keys): dK and dV.  Query-row tile by tile, every
  // key of the block and query head of the group: the same scores with the roles swapped (eight query
  // rows at a time), then dV_j += P_ij dO_i and dK_j += dS_ij Q_i into rows only this task writes.
  const int kblocks = (S + ROWS_PER_TASK - 1) / ROWS_PER_TASK;
  parallel_tasks(B * hk * kblocks, threads, [&](int task) {
    const int blk = task % kblocks, hkv = (task / kblocks) % hk, b = task / (kblocks * hk);
    const int j0 = blk * ROWS_PER_TASK, j1 = std::min(S, j0 + ROWS_PER_TASK);
    for (int j = j0; j < j1; ++j) {
      std::memset(dk + ((int64_t)b * S + j) * lddk + (int64_t)hkv * hd, 0, sizeof(float) * hd);
      std::memset(dv + ((int64_t)b * S + j) * lddv + (int64_t)hkv * hd, 0, sizeof(float) * hd);
    }
    alignas(32) float p[TILE + 8], ds[TILE + 8];
    // query rows that see key j: i >= j - (S - T) when causal, all rows otherwise
    const int first = causal ? std::max(0, j0 - (S - T)) : 0;
    for (int t0 = first; t0 < T; t0 += TILE) {
      for (int j = j0; j < j1; ++j) {
        const int a = std::max(t0, causal ? std::max(0, j - (S - T)) : 0), e = std::min(T, t0 + TILE);
        const int n = e - a;
        if (n <= 0) continue;
        const int64_t kr = (int64_t)b * S + j;
        const float* kj = k + kr * ldk + (int64_t)hkv * hd;
        const float* vj = v + kr * ldv + (int64_t)hkv * hd;
        float* dkj = dk + kr * lddk + (int64_t)hkv * hd;
        float* dvj = dv + kr * lddv + (int64_t)hkv * hd;
        for (int h = hkv * g; h < (hkv + 1) * g; ++h) {
          const float* qb = q + ((int64_t)b * T + a) * ldq + (int64_t)h * hd;
          const float* dob = dout + ((int64_t)b * T + a) * lddo + (int64_t)h * hd;
          const float* lrow = lse + ((int64_t)b * hq + h) * T + a;
          const float* drow = delta.data() + ((size_t)b * hq + h) * T + a;
          int i = 0;
          for (; i + 8 <= n; i += 8) {
            const __m256 s8 = _mm256_mul_ps(vscale, dot8(kj, qb + (int64_t)i * ldq, ldq, hd));
            const __m256 p8 = exp256(_mm256_sub_ps(s8, _mm256_loadu_ps(lrow + i)));
            const __m256 dp8 = dot8(vj, dob + (int64_t)i * lddo, lddo, hd);
            _mm256_storeu_ps(p + i, p8);
            _mm256_storeu_ps(ds + i, _mm256_mul_ps(_mm256_mul_ps(p8, _mm256_sub_ps(dp8, _mm256_loadu_ps(drow + i))), vscale));
          }
          for (; i < n; ++i) {
            const float sc1 = scale * dot(kj, qb + (int64_t)i * ldq, hd) - lrow[i];
            const float pi = sc1 < -87.0f ? 0.0f : std::exp(sc1);
            p[i] = pi;
            ds[i] = pi * (dot(vj, dob + (int64_t)i * lddo, hd) - drow[i]) * scale;
          }
          rows_axpy(p, dob, lddo, n, dvj, hd);
          rows_axpy(ds, qb, ldq, n, dkj, hd);
        }
      }
    }
  });
  return 0;
}
