// Host-resident AdamW for optimiser-state offload: fp32 master weights and both moments live in
// pinned host memory, the device only holds bf16 working weights and the gradient bucket.
// Reference behaviour: crates/optim/src/lib.rs (OffloadAdam: moments in host RAM, the step runs on
// the CPU, updated weights are uploaded) — here the update is split over std::thread workers and
// writes the bf16 copy that is uploaded in the same pass.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);   // NaN stays NaN
    u += 0x7fffu + ((u >> 16) & 1u);                                          // round to nearest even
    return uint16_t(u >> 16);
}

template <class F>
void parallel_for(int64_t n, int threads, F&& fn) {
    if (threads <= 1 || n < (1 << 16)) { fn(0, n); return; }
    std::vector<std::thread> pool;
    int64_t chunk = (n + threads - 1) / threads;
    chunk = (chunk + 15) & ~int64_t(15);
    for (int t = 0; t < threads; ++t) {
        int64_t a = t * chunk, b = std::min<int64_t>(n, a + chunk);
        if (a >= b) break;
        pool.emplace_back([=, &fn] { fn(a, b); });
    }
    for (auto& th : pool) th.join();
}

}  // namespace

// sum of squares in double.  The vector is cut into fixed pieces of 2^18 elements whose partial sums
// are added in index order, so the result does not depend on the number of threads.
BBH_API double bbh_sumsq_f32(const float* g, int64_t n, int threads) {
    if (threads < 1) threads = 1;
    constexpr int64_t PIECE = int64_t(1) << 18;
    const int64_t pieces = (n + PIECE - 1) / PIECE;
    if (pieces <= 0) return 0.0;
    std::vector<double> part(size_t(pieces), 0.0);
    auto run = [&](int64_t first, int64_t step) {
        for (int64_t p = first; p < pieces; p += step) {
            const int64_t a = p * PIECE, b = std::min<int64_t>(n, a + PIECE);
            double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
            int64_t i = a;
            for (; i + 4 <= b; i += 4) {
                s0 += double(g[i]) * double(g[i]);
                s1 += double(g[i + 1]) * double(g[i + 1]);
                s2 += double(g[i + 2]) * double(g[i + 2]);
                s3 += double(g[i + 3]) * double(g[i + 3]);
            }
            for (; i < b; ++i) s0 += double(g[i]) * double(g[i]);
            part[size_t(p)] = (s0 + s1) + (s2 + s3);
        }
    };
    const int64_t nt = std::min<int64_t>(threads, pieces);
    if (nt <= 1) {
        run(0, 1);
    } else {
        std::vector<std::thread> pool;
        for (int64_t t = 0; t < nt; ++t) pool.emplace_back(run, t, nt);
        for (auto& th : pool) th.join();
    }
    double s = 0.0;
    for (double p : part) s += p;
    return s;
}

// One AdamW step over [0, n): g is scaled by coef first; decoupled weight decay; bias correction
// by step t (1-based).  w16 (optional) receives the bf16 rounding of the new master weights.
BBH_API void bbh_adamw_f32(float* master, float* m, float* v, const float* g, uint16_t* w16, int64_t n,
                   float lr, float b1, float b2, float eps, float wd, int64_t t, float coef,
                   int threads) {
    const double bc1 = 1.0 - std::pow(double(b1), double(t));
    const double bc2 = 1.0 - std::pow(double(b2), double(t));
    const float inv_bc1 = float(1.0 / bc1), inv_bc2 = float(1.0 / bc2);
    parallel_for(n, threads, [=](int64_t a, int64_t b) {
        for (int64_t i = a; i < b; ++i) {
            float gi = g[i] * coef;
            float mi = b1 * m[i] + (1.0f - b1) * gi;
            float vi = b2 * v[i] + (1.0f - b2) * gi * gi;
            m[i] = mi;
            v[i] = vi;
            float w = master[i];
            w -= lr * (mi * inv_bc1 / (std::sqrt(vi * inv_bc2) + eps) + wd * w);
            master[i] = w;
            if (w16) w16[i] = f32_to_bf16(w);
        }
    });
}
