// Host-resident AdamW for optimiser-state offload: fp32 master weights and both moments live in
// pinned host memory, the device only holds bf16 working weights and the gradient bucket.
// Reference behaviour: crates/optim/src/lib.rs (OffloadAdam: moments in host RAM, the step runs on
// the CPU, updated weights are uploaded) — here the update is split over std::thread workers and
// writes the bf16 copy that is uploaded in the same pass.
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

// sum of squares in double, deterministic for a fixed thread count (fixed chunking + ordered sum)
BBH_API double bbh_sumsq_f32(const float* g, int64_t n, int threads) {
    if (threads < 1) threads = 1;
    std::vector<double> part(size_t(threads), 0.0);
    int64_t chunk = (n + threads - 1) / threads;
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) {
        int64_t a = t * chunk, b = std::min<int64_t>(n, a + chunk);
        if (a >= b) break;
        pool.emplace_back([=, &part] {
            double s = 0.0;
            for (int64_t i = a; i < b; ++i) s += double(g[i]) * double(g[i]);
            part[size_t(t)] = s;
        });
    }
    for (auto& th : pool) th.join();
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
