// Host data runtime: SplitMix64 stream (bit-compatible with the reference's dataset RNG,
// crates/data/src/rng.rs:14-80) and the token-window batch sampler with target masking
// (crates/data/src/loader.rs:125-290).  C ABI, driven from brain_b200/data/loader.py.
#include <cstdint>
#include <cstring>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr uint64_t GOLDEN = 0x9E3779B97F4A7C15ull;
constexpr int32_t IGNORE = -1;

inline uint64_t splitmix_next(uint64_t& state) {
  state += GOLDEN;
  uint64_t z = state;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

inline int64_t range_inclusive(uint64_t& state, int64_t lo, int64_t hi) {
  const uint64_t span = static_cast<uint64_t>(hi - lo + 1);
  return lo + static_cast<int64_t>(splitmix_next(state) % span);
}

struct Dataset {
  std::vector<uint32_t> data;
  std::vector<uint8_t> mask;     // empty = every target supervised
  std::vector<float> weights;    // empty = 1.0
  std::vector<size_t> line_starts;
  bool aligned = false;
};

void line_starts_for(Dataset& ds, uint32_t newline, size_t block) {
  std::vector<size_t> nl;
  for (size_t i = 0; i < ds.data.size(); ++i)
    if (ds.data[i] == newline) nl.push_back(i);
  auto fits = [&](size_t s) { return s + block < ds.data.size(); };
  ds.line_starts.clear();
  if (fits(0) && (nl.empty() || nl.front() < block)) ds.line_starts.push_back(0);
  for (size_t i = 0; i + 1 < nl.size(); ++i) {
    const size_t s = nl[i] + 1, e = nl[i + 1];
    if (e - s < block && fits(s)) ds.line_starts.push_back(s);
  }
  if (!nl.empty()) {
    const size_t s = nl.back() + 1;
    if (fits(s)) ds.line_starts.push_back(s);
  }
}

}  // namespace

BBH_API uint64_t bbh_rng_seed(uint64_t seed) { return seed + GOLDEN; }
BBH_API uint64_t bbh_rng_next_u64(uint64_t* state) { return splitmix_next(*state); }
BBH_API double bbh_rng_next_f64(uint64_t* state) {
  return static_cast<double>(splitmix_next(*state) >> 11) / static_cast<double>(1ull << 53);
}
BBH_API void bbh_rng_fill_u64(uint64_t* state, uint64_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = splitmix_next(*state);
}
// Uniform token ids in [0, vocab) — the synthetic batches of the benchmarks.
BBH_API void bbh_rng_fill_tokens(uint64_t* state, int32_t* out, int64_t n, int64_t vocab) {
  for (int64_t i = 0; i < n; ++i)
    out[i] = static_cast<int32_t>(range_inclusive(*state, 0, vocab - 1));
}

BBH_API void* bbh_dataset_new(const uint32_t* data, int64_t n, const uint8_t* mask,
                              const float* weights) {
  auto* ds = new Dataset();
  ds->data.assign(data, data + n);
  if (mask) ds->mask.assign(mask, mask + n);
  if (weights) ds->weights.assign(weights, weights + n);
  return ds;
}
BBH_API void bbh_dataset_free(void* h) { delete static_cast<Dataset*>(h); }
BBH_API int64_t bbh_dataset_len(void* h) { return static_cast<Dataset*>(h)->data.size(); }
BBH_API int64_t bbh_dataset_align(void* h, uint32_t newline, int64_t block) {
  auto* ds = static_cast<Dataset*>(h);
  line_starts_for(*ds, newline, static_cast<size_t>(block));
  ds->aligned = true;
  return static_cast<int64_t>(ds->line_starts.size());
}

// Draw `batch` windows of `block` tokens. y = next-token targets, IGNORE (-1) where masked.
// mask_before < 0 disables prompt masking; newline < 0 = no newline token.
// Returns 0, or -1 when the dataset is shorter than block+1.
BBH_API int bbh_dataset_get_batch(void* h, uint64_t* rng_state, int64_t batch, int64_t block,
                                  int64_t mask_before, int mask_per_line, int64_t newline,
                                  int32_t* x, int32_t* y, float* w, int64_t* starts_out) {
  auto* ds = static_cast<Dataset*>(h);
  const int64_t n = static_cast<int64_t>(ds->data.size());
  if (n < block + 1) return -1;
  for (int64_t b = 0; b < batch; ++b) {
    size_t start;
    if (ds->aligned && !ds->line_starts.empty())
      start = ds->line_starts[range_inclusive(*rng_state, 0,
                                              static_cast<int64_t>(ds->line_starts.size()) - 1)];
    else
      start = static_cast<size_t>(range_inclusive(*rng_state, 0, n - block - 1));
    if (starts_out) starts_out[b] = static_cast<int64_t>(start);
    for (int64_t t = 0; t < block; ++t) {
      x[b * block + t] = static_cast<int32_t>(ds->data[start + t]);
      y[b * block + t] = static_cast<int32_t>(ds->data[start + 1 + t]);
      if (w) w[b * block + t] = ds->weights.empty() ? 1.0f : ds->weights[start + 1 + t];
    }
    int32_t* row = y + b * block;
    if (mask_before >= 0) {
      const int32_t mt = static_cast<int32_t>(mask_before);
      if (mask_per_line) {
        int64_t line_start = 0;
        for (int64_t pos = 0; pos < block; ++pos) {
          const int32_t v = row[pos];
          if (v == mt)
            for (int64_t i = line_start; i <= pos; ++i) row[i] = IGNORE;
          if (newline >= 0 && v == static_cast<int32_t>(newline)) line_start = pos + 1;
        }
      } else {
        for (int64_t pos = 0; pos < block; ++pos)
          if (row[pos] == mt) {
            for (int64_t i = 0; i <= pos; ++i) row[i] = IGNORE;
            break;
          }
      }
    }
    if (!ds->mask.empty())
      for (int64_t t = 0; t < block; ++t)
        if (!ds->mask[start + 1 + t]) row[t] = IGNORE;
  }
  return 0;
}
