// Parallelism planners and the pipeline schedule generator (host side, C ABI).
//   bbh_plan_balanced   exact min-max partition of L layers into k contiguous stages with embed /
//                       head costs on the first / last stage (dynamic programme)
//   bbh_plan_by_capacity fewest stages such that every stage's bytes fit its device
//   bbh_tp_step_secs    analytic step time of tensor parallel degree t (two reductions per layer)
//   bbh_plan_tp         smallest degree dividing n_gpus whose state fits
//   bbh_schedule_1f1b   per-stage op list of the one-forward-one-backward pipeline schedule
//   bbh_schedule_gpipe  all-forward-then-all-backward (the reference's schedule)
// Reference: crates/model/src/shard.rs:138-184 (plan_balanced), :265-343 (capacity planners),
// :551-642 (GPipe), crates/model/src/plan.rs:68-127.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

// bounds_out: k+1 layer boundaries (stage s owns [bounds[s], bounds[s+1])).
BBH_API int bbh_plan_balanced(int n_layers, int k, double per_layer, double embed, double head,
                              int* bounds_out) {
  if (k < 1 || n_layers < 0) return -1;
  const int L = n_layers;
  auto stage_cost = [&](int a, int b, int s) {
    double c = per_layer * (b - a);
    if (s == 0) c += embed;
    if (s == k - 1) c += head;
    return c;
  };
  if (k == 1) {
    bounds_out[0] = 0;
    bounds_out[1] = L;
    return 0;
  }
  const double inf = std::numeric_limits<double>::infinity();
  std::vector<std::vector<double>> best(k, std::vector<double>(L + 1, inf));
  std::vector<std::vector<int>> cut(k, std::vector<int>(L + 1, 0));
  for (int i = 0; i <= L; ++i) best[0][i] = stage_cost(0, i, 0);
  for (int s = 1; s < k; ++s)
    for (int i = 0; i <= L; ++i)
      for (int j = 0; j <= i; ++j) {
        const double cand = std::max(best[s - 1][j], stage_cost(j, i, s));
        if (cand < best[s][i]) {
          best[s][i] = cand;
          cut[s][i] = j;
        }
      }
  bounds_out[k] = L;
  int i = L;
  for (int s = k - 1; s >= 1; --s) {
    bounds_out[s] = cut[s][i];
    i = bounds_out[s];
  }
  bounds_out[0] = 0;
  return 0;
}

// Greedy capacity fill: returns the number of stages used (<= n_devices) or -1 when it cannot fit.
BBH_API int bbh_plan_by_capacity(int n_layers, double layer_bytes, double embed_bytes,
                                 double head_bytes, const double* capacity, int n_devices,
                                 int* bounds_out) {
  int layer = 0, stage = 0;
  bounds_out[0] = 0;
  for (; stage < n_devices && layer < n_layers; ++stage) {
    double used = stage == 0 ? embed_bytes : 0.0;
    int start = layer;
    while (layer < n_layers) {
      double need = used + layer_bytes;
      if (layer == n_layers - 1) need += head_bytes;
      if (need > capacity[stage]) break;
      used += layer_bytes;
      ++layer;
    }
    if (layer == start && !(start == n_layers)) {
      if (stage == n_devices - 1 || layer_bytes > capacity[stage]) return -1;
    }
    bounds_out[stage + 1] = layer;
  }
  return layer == n_layers ? stage : -1;
}

BBH_API double bbh_tp_step_secs(double tokens, double d_model, double d_ff, double n_layers, int t,
                                double peak_flops, double link_bytes_per_s, double link_latency_s,
                                double gemm_min_dim, double bytes_per_elem) {
  const double layer_flops = 2.0 * (2.0 * tokens * d_model * d_ff) + 4.0 * (2.0 * tokens * d_model * d_model);
  const double local_dim = std::min(d_ff, d_model) / t;
  const double eff = local_dim >= gemm_min_dim ? 1.0 : std::max(local_dim / gemm_min_dim, 1e-3);
  const double t_local = n_layers * layer_flops / t / (peak_flops * eff);
  const double msg = tokens * d_model * bytes_per_elem;
  // through NVSwitch every peer is one hop away: a reduce-scatter + all-gather pair moves
  // 2 (t-1)/t of the message per GPU, as a ring does, but with one latency term per collective
  const double t_comm = t <= 1 ? 0.0
                               : n_layers * 2.0 * (2.0 * (t - 1.0) / t * msg / link_bytes_per_s + link_latency_s);
  return 2.0 * (t_local + t_comm);
}

// Returns the chosen degree; *fits_out = 0 when even the largest degree does not fit.
BBH_API int bbh_plan_tp(int n_gpus, double mem_bytes, double state_bytes, double act_bytes, int* fits_out) {
  int last = 1;
  for (int t = 1; t <= n_gpus; ++t) {
    if (n_gpus % t) continue;
    last = t;
    if (state_bytes / t + act_bytes <= mem_bytes) {
      *fits_out = 1;
      return t;
    }
  }
  *fits_out = 0;
  return last;
}

// Ops: +m+1 = forward of micro-batch m, -(m+1) = backward of micro-batch m.  Returns the number of
// ops written (2*n_micro).  1F1B: min(pp-stage-1, n_micro) warm-up forwards, then alternate.
BBH_API int bbh_schedule_1f1b(int stage, int pp, int n_micro, int* ops_out) {
  if (stage < 0 || stage >= pp || n_micro < 1) return -1;
  const int warm = std::min(pp - stage - 1, n_micro);
  int n = 0, f = 0, b = 0;
  for (int i = 0; i < warm; ++i) ops_out[n++] = ++f;
  while (f < n_micro) {
    ops_out[n++] = ++f;
    ops_out[n++] = -(++b);
  }
  while (b < n_micro) ops_out[n++] = -(++b);
  return n;
}

BBH_API int bbh_schedule_gpipe(int stage, int pp, int n_micro, int* ops_out) {
  (void)stage;
  (void)pp;
  int n = 0;
  for (int m = 1; m <= n_micro; ++m) ops_out[n++] = m;
  for (int m = n_micro; m >= 1; --m) ops_out[n++] = -m;
  return n;
}
