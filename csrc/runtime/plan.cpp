// Parallelism planners and the pipeline schedule generator (host side, C ABI).
//
//   bbh_plan_stages      contiguous pipeline stages over MEASURED per-layer costs (one number per
//                        layer, e.g. milliseconds from a profiled step) plus the embedding on the
//                        first and the head on the last stage.  Minimises the slowest stage by a
//                        parametric search: "can the layers be packed into k stages of cost <= B"
//                        is a greedy linear scan, and B is bisected between the heaviest single
//                        item and the total.  O(L log(1/eps)) instead of a k x L x L table.  Slack
//                        is pushed towards the FIRST stages (the scan packs from the last layer
//                        backwards), because under a one-forward-one-backward schedule stage s
//                        keeps pp - s micro-batches of activations alive and is the one that runs
//                        out of memory first.
//   bbh_plan_balanced    the same with one cost for every layer
//   bbh_plan_by_capacity fewest stages such that every stage's bytes fit its device
//   bbh_tp_step_secs     step-time model of tensor parallel degree t on an NVSwitch fabric
//   bbh_plan_tp          degree that fits and is predicted fastest
//   bbh_schedule_1f1b    per-stage op list of the one-forward-one-backward pipeline schedule
//   bbh_schedule_gpipe   all-forward-then-all-backward
//
// What the reference plans with (crates/model/src/shard.rs:138-184, :265-343, crates/model/src/plan.rs:68-127)
// is a uniform per-layer cost and a ring all-reduce term for PCIe peers; the cost model here is for
// a switch: every peer is one hop away at full per-GPU bandwidth and the fused GEMM+collective
// kernels hide the transfer behind the tiles of the same layer.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

// Pack layers L-1 .. 0 into stages k-1 .. 0, each of cost <= bound.  Returns false when more than
// k stages would be needed.  cuts[s] = first layer of stage s.
bool pack_from_the_back(const double* cost, int L, int k, double embed, double head, double bound,
                        int* cuts) {
  bound *= 1.0 + 1e-12;  // costs that add up to the bound exactly must fit
  int stage = k - 1;
  double used = head;  // the head lives on the last stage whatever else that stage holds
  if (used > bound) return false;
  cuts[k] = L;
  for (int l = L - 1; l >= 0; --l) {
    if (used + cost[l] > bound) {  // close this stage, the layer opens the one before it
      cuts[stage] = l + 1;
      if (--stage < 0 || cost[l] > bound) return false;
      used = 0.0;
    }
    used += cost[l];
  }
  // `stage` owns layer 0.  The embedding lives on stage 0: together with layer 0's stage when that
  // is stage 0, alone (stages below `stage` hold no layers) otherwise.
  if ((stage == 0 ? used + embed : embed) > bound) return false;
  for (int s = stage; s >= 0; --s) cuts[s] = 0;
  return true;
}

}  // namespace

// bounds_out: k+1 layer boundaries (stage s owns [bounds[s], bounds[s+1])).
BBH_API int bbh_plan_stages(const double* layer_cost, int n_layers, int k, double embed, double head,
                            int* bounds_out) {
  if (k < 1 || n_layers < 0) return -1;
  const int L = n_layers;
  double total = embed + head, heaviest = std::max(embed, head);
  for (int l = 0; l < L; ++l) {
    if (!(layer_cost[l] >= 0.0)) return -1;
    total += layer_cost[l];
    heaviest = std::max(heaviest, layer_cost[l]);
  }
  std::vector<int> cuts(k + 1, 0), best(k + 1, 0);
  double lo = std::max(heaviest, total / k), hi = total;
  if (!pack_from_the_back(layer_cost, L, k, embed, head, hi, best.data())) return -1;
  if (pack_from_the_back(layer_cost, L, k, embed, head, lo, cuts.data())) {
    best = cuts;
  } else {
    for (int iter = 0; iter < 64 && hi - lo > 1e-12 * total; ++iter) {
      const double mid = 0.5 * (lo + hi);
      if (pack_from_the_back(layer_cost, L, k, embed, head, mid, cuts.data())) {
        hi = mid;
        best = cuts;
      } else {
        lo = mid;
      }
    }
  }
  for (int s = 0; s <= k; ++s) bounds_out[s] = best[s];
  return 0;
}

BBH_API int bbh_plan_balanced(int n_layers, int k, double per_layer, double embed, double head,
                              int* bounds_out) {
  if (n_layers < 0) return -1;
  std::vector<double> c(static_cast<size_t>(n_layers), per_layer);
  return bbh_plan_stages(c.data(), n_layers, k, embed, head, bounds_out);
}

// Capacity-first placement: walk the devices in order and give each as many whole layers as its
// bytes allow (embedding bytes on the first, head bytes with the last layer).  Returns the number of
// stages used (<= n_devices) or -1 when the model does not fit.
BBH_API int bbh_plan_by_capacity(int n_layers, double layer_bytes, double embed_bytes,
                                 double head_bytes, const double* capacity, int n_devices,
                                 int* bounds_out) {
  if (n_layers < 0 || n_devices < 1) return -1;
  int next = 0;  // first layer not placed yet
  bounds_out[0] = 0;
  for (int d = 0; d < n_devices; ++d) {
    double room = capacity[d] - (d == 0 ? embed_bytes : 0.0);
    int take = 0;
    while (next + take < n_layers) {
      const bool is_last = next + take == n_layers - 1;
      const double need = layer_bytes + (is_last ? head_bytes : 0.0);
      if (need > room) break;
      room -= need;
      ++take;
    }
    next += take;
    bounds_out[d + 1] = next;
    if (next == n_layers) return d + 1;
    if (take == 0 && d > 0) return -1;  // a later device that cannot hold even one layer
  }
  return -1;
}

// Step time (forward + backward) of a dense transformer at tensor-parallel degree t on a switch.
//   compute  per layer 6 GEMMs' worth of FLOPs split t ways; GEMMs whose local dimension falls
//            below `gemm_min_dim` lose efficiency in proportion (they no longer fill a 128 x 256 tile
//            grid over all SMs)
//   comm     per layer and pass one reduce-scatter and one all-gather of the [tokens, d_model]
//            activation: each moves (t-1)/t of the message through this GPU's own links, one hop,
//            at the measured peer bandwidth
//   overlap  the fused kernels move tile k+1 while tile k multiplies, so a layer costs
//            max(compute, comm) plus the part of the transfer that cannot be hidden: the first
//            tile's rows and one launch latency per collective
BBH_API double bbh_tp_step_secs(double tokens, double d_model, double d_ff, double n_layers, int t,
                                double peak_flops, double link_bytes_per_s, double link_latency_s,
                                double gemm_min_dim, double bytes_per_elem) {
  if (t < 1) t = 1;
  const double flops = 2.0 * tokens * (3.0 * d_model * d_ff + 4.0 * d_model * d_model);
  const double local = std::min(d_ff, d_model) / t;
  const double eff = local >= gemm_min_dim ? 1.0 : std::max(local / gemm_min_dim, 1e-3);
  const double compute = flops / t / (peak_flops * eff);
  double layer = compute;
  if (t > 1) {
    const double msg = tokens * d_model * bytes_per_elem;
    const double wire = 2.0 * (t - 1.0) / t * msg / link_bytes_per_s;  // RS + AG of one pass
    const double tiles = std::max(tokens / 128.0, 1.0);
    const double exposed = wire / tiles + 2.0 * link_latency_s;
    layer = std::max(compute, wire) + exposed;
  }
  return 3.0 * n_layers * layer;  // backward costs twice the forward in both FLOPs and bytes
}

// Among the degrees that divide n_gpus and whose sharded state fits, the one with the smallest
// predicted step time when a cost model is supplied (tokens > 0), else the smallest that fits.
// *fits_out = 0 (and the largest degree is returned) when nothing fits.
BBH_API int bbh_plan_tp_model(int n_gpus, double mem_bytes, double state_bytes, double act_bytes,
                              double tokens, double d_model, double d_ff, double n_layers,
                              double peak_flops, double link_bytes_per_s, double link_latency_s,
                              double gemm_min_dim, int* fits_out) {
  int best = 0, largest = 1;
  double best_secs = std::numeric_limits<double>::infinity();
  for (int t = 1; t <= n_gpus; ++t) {
    if (n_gpus % t) continue;
    largest = t;
    if (state_bytes / t + act_bytes > mem_bytes) continue;
    if (tokens <= 0) {
      best = t;
      break;
    }
    const double secs = bbh_tp_step_secs(tokens, d_model, d_ff, n_layers, t, peak_flops,
                                         link_bytes_per_s, link_latency_s, gemm_min_dim, 2.0);
    if (secs < best_secs) {
      best_secs = secs;
      best = t;
    }
  }
  *fits_out = best != 0;
  return best ? best : largest;
}

BBH_API int bbh_plan_tp(int n_gpus, double mem_bytes, double state_bytes, double act_bytes, int* fits_out) {
  return bbh_plan_tp_model(n_gpus, mem_bytes, state_bytes, act_bytes, 0, 0, 0, 0, 0, 0, 0, 0, fits_out);
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
