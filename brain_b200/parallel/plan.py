"""Planners (native: csrc/runtime/plan.cpp): pipeline cuts over measured per-layer costs (parametric
search on the slowest stage, slack pushed to the early stages that hold the most activations under
1F1B), capacity-first stage packing, the tensor-parallel degree planner whose cost model is a switch
(one-hop reduce-scatter + all-gather at the measured per-GPU peer bandwidth, transfers hidden behind
the tiles of the fused kernels), and the pipeline schedules.  Reference: crates/model/src/shard.rs:64-184,
265-343; crates/model/src/plan.rs:26-127."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from .. import _host

c = ctypes
_host.register({
    "bbh_plan_balanced": (c.c_int, [c.c_int, c.c_int, c.c_double, c.c_double, c.c_double, c.c_void_p]),
    "bbh_plan_stages": (c.c_int, [c.c_void_p, c.c_int, c.c_int, c.c_double, c.c_double, c.c_void_p]),
    "bbh_plan_tp_model": (c.c_int, [c.c_int] + [c.c_double] * 11 + [c.POINTER(c.c_int)]),
    "bbh_plan_by_capacity": (c.c_int, [c.c_int, c.c_double, c.c_double, c.c_double, c.c_void_p, c.c_int, c.c_void_p]),
    "bbh_tp_step_secs": (c.c_double, [c.c_double] * 4 + [c.c_int] + [c.c_double] * 5),
    "bbh_plan_tp": (c.c_int, [c.c_int, c.c_double, c.c_double, c.c_double, c.POINTER(c.c_int)]),
    "bbh_schedule_1f1b": (c.c_int, [c.c_int, c.c_int, c.c_int, c.c_void_p]),
    "bbh_schedule_gpipe": (c.c_int, [c.c_int, c.c_int, c.c_int, c.c_void_p]),
})


@dataclass
class Shard:
    start: int
    end: int
    embed: bool
    head: bool
    gpu_index: int = -1

    def owns(self, l: int) -> bool:
        return self.start <= l < self.end

    def is_whole(self, n_layers: int) -> bool:
        return self.start == 0 and self.end == n_layers and self.embed and self.head


@dataclass
class ShardCost:
    n_layers: int
    per_layer: float
    embed: float
    head: float
    boundary_words: int = 0


def plan_balanced(cost: ShardCost, gpus: List[int]) -> List[Shard]:
    """Contiguous stages minimising the maximum stage cost (exact)."""
    k = len(gpus)
    b = np.zeros(k + 1, dtype=np.int32)
    if _host.lib().bbh_plan_balanced(cost.n_layers, k, cost.per_layer, cost.embed, cost.head,
                                     b.ctypes.data) != 0:
        raise ValueError("pipeline needs >= 1 stage")
    return [Shard(int(b[s]), int(b[s + 1]), s == 0, s == k - 1, gpus[s]) for s in range(k)]


def plan_stages(layer_costs, gpus: List[int], embed: float = 0.0, head: float = 0.0) -> List[Shard]:
    """Contiguous stages over per-layer costs (e.g. measured milliseconds per layer) minimising the
    slowest stage; ties leave the slack with the early stages."""
    k = len(gpus)
    lc = np.ascontiguousarray(np.asarray(layer_costs, dtype=np.float64))
    b = np.zeros(k + 1, dtype=np.int32)
    if _host.lib().bbh_plan_stages(lc.ctypes.data, lc.size, k, embed, head, b.ctypes.data) != 0:
        raise ValueError("bad pipeline plan arguments")
    return [Shard(int(b[s]), int(b[s + 1]), s == 0, s == k - 1, gpus[s]) for s in range(k)]


def measured_layer_costs(blocks, x, repeats: int = 3) -> List[float]:
    """Milliseconds of forward + backward per block, timed on the device the blocks live on
    (CUDA events; wall clock on the CPU backend).  Feed the result to :func:`plan_stages`."""
    import time
    import torch
    out = []
    for blk in blocks:
        xin = x.detach().clone().requires_grad_(True)
        best = float("inf")
        for _ in range(repeats):
            if xin.is_cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                y = blk(xin)
                y.backward(torch.ones_like(y))
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
            else:
                t0 = time.perf_counter()
                y = blk(xin)
                y.backward(torch.ones_like(y))
                best = min(best, (time.perf_counter() - t0) * 1e3)
            xin.grad = None
        out.append(best)
    return out


def plan_by_capacity(n_layers: int, layer_bytes: float, embed_bytes: float, head_bytes: float,
                     capacities: List[float]) -> Optional[List[Shard]]:
    """Fill devices in order until the model is placed; None when it cannot fit."""
    cap = np.asarray(capacities, dtype=np.float64)
    b = np.zeros(len(capacities) + 1, dtype=np.int32)
    k = _host.lib().bbh_plan_by_capacity(n_layers, layer_bytes, embed_bytes, head_bytes,
                                         cap.ctypes.data, len(capacities), b.ctypes.data)
    if k < 0:
        return None
    return [Shard(int(b[s]), int(b[s + 1]), s == 0, s == k - 1, s) for s in range(k)]


def plan_fewest_devices(n_layers, layer_bytes, embed_bytes, head_bytes, capacity: float,
                        max_devices: int) -> Optional[List[Shard]]:
    for k in range(1, max_devices + 1):
        p = plan_by_capacity(n_layers, layer_bytes, embed_bytes, head_bytes, [capacity] * k)
        if p is not None:
            return p
    return None


@dataclass
class Hardware:
    """Defaults: one B200 of this pool (measured cuBLAS bf16 burst, NVLink peer copy per direction)."""
    n_gpus: int = 8
    mem_bytes: float = 180e9
    peak_flops: float = 1.4e15
    link_bytes_per_s: float = 770e9
    link_latency_s: float = 8e-6
    gemm_min_dim: int = 256


@dataclass
class ModelShape:
    tokens: int
    d_model: int
    d_ff: int
    n_layers: int
    state_bytes: float
    act_bytes: float


@dataclass
class TpPlan:
    degree: int
    predicted_secs: float
    fits: bool
    note: str


def tp_step_secs(hw: Hardware, s: ModelShape, t: int, bytes_per_elem: float = 2.0) -> float:
    return float(_host.lib().bbh_tp_step_secs(s.tokens, s.d_model, s.d_ff, s.n_layers, t, hw.peak_flops,
                                              hw.link_bytes_per_s, hw.link_latency_s, hw.gemm_min_dim,
                                              bytes_per_elem))


def plan_tp(hw: Hardware, s: ModelShape, fastest: bool = False) -> TpPlan:
    """Capacity first: the smallest degree dividing n_gpus whose sharded state fits; with
    ``fastest`` the fitting degree with the smallest predicted step time instead."""
    fits = c.c_int(0)
    if fastest:
        t = _host.lib().bbh_plan_tp_model(hw.n_gpus, hw.mem_bytes, s.state_bytes, s.act_bytes, s.tokens,
                                          s.d_model, s.d_ff, s.n_layers, hw.peak_flops, hw.link_bytes_per_s,
                                          hw.link_latency_s, hw.gemm_min_dim, c.byref(fits))
    else:
        t = _host.lib().bbh_plan_tp(hw.n_gpus, hw.mem_bytes, s.state_bytes, s.act_bytes, c.byref(fits))
    secs = tp_step_secs(hw, s, t)
    if not fits.value:
        return TpPlan(t, secs, False, "model does not fit even at max TP")
    if t == 1:
        note = "fits on one GPU; no tensor parallelism needed"
    elif min(s.d_ff, s.d_model) // t < hw.gemm_min_dim:
        note = "TP forced by memory, and it shrinks local GEMMs below the efficient tile"
    else:
        note = "smallest TP that fits, keeping local GEMMs large"
    return TpPlan(t, secs, True, note)


def schedule(kind: str, stage: int, pp: int, n_micro: int) -> List[int]:
    """Per-stage op list: +m+1 forward of micro-batch m, -(m+1) its backward."""
    out = np.zeros(2 * n_micro, dtype=np.int32)
    fn = _host.lib().bbh_schedule_1f1b if kind == "1f1b" else _host.lib().bbh_schedule_gpipe
    n = fn(stage, pp, n_micro, out.ctypes.data)
    if n < 0:
        raise ValueError("bad schedule arguments")
    return out[:n].tolist()
