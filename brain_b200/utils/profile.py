"""Per-kernel device timing and the ``% of measured roof`` table (reference:
crates/backend-api/src/lib.rs:696-908 ``set_kernel_timing``/``kernel_times`` — a timestamp pair per
dispatch; crates/gpu-core/src/profile.rs:385 ``profile`` prints kernel, time, GFLOP/s, GB/s, bound,
% of roof and flags rates above ``IMPOSSIBLE_PCT`` (:55,194) as measurement bugs; ``BRAIN_PROFILE=1``
turns on ``stage_time`` (:338) and a dump at exit).

Timing brackets each native launch with CUDA events on the launching stream, so it serialises
nothing but adds two event records per launch; it is a diagnosis mode, never a benchmark mode."""
from __future__ import annotations

import atexit
import os
from collections import defaultdict
from typing import Callable, Dict, List, Optional

import torch

from ..ops import _cuda
from . import cost as costs

IMPOSSIBLE_PCT = 105.0

_records: List = []
_orig_call = None
_stages: Dict[str, float] = defaultdict(float)


def _decode(name: str, args) -> Optional[costs.OpCost]:
    try:
        if name == "gemm_bf16":
            out = args[2]
            return costs.kernel_cost(name, M=args[4], N=args[5], K=args[6],
                                     es_out=out.element_size() if isinstance(out, torch.Tensor) else 2)
        if name == "gemm_i8":
            return costs.kernel_cost(name, M=args[5], N=args[6], K=args[7])
        if name in ("flash_fwd", "flash_bwd"):
            tail = [a for a in args if isinstance(a, (int, float)) and not isinstance(a, bool)]
            B, T, S, hq, hk, hd = [int(x) for x in tail[-8:-2]]
            return costs.kernel_cost(name, B=B, T=T, S=S, hq=hq, hk=hk, hd=hd, causal=bool(tail[-1]))
    except Exception:
        pass
    by = sum(a.numel() * a.element_size() for a in args if isinstance(a, torch.Tensor))
    return costs.OpCost(0.0, 0.0, float(by)) if by else None


def set_kernel_timing(on: bool) -> None:
    global _orig_call
    if on and _orig_call is None:
        _orig_call = _cuda.call

        def timed(name, *args):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _orig_call(name, *args)
            e1.record()
            _records.append((name, e0, e1, _decode(name, args)))

        _cuda.call = timed
        _rebind(timed)
    elif not on and _orig_call is not None:
        _cuda.call = _orig_call
        _rebind(_orig_call)
        _orig_call = None


def _rebind(fn) -> None:
    """Modules that did ``from ._cuda import call`` hold their own reference: repoint them."""
    import sys
    for mod in list(sys.modules.values()):
        name = getattr(mod, "__name__", "") or ""
        if name.startswith("brain_b200.") and getattr(mod, "call", None) is not None and mod is not _cuda:
            if getattr(mod.call, "__module__", "").startswith("brain_b200"):
                mod.call = fn


def kernel_times(reset: bool = True) -> Dict[str, Dict]:
    torch.cuda.synchronize()
    agg: Dict[str, Dict] = {}
    for name, e0, e1, c in _records:
        a = agg.setdefault(name, {"n": 0, "ms": 0.0, "flops": 0.0, "int_ops": 0.0, "bytes": 0.0, "uncosted": 0})
        a["n"] += 1
        a["ms"] += e0.elapsed_time(e1)
        if c is None:
            a["uncosted"] += 1
        else:
            a["flops"] += c.flops
            a["int_ops"] += c.int_ops
            a["bytes"] += c.bytes
    if reset:
        _records.clear()
    return agg


def render(agg: Dict[str, Dict], label: str = "", roof=None) -> str:
    if roof is None:
        from .roof import measure
        try:
            roof = measure()
        except Exception:
            roof = None
    tot = sum(a["ms"] for a in agg.values()) or 1e-9
    lines = [f"---- profile {label} ----",
             f"{'kernel':<24} {'n':>6} {'ms':>10} {'%':>6} {'TFLOP/s':>9} {'GB/s':>9} {'bound':>8} {'%roof':>7}"]
    for name, a in sorted(agg.items(), key=lambda kv: -kv[1]["ms"]):
        s = a["ms"] * 1e-3
        tf = (a["flops"] + a["int_ops"]) / s / 1e12 if s else 0.0
        gb = a["bytes"] / s / 1e9 if s else 0.0
        bound, pct = "-", float("nan")
        if roof is not None and (a["flops"] or a["bytes"] or a["int_ops"]):
            bound = roof.bound(a["flops"], a["bytes"], a["int_ops"])
            pct = 100.0 * roof.min_seconds(a["flops"], a["bytes"], a["int_ops"]) / s if s else 0.0
        flag = "  <-- above the measured roof: timing or cost bug" if pct == pct and pct > IMPOSSIBLE_PCT else ""
        lines.append(f"{name:<24} {a['n']:>6} {a['ms']:>10.3f} {100 * a['ms'] / tot:>6.1f} {tf:>9.1f} {gb:>9.0f} "
                     f"{bound:>8} {pct:>7.1f}{flag}")
    lines.append(f"{'total':<24} {sum(a['n'] for a in agg.values()):>6} {tot:>10.3f}")
    if roof is not None:
        lines.append(f"roof: HBM {roof.hbm_gbs:.0f} GB/s, bf16 {roof.bf16_tflops:.0f} TFLOP/s ({roof.source})")
    return "\n".join(lines)


def profile(label: str, step: Callable[[], None], steps: int = 3, warmup: int = 2) -> str:
    """Run ``step`` with kernel timing on and return the per-kernel table."""
    for _ in range(warmup):
        step()
    set_kernel_timing(True)
    try:
        for _ in range(steps):
            step()
        agg = kernel_times()
    finally:
        set_kernel_timing(False)
    return render(agg, f"{label} ({steps} steps)")


class stage_time:
    """``with stage_time('backward'):`` — host wall time per stage, summed (``BRAIN_PROFILE=1``)."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        import time
        self.t = time.perf_counter()

    def __exit__(self, *exc):
        import time
        if enabled():
            _stages[self.name] += time.perf_counter() - self.t
        return False


def enabled() -> bool:
    return os.environ.get("BRAIN_PROFILE") == "1"


def dump_profile(out=print) -> None:
    if _stages:
        out("---- stage times ----")
        for k, v in sorted(_stages.items(), key=lambda kv: -kv[1]):
            out(f"{k:<24} {v * 1e3:>10.1f} ms")
    if _records:
        out(render(kernel_times(), "at exit"))


if enabled():
    atexit.register(dump_profile)
