"""Autotune cache (reference: crates/gpu-core/src/tune.rs and the ``AutoTuner`` of
crates/backend-api/src/select.rs:197-225 — time the variants of an op once per shape, remember the
winner on disk, fall back to the static selector when tuning is off).

Here the tunable is the GEMM tile width ``bn`` (0 = the launcher's own heuristic).  Tuning is off by
default; ``BRAIN_AUTOTUNE=1`` (or ``enable()``) turns it on and ``BRAIN_TUNE_CACHE`` names the JSON
cache file.  Keys carry the device name, so a cache written on one GPU model is ignored on another."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterable, Optional


class AutoTuner:
    def __init__(self, path: Optional[str] = None, device_name: str = "cpu",
                 timer: Optional[Callable[[Callable[[], None]], float]] = None):
        self.path = path
        self.device = device_name
        self.timer = timer or _cuda_timer
        self.table: Dict[str, int] = {}
        self.trials = 0
        if path and os.path.exists(path):
            try:
                self.table = {k: int(v) for k, v in json.loads(open(path).read()).items()}
            except (ValueError, OSError):
                self.table = {}

    def key(self, op: str, *dims) -> str:
        return f"{self.device}|{op}|" + "x".join(str(int(d)) for d in dims)

    def pick(self, key: str, candidates: Iterable[int], run: Callable[[int], None]) -> int:
        """The cached winner for ``key``, or time ``run(c)`` for every candidate (a candidate that
        raises is skipped) and remember the fastest."""
        hit = self.table.get(key)
        if hit is not None:
            return hit
        best, best_t = None, float("inf")
        for c in candidates:
            try:
                t = self.timer(lambda: run(c))
            except Exception:   # noqa: BLE001 - an unsupported variant is not a candidate
                continue
            self.trials += 1
            if t < best_t:
                best, best_t = c, t
        if best is None:
            raise RuntimeError(f"no candidate ran for {key}")
        self.table[key] = best
        self.save()
        return best

    def save(self) -> None:
        if not self.path:
            return
        tmp = self.path + ".tmp"
        os.makedirs(os.path.dirname(self.path) or ".", exist_ok=True)
        with open(tmp, "w") as f:
            f.write(json.dumps(self.table, indent=0, sort_keys=True))
        os.replace(tmp, self.path)


def _cuda_timer(fn: Callable[[], None], warmup: int = 2, iters: int = 5) -> float:
    import torch
    for _ in range(warmup):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


_TUNER: Optional[AutoTuner] = None


def enable(path: Optional[str] = None) -> AutoTuner:
    global _TUNER
    import torch
    name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    path = path or os.environ.get("BRAIN_TUNE_CACHE") or os.path.join(
        os.environ.get("XDG_CACHE_HOME") or os.path.join(os.environ.get("HOME", "."), ".cache"), "brain", "tune.json")
    _TUNER = AutoTuner(path, name)
    return _TUNER


def disable() -> None:
    global _TUNER
    _TUNER = None


def tuner() -> Optional[AutoTuner]:
    global _TUNER
    if _TUNER is None and os.environ.get("BRAIN_AUTOTUNE") == "1":
        enable()
    return _TUNER


GEMM_BN = (0, 64, 128, 256)

if os.environ.get("BRAIN_AUTOTUNE") == "1":
    try:
        enable()
    except Exception:   # noqa: BLE001 - tuning is an optimisation; never fail an import over it
        _TUNER = None
