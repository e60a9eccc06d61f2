"""Measured roofline (reference: crates/gpu-core/src/roof.rs:340 ``measure`` — probes run on the
device, cached per adapter (:510-568), time-boxed by ``BRAIN_ROOF_BUDGET_S`` (:223-227); a
spec-sheet peak is never used as a denominator).

Resolution order: a ``MEASURED_PEAKS.json`` next to the package or in the working directory (written
by whoever benchmarked this machine), then the per-device cache, then our own probes: a streaming
copy for HBM, the tcgen05 GEMM for bf16 and int8 tensor throughput."""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Optional

import torch

NVLINK_P2P_GBS_DEFAULT = 770.0       # measured peer copy per direction on NVLink 5 / NVSwitch


@dataclass
class Roof:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    i8_tops: float = 0.0
    nvlink_gbs: float = NVLINK_P2P_GBS_DEFAULT
    source: str = "probe"
    device: str = ""

    def bound(self, flops: float, bytes_: float, int_ops: float = 0.0) -> str:
        tc = flops / (self.bf16_tflops * 1e12) + (int_ops / (self.i8_tops * 1e12) if self.i8_tops else 0.0)
        tm = bytes_ / (self.hbm_gbs * 1e9)
        return "compute" if tc >= tm else "memory"

    def min_seconds(self, flops: float, bytes_: float, int_ops: float = 0.0, sustained: bool = False) -> float:
        peak = self.bf16_tflops_sustained if sustained else self.bf16_tflops
        tc = flops / (peak * 1e12) + (int_ops / (self.i8_tops * 1e12) if self.i8_tops else 0.0)
        return max(tc, bytes_ / (self.hbm_gbs * 1e9))


def _peaks_file() -> Optional[Path]:
    for p in (Path.cwd() / "MEASURED_PEAKS.json", Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"):
        if p.exists():
            return p
    return None


def _cache_path(device_name: str) -> Path:
    root = Path(os.environ.get("BRAIN_CACHE_DIR", Path.home() / ".cache" / "brain_b200"))
    return root / ("roof_" + "".join(c if c.isalnum() else "_" for c in device_name) + ".json")


def _time_events(fn, reps: int, budget_s: float) -> float:
    t_end = time.time() + budget_s
    fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e-3)
        if time.time() > t_end:
            break
    return best


def probe(budget_s: Optional[float] = None) -> Roof:
    """Run the probes on the current CUDA device (a few hundred MB, well under the time box)."""
    from ..ops import functional as F
    budget = float(os.environ.get("BRAIN_ROOF_BUDGET_S", budget_s or 6.0))
    dev = torch.device("cuda", torch.cuda.current_device())
    n = 512 << 20
    a = torch.empty(n, device=dev, dtype=torch.uint8)
    b = torch.empty_like(a)
    t = _time_events(lambda: b.copy_(a), 8, budget / 3)
    hbm = 2 * n / t / 1e9
    del a, b
    M = 8192
    x = torch.randn(M, M, device=dev, dtype=torch.bfloat16)
    w = torch.randn(M, M, device=dev, dtype=torch.bfloat16)
    t = _time_events(lambda: F.gemm(x, w), 8, budget / 3)
    bf16 = 2.0 * M ** 3 / t / 1e12
    xq = torch.randint(-127, 127, (M, M), device=dev, dtype=torch.int8)
    wq = torch.randint(-127, 127, (M, M), device=dev, dtype=torch.int8)
    sm = torch.ones(M, device=dev)
    t = _time_events(lambda: F.gemm_i8(xq, wq, sm, sm), 8, budget / 3)
    i8 = 2.0 * M ** 3 / t / 1e12
    return Roof(hbm, bf16, bf16 * 0.85, i8, probe_nvlink(budget / 3) or NVLINK_P2P_GBS_DEFAULT, source="probe",
                device=torch.cuda.get_device_name(dev))


def probe_nvlink(budget_s: float = 2.0) -> Optional[float]:
    """Peer-copy bandwidth (GB/s, one direction) from the current device to the next visible one,
    or None with fewer than two peer-accessible GPUs in this process."""
    if torch.cuda.device_count() < 2:
        return None
    src = torch.cuda.current_device()
    dst = (src + 1) % torch.cuda.device_count()
    if not torch.cuda.can_device_access_peer(src, dst):
        return None
    n = 256 << 20
    a = torch.empty(n, device=torch.device("cuda", src), dtype=torch.uint8)
    b = torch.empty(n, device=torch.device("cuda", dst), dtype=torch.uint8)
    t = _time_events(lambda: b.copy_(a, non_blocking=True), 8, budget_s)
    torch.cuda.synchronize(dst)
    return n / t / 1e9


def measure(refresh: bool = False) -> Roof:
    name = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
    pf = _peaks_file()
    if pf is not None and not refresh:
        d = json.loads(pf.read_text())
        return Roof(float(d["hbm_gbs"]), float(d["bf16_tflops"]),
                    float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), float(d.get("i8_tops", 0.0)),
                    source=str(pf.name), device=d.get("gpu_name", name))
    cp = _cache_path(name)
    if cp.exists() and not refresh:
        return Roof(**json.loads(cp.read_text()))
    if not torch.cuda.is_available():
        raise RuntimeError("no measured peaks file and no CUDA device to probe")
    r = probe()
    cp.parent.mkdir(parents=True, exist_ok=True)
    cp.write_text(json.dumps(asdict(r)))
    return r
