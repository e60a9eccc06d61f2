"""Per-request records and run summaries (reference: crates/perf/src/metrics.rs:28-253 — queue,
time-to-first-artifact, time-per-output-artifact, inter-artifact latencies, end-to-end; summary
percentiles, throughput, goodput = output that met its SLO)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .workload import Slo


@dataclass
class ReqRecord:
    id: int
    cls: int
    input_artifacts: int
    warmup: bool
    submit: float
    admit: Optional[float] = None
    first: Optional[float] = None
    done: Optional[float] = None
    artifacts: List[float] = field(default_factory=list)
    counts: List[int] = field(default_factory=list)     # artifacts delivered at each timestamp
    failed: bool = False
    rejected: bool = False
    error: Optional[str] = None

    def queue_ms(self):
        return None if self.admit is None else (self.admit - self.submit) * 1e3

    def ttfa_ms(self):
        return None if self.first is None else (self.first - self.submit) * 1e3

    def e2e_ms(self):
        return None if self.done is None else (self.done - self.submit) * 1e3

    def output_artifacts(self) -> int:
        return sum(self.counts)

    def ial_ms(self) -> List[float]:
        """Gaps between deliveries, spread over the artifacts each delivery carried."""
        out = []
        for (t0, t1, n) in zip(self.artifacts, self.artifacts[1:], self.counts[1:]):
            out += [(t1 - t0) * 1e3 / max(n, 1)] * max(n, 1)
        return out

    def tpoa_ms(self):
        n = self.output_artifacts()
        if self.first is None or self.done is None or n < 2:
            return None
        return (self.done - self.first) * 1e3 / (n - 1)

    def meets(self, slo: Slo) -> bool:
        if self.failed or self.rejected or self.done is None:
            return False
        if slo.ttfa_ms is not None and (self.ttfa_ms() is None or self.ttfa_ms() > slo.ttfa_ms):
            return False
        if slo.ial_ms is not None:
            t = self.tpoa_ms()
            if t is not None and t > slo.ial_ms:
                return False
        return True


class Dist:
    def __init__(self):
        self.v: List[float] = []

    def push(self, x: float):
        self.v.append(float(x))

    def pct(self, p: float) -> Optional[float]:
        if not self.v:
            return None
        s = sorted(self.v)
        k = (len(s) - 1) * p
        lo = int(k)
        hi = min(lo + 1, len(s) - 1)
        return s[lo] + (s[hi] - s[lo]) * (k - lo)

    def mean(self) -> Optional[float]:
        return sum(self.v) / len(self.v) if self.v else None

    def to_json(self):
        if not self.v:
            return {"n": 0}
        return {"n": len(self.v), "mean": self.mean(), "p50": self.pct(0.5), "p90": self.pct(0.9),
                "p99": self.pct(0.99), "max": max(self.v)}


@dataclass
class Summary:
    wall_s: float
    requests: int
    completed: int
    failed: int
    rejected: int
    input_artifacts: int
    output_artifacts: int
    requests_per_s: float
    input_per_s: float
    output_per_s: float
    goodput_per_s: float
    slo_attainment: float
    ttfa: Dist
    ial: Dist
    tpoa: Dist
    e2e: Dist
    queue: Dist
    slo: Slo
    errors: List[str]

    @staticmethod
    def build(records: List[ReqRecord], wall_s: float, slo: Slo) -> "Summary":
        ms = [r for r in records if not r.warmup]
        ttfa, ial, tpoa, e2e, queue = Dist(), Dist(), Dist(), Dist(), Dist()
        completed = failed = rejected = in_a = out_a = met = good = 0
        errors: List[str] = []
        for r in ms:
            if r.rejected:
                rejected += 1
                continue
            if r.failed:
                failed += 1
                if r.error and r.error not in errors and len(errors) < 5:
                    errors.append(r.error)
            elif r.done is not None:
                completed += 1
            in_a += r.input_artifacts
            out_a += r.output_artifacts()
            for d, v in ((ttfa, r.ttfa_ms()), (e2e, r.e2e_ms()), (queue, r.queue_ms()), (tpoa, r.tpoa_ms())):
                if v is not None:
                    d.push(v)
            for g in r.ial_ms():
                ial.push(g)
            if r.meets(slo):
                met += 1
                good += r.output_artifacts()
        secs = max(wall_s, 1e-9)
        admitted = len(ms) - rejected
        return Summary(wall_s, len(ms), completed, failed, rejected, in_a, out_a, completed / secs, in_a / secs,
                       out_a / secs, good / secs, 1.0 if admitted == 0 else met / admitted, ttfa, ial, tpoa, e2e,
                       queue, slo, errors)

    def to_json(self) -> Dict:
        return {"wall_s": self.wall_s, "requests": self.requests, "completed": self.completed, "failed": self.failed,
                "rejected": self.rejected, "input_artifacts": self.input_artifacts,
                "output_artifacts": self.output_artifacts, "requests_per_s": self.requests_per_s,
                "input_per_s": self.input_per_s, "output_per_s": self.output_per_s,
                "goodput_per_s": self.goodput_per_s, "slo_attainment": self.slo_attainment,
                "ttfa_ms": self.ttfa.to_json(), "ial_ms": self.ial.to_json(), "tpoa_ms": self.tpoa.to_json(),
                "e2e_ms": self.e2e.to_json(), "queue_ms": self.queue.to_json(), "slo": self.slo.to_json(),
                "errors": self.errors}
