"""Workload vocabulary of the perf harness (reference: crates/perf/src/workload.rs — arrival
processes :20-45, length distributions :48-75, gamma inter-arrival :232-252, the standard workload
table :262-269 with its SLOs)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from ..data.rng import Rng


@dataclass
class Arrival:
    kind: str = "closed_loop"            # closed_loop | saturated | rate | ramp
    concurrency: int = 1
    per_s: float = 0.0
    burstiness: float = 1.0              # gamma shape: 1 = Poisson, <1 burstier
    to_per_s: float = 0.0

    @staticmethod
    def closed_loop(c: int) -> "Arrival":
        return Arrival("closed_loop", concurrency=max(c, 1))

    @staticmethod
    def saturated() -> "Arrival":
        return Arrival("saturated")

    @staticmethod
    def rate(per_s: float, burstiness: float = 1.0) -> "Arrival":
        return Arrival("rate", per_s=per_s, burstiness=burstiness)

    @staticmethod
    def ramp(a: float, b: float) -> "Arrival":
        return Arrival("ramp", per_s=a, to_per_s=b)

    def to_json(self):
        return {k: v for k, v in vars(self).items() if v or k == "kind"}


@dataclass
class Lengths:
    kind: str = "fixed"                  # fixed | uniform | lognormal
    n: int = 0
    lo: int = 0
    hi: int = 0
    sigma: float = 0.0

    @staticmethod
    def fixed(n: int) -> "Lengths":
        return Lengths("fixed", n=n)

    @staticmethod
    def uniform(lo: int, hi: int) -> "Lengths":
        return Lengths("uniform", lo=lo, hi=hi)

    @staticmethod
    def lognormal(median: int, sigma: float, lo: int, hi: int) -> "Lengths":
        return Lengths("lognormal", n=median, lo=lo, hi=hi, sigma=sigma)

    def sample(self, rng: Rng) -> int:
        if self.kind == "fixed":
            return self.n
        if self.kind == "uniform":
            return self.lo if self.hi <= self.lo else self.lo + rng.next_u64() % (self.hi - self.lo + 1)
        v = self.n * math.exp(rng.next_gaussian() * self.sigma)
        return int(min(max(round(v), self.lo), self.hi))

    def to_json(self):
        return {k: v for k, v in vars(self).items() if v or k == "kind"}


@dataclass
class Slo:
    ttfa_ms: Optional[float] = None      # time to first artifact (token)
    ial_ms: Optional[float] = None       # inter-artifact latency (per request mean)

    @staticmethod
    def interactive(ttfa: float, ial: float) -> "Slo":
        return Slo(ttfa, ial)

    @staticmethod
    def ttfa(ms: float) -> "Slo":
        return Slo(ms, None)

    def to_json(self):
        return {"ttfa_ms": self.ttfa_ms, "ial_ms": self.ial_ms}


@dataclass
class PerfRequest:
    cls: int
    prompt: np.ndarray
    max_new: int
    ignore_stop: bool = True
    seed: int = 0

    @property
    def input_artifacts(self) -> int:
        return int(self.prompt.size)


@dataclass
class Class:
    name: str
    input: Lengths
    output: Lengths
    weight: float = 1.0
    slo: Slo = field(default_factory=Slo)
    shared_prefix: int = 0               # leading tokens identical across the class's requests


@dataclass
class Workload:
    name: str
    classes: List[Class]
    arrival: Arrival
    num_requests: int
    warmup_requests: int = 0
    ignore_stop: bool = True
    seed: int = 0
    vocab: int = 32000

    def requests(self) -> List[PerfRequest]:
        rng = Rng(self.seed)
        total_w = sum(c.weight for c in self.classes)
        prefixes = {i: Rng(self.seed ^ (0x9E37 + i)).tokens(c.shared_prefix, self.vocab)
                    for i, c in enumerate(self.classes) if c.shared_prefix}
        out = []
        for r in range(self.num_requests + self.warmup_requests):
            u = rng.next_f64() * total_w
            ci = 0
            for i, c in enumerate(self.classes):
                if u < c.weight:
                    ci = i
                    break
                u -= c.weight
            c = self.classes[ci]
            n_in = max(c.input.sample(rng), 1)
            n_out = max(c.output.sample(rng), 1)
            toks = rng.tokens(n_in, self.vocab).astype(np.int64)
            if ci in prefixes:
                k = min(n_in, prefixes[ci].size)
                toks[:k] = prefixes[ci][:k]
            out.append(PerfRequest(ci, toks, n_out, self.ignore_stop, seed=r))
        return out

    def arrival_delays(self) -> List[float]:
        """Seconds between consecutive submissions (open-loop arrivals only)."""
        n = self.num_requests + self.warmup_requests
        a = self.arrival
        if a.kind in ("closed_loop", "saturated"):
            return [0.0] * n
        rng = Rng(self.seed ^ 0xA221)
        out = []
        for i in range(n):
            rate = a.per_s if a.kind == "rate" else a.per_s + (a.to_per_s - a.per_s) * i / max(n - 1, 1)
            out.append(gamma_interarrival(rng, rate, a.burstiness if a.kind == "rate" else 1.0))
        return out

    def to_json(self):
        return {"name": self.name, "arrival": self.arrival.to_json(), "num_requests": self.num_requests,
                "warmup_requests": self.warmup_requests, "ignore_stop": self.ignore_stop, "seed": self.seed,
                "classes": [{"name": c.name, "weight": c.weight, "input": c.input.to_json(),
                             "output": c.output.to_json(), "slo": c.slo.to_json()} for c in self.classes]}


def gamma_interarrival(rng: Rng, rate: float, shape: float) -> float:
    mean = 1.0 / max(rate, 1e-9)

    def exp1():
        u = min(max(rng.next_f64(), 1e-12), 1.0 - 1e-12)
        return -math.log(1.0 - u)
    if abs(shape - 1.0) < 1e-9:
        return mean * exp1()
    n = max(int(round(max(shape, 0.05))), 1)
    return mean * sum(exp1() for _ in range(n)) / n


_STANDARD = {
    "interactive": (128, 256, Slo.interactive(500.0, 50.0)),
    "chat": (1024, 256, Slo.interactive(2000.0, 50.0)),
    "rag": (4096, 128, Slo.interactive(4000.0, 50.0)),
    "rag_long": (16384, 256, Slo.interactive(10000.0, 80.0)),
    "agent": (8192, 1024, Slo.interactive(6000.0, 50.0)),
    "decode_heavy": (128, 2048, Slo.interactive(500.0, 40.0)),
    "prefill_heavy": (32768, 64, Slo.ttfa(20000.0)),
    "shared_prefix": (8192, 256, Slo.interactive(6000.0, 50.0)),
}


def standard_names() -> List[str]:
    return list(_STANDARD) + ["serving_mix"]


def standard(name: str, arrival: Arrival, num_requests: int, seed: int = 0, vocab: int = 32000) -> Optional[Workload]:
    if name == "serving_mix":
        # 512 requests at 256 concurrent, prompts U[128, 2048], 256 greedy tokens, stop ignored
        c = Class(name, Lengths.uniform(128, 2048), Lengths.fixed(256), 1.0, Slo.interactive(4000.0, 80.0))
        return Workload(name, [c], arrival, num_requests, 0, True, seed, vocab)
    if name not in _STANDARD:
        return None
    i, o, slo = _STANDARD[name]
    c = Class(name, Lengths.fixed(i), Lengths.fixed(o), 1.0, slo, shared_prefix=(i * 3 // 4 if name == "shared_prefix" else 0))
    return Workload(name, [c], arrival, num_requests, 0, True, seed, vocab)
