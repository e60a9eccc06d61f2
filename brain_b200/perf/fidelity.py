"""Fidelity probe (reference: crates/perf/src/fidelity.rs:26-110): before a throughput number is
trusted, the same requests are run one at a time and concurrently and their greedy outputs must
agree (token-for-token, above a threshold for numerically sensitive paths)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence


@dataclass
class Fidelity:
    gate: str
    reference: str
    compared: int
    matching: int
    agreement: float
    threshold: float
    detail: str = ""

    @property
    def passed(self) -> bool:
        return self.compared > 0 and self.agreement >= self.threshold

    def to_json(self) -> Dict:
        return {"gate": self.gate, "reference": self.reference, "compared": self.compared, "matching": self.matching,
                "agreement": self.agreement, "threshold": self.threshold, "passed": self.passed, "detail": self.detail}


def greedy(reference: str, cand: Sequence[Sequence[int]], refr: Sequence[Sequence[int]], threshold: float = 1.0) -> Fidelity:
    """Mean longest-common-prefix fraction over request pairs (exact match = 1.0)."""
    n = min(len(cand), len(refr))
    tot, exact = 0.0, 0
    for a, b in zip(cand[:n], refr[:n]):
        k = 0
        for x, y in zip(a, b):
            if x != y:
                break
            k += 1
        tot += k / max(len(b), len(a), 1)
        exact += int(list(a) == list(b))
    return Fidelity("greedy_tokens", reference, n, exact, tot / max(n, 1), threshold)


def serial_vs_concurrent(make_target, workload, n: int = 4, threshold: float = 1.0) -> Fidelity:
    """Run the first ``n`` requests serially on one target and concurrently on another."""
    from .driver import drive
    from .workload import Arrival, Workload
    import copy
    small = copy.copy(workload)
    small.num_requests, small.warmup_requests = n, 0
    outs = []
    for conc in (1, n):
        small.arrival = Arrival.closed_loop(conc)
        t = make_target()
        try:
            run = drive(t, small)
            outs.append([t.outputs(rid) for rid in run.ids])
        finally:
            t.close()
    return greedy("serial", outs[1], outs[0], threshold)
