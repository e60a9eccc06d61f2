"""Regression gate between two result rows (reference: crates/perf/src/gate.rs:30-142): throughput
metrics must stay above ``floor_frac`` of the baseline, latency percentiles below ``1/floor_frac``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

_HIGHER = ("output_per_s", "requests_per_s", "goodput_per_s", "slo_attainment")
_LOWER = (("ttfa_ms", "p50"), ("ttfa_ms", "p99"), ("tpoa_ms", "p50"), ("e2e_ms", "p99"))


@dataclass
class Check:
    name: str
    candidate: float
    baseline: float
    ratio: float
    ok: bool


def compare(cand: Dict, base: Dict, floor_frac: float = 0.9) -> List[Check]:
    out = []
    for k in _HIGHER:
        if k in cand and k in base and base[k]:
            r = cand[k] / base[k]
            out.append(Check(k, cand[k], base[k], r, r >= floor_frac))
    for d, p in _LOWER:
        c, b = (cand.get(d) or {}).get(p), (base.get(d) or {}).get(p)
        if c is not None and b:
            r = c / b
            out.append(Check(f"{d}.{p}", c, b, r, r <= 1.0 / floor_frac))
    return out


def passed(checks: List[Check]) -> bool:
    return all(c.ok for c in checks)


def render(checks: List[Check], floor_frac: float) -> str:
    lines = [f"{'metric':<18} {'candidate':>12} {'baseline':>12} {'ratio':>8}  verdict (floor {floor_frac:.2f})"]
    for c in checks:
        lines.append(f"{c.name:<18} {c.candidate:>12.3f} {c.baseline:>12.3f} {c.ratio:>8.3f}  {'ok' if c.ok else 'REGRESSION'}")
    lines.append("gate: " + ("PASS" if passed(checks) else "FAIL"))
    return "\n".join(lines)
