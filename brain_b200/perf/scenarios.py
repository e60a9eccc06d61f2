"""Named scenarios of the perf harness (reference: crates/perf/src/scenarios/mod.rs — tier 1
``latency`` / ``throughput`` / ``serve`` / ``sweep`` / ``startup`` differ only in their arrival
process and are never averaged together; tier 2 ``mixed`` / ``overload`` / ``cancel`` / ``kvcache``
/ ``soak`` measure what a single-request harness cannot: crates/perf/src/scenarios/{mixed,overload,
cancel,kvcache,soak}.rs).  ``faults`` lives in ``perf/faults.py``.

Every scenario takes ``make() -> PerfTarget`` (a fresh target per measurement) and returns one
JSON-able dict; the pass/fail rule of a tier-2 scenario is the ``passed`` key."""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence

from .driver import drive
from .metrics import Summary
from .targets import Emission, PerfTarget
from .workload import Arrival, Class, Lengths, Slo, Workload, standard

Make = Callable[[], PerfTarget]


def _run(make: Make, wl: Workload) -> Summary:
    t = make()
    try:
        r = drive(t, wl)
    finally:
        t.close()
    return Summary.build(r.records, r.wall_s, wl.classes[0].slo)


def _wl(name: str, arrival: Arrival, n: int, seed: int, vocab: int, input_override: Optional[int]) -> Workload:
    wl = standard(name, arrival, n, seed, vocab)
    if wl is None:
        raise ValueError(f"unknown workload {name!r}")
    if input_override:
        for c in wl.classes:
            c.input = Lengths.fixed(input_override)
    return wl


# ------------------------------------------------------------------------------------ tier 1
def latency(make: Make, workload: str = "interactive", n: int = 16, seed: int = 0, vocab: int = 32000,
            input_override: Optional[int] = None) -> Dict:
    """One request at a time: the floor of TTFA / per-token latency with no batching."""
    s = _run(make, _wl(workload, Arrival.closed_loop(1), n, seed, vocab, input_override))
    return {"scenario": "latency", "workload": workload, "summary": s.to_json()}


def throughput(make: Make, workload: str = "interactive", n: int = 64, seed: int = 0, vocab: int = 32000,
               input_override: Optional[int] = None) -> Dict:
    """Everything queued at t = 0: the engine's peak artifact rate."""
    s = _run(make, _wl(workload, Arrival.saturated(), n, seed, vocab, input_override))
    return {"scenario": "throughput", "workload": workload, "summary": s.to_json()}


def serve(make: Make, per_s: float, workload: str = "interactive", n: int = 64, seed: int = 0, vocab: int = 32000,
          burstiness: float = 1.0, input_override: Optional[int] = None) -> Dict:
    """Open-loop arrivals at a rate: what a client population sees (goodput under the SLO)."""
    s = _run(make, _wl(workload, Arrival.rate(per_s, burstiness), n, seed, vocab, input_override))
    return {"scenario": "serve", "workload": workload, "rate_per_s": per_s, "summary": s.to_json()}


def sweep(make: Make, ladder: Sequence[int] = (1, 2, 4, 8, 16), workload: str = "interactive", n: int = 32,
          seed: int = 0, vocab: int = 32000, input_override: Optional[int] = None) -> Dict:
    """Closed-loop concurrency ladder; the knee is where output rate stops growing (< 10 % gain)."""
    rows = []
    for c in ladder:
        s = _run(make, _wl(workload, Arrival.closed_loop(c), max(n, 2 * c), seed, vocab, input_override))
        rows.append({"concurrency": c, "output_per_s": s.output_per_s, "ttfa_ms_p50": s.ttfa.pct(0.5),
                     "tpoa_ms_p50": s.tpoa.pct(0.5), "slo_attainment": s.slo_attainment})
    knee = rows[-1]["concurrency"]
    for a, b in zip(rows, rows[1:]):
        if b["output_per_s"] < 1.10 * a["output_per_s"]:
            knee = a["concurrency"]
            break
    return {"scenario": "sweep", "workload": workload, "rows": rows, "knee": knee}


def startup(make: Make, vocab: int = 32000, seed: int = 0) -> Dict:
    """Cold start: time to build the target, then time to the first artifact of the first request."""
    t0 = time.perf_counter()
    t = make()
    build_s = time.perf_counter() - t0
    wl = standard("interactive", Arrival.closed_loop(1), 1, seed, vocab)
    wl.classes[0].input, wl.classes[0].output = Lengths.fixed(32), Lengths.fixed(4)
    try:
        t1 = time.perf_counter()
        r = drive(t, wl)
    finally:
        t.close()
    rec = r.records[0]
    first = (rec.first - t1) if rec.first is not None else None
    return {"scenario": "startup", "build_s": build_s, "first_artifact_s": first,
            "cold_ttfa_s": (build_s + first) if first is not None else None}


# ------------------------------------------------------------------------------------ tier 2
def mixed(make: Make, n: int = 48, concurrency: int = 8, seed: int = 0, vocab: int = 32000, short: int = 32,
          long: int = 512, out_tokens: int = 16) -> Dict:
    """Short interactive requests sharing the engine with long-prompt requests: the short class's
    TTFA must not collapse to the long class's (chunked prefill / fair admission)."""
    classes = [Class("short", Lengths.fixed(short), Lengths.fixed(out_tokens), 3.0, Slo.interactive(2000.0, 200.0)),
               Class("long", Lengths.fixed(long), Lengths.fixed(out_tokens), 1.0, Slo.ttfa(10000.0))]
    wl = Workload("mixed", classes, Arrival.closed_loop(concurrency), n, 0, True, seed, vocab)
    t = make()
    try:
        r = drive(t, wl)
    finally:
        t.close()
    per = {}
    for ci, c in enumerate(classes):
        recs = [x for x in r.records if x.cls == ci]
        s = Summary.build(recs, r.wall_s, c.slo)
        per[c.name] = {"requests": s.requests, "completed": s.completed, "ttfa_ms_p50": s.ttfa.pct(0.5),
                       "ttfa_ms_p99": s.ttfa.pct(0.99), "slo_attainment": s.slo_attainment}
    ok = all(v["completed"] == v["requests"] for v in per.values())
    return {"scenario": "mixed", "classes": per, "passed": ok}


def overload(make_bounded: Make, capacity_per_s: float, factor: float = 3.0, n: int = 64, seed: int = 0,
             vocab: int = 32000, workload: str = "interactive", input_override: Optional[int] = None) -> Dict:
    """Arrivals at ``factor`` x the measured capacity against a target with a bounded queue: the
    excess is REJECTED quickly (not queued forever), accepted requests still finish, and goodput
    stays near capacity instead of collapsing."""
    wl = _wl(workload, Arrival.rate(capacity_per_s * factor), n, seed, vocab, input_override)
    s = _run(make_bounded, wl)
    accepted = s.requests - s.rejected
    ok = s.rejected > 0 and s.completed == accepted and s.failed == 0
    return {"scenario": "overload", "offered_per_s": capacity_per_s * factor, "summary": s.to_json(),
            "rejected_fraction": s.rejected / max(s.requests, 1), "passed": ok}


def cancel(make: Make, n: int = 16, cancel_every: int = 2, after_artifacts: int = 2, seed: int = 0,
           vocab: int = 32000, input_len: int = 64, out_tokens: int = 32) -> Dict:
    """Cancel every ``cancel_every``-th request after its first artifacts: cancelled requests stop
    producing, their KV blocks return to the pool, and the survivors' outputs equal an undisturbed
    run's (crates/perf/src/scenarios/cancel.rs)."""
    wl = standard("interactive", Arrival.saturated(), n, seed, vocab)
    wl.classes[0].input, wl.classes[0].output = Lengths.fixed(input_len), Lengths.fixed(out_tokens)
    reqs = wl.requests()
    # undisturbed reference outputs
    t = make()
    try:
        ids = [t.submit(q) for q in reqs]
        ems: List[Emission] = []
        while t.step(ems):
            ems.clear()
        want = {i: list(t.outputs(rid)) for i, rid in enumerate(ids)}
    finally:
        t.close()
    t = make()
    try:
        if not hasattr(t, "cancel"):
            return {"scenario": "cancel", "skipped": "target has no cancel", "passed": True}
        free0 = t.free_blocks() if hasattr(t, "free_blocks") else None
        ids = [t.submit(q) for q in reqs]
        by = {rid: i for i, rid in enumerate(ids)}
        victims = {rid for i, rid in enumerate(ids) if i % cancel_every == 0}
        seen = {rid: 0 for rid in ids}
        cancelled_at: Dict[int, int] = {}
        late = 0
        ems = []
        busy = True
        while busy:
            ems.clear()
            busy = t.step(ems)
            for e in ems:
                if e.kind != "artifact":
                    continue
                if e.id in cancelled_at:
                    late += e.count
                    continue
                seen[e.id] += e.count
                if e.id in victims and seen[e.id] >= after_artifacts:
                    t.cancel(e.id)
                    cancelled_at[e.id] = seen[e.id]
        survivors_equal = all(list(t.outputs(rid)) == want[by[rid]] for rid in ids if rid not in victims)
        free1 = t.free_blocks() if hasattr(t, "free_blocks") else None
    finally:
        t.close()
    ok = survivors_equal and late == 0 and len(cancelled_at) == len(victims) and (free0 is None or free1 == free0)
    return {"scenario": "cancel", "cancelled": len(cancelled_at), "late_artifacts": late,
            "survivors_equal": survivors_equal, "blocks_before": free0, "blocks_after": free1, "passed": ok}


def kvcache(make_cached: Make, make_uncached: Make, n: int = 16, prefix: int = 192, tail: int = 32,
            out_tokens: int = 8, seed: int = 0, vocab: int = 32000) -> Dict:
    """Requests that share a long prompt prefix, with and without the prefix cache: the cache must
    cut the prompt tokens actually prefilled and leave the outputs unchanged
    (crates/perf/src/scenarios/kvcache.rs)."""
    c = Class("shared", Lengths.fixed(prefix + tail), Lengths.fixed(out_tokens), 1.0, Slo.ttfa(5000.0),
              shared_prefix=prefix)
    wl = Workload("kvcache", [c], Arrival.closed_loop(1), n, 0, True, seed, vocab)
    res = {}
    outs = {}
    for name, make in (("cached", make_cached), ("uncached", make_uncached)):
        t = make()
        try:
            r = drive(t, wl)
            s = Summary.build(r.records, r.wall_s, c.slo)
            outs[name] = [list(t.outputs(rid)) for rid in r.ids]
            res[name] = {"ttfa_ms_p50": s.ttfa.pct(0.5), "output_per_s": s.output_per_s,
                         "prefill_tokens": t.prefill_tokens() if hasattr(t, "prefill_tokens") else None}
        finally:
            t.close()
    same = outs["cached"] == outs["uncached"]
    pc, pu = res["cached"]["prefill_tokens"], res["uncached"]["prefill_tokens"]
    saved = (1.0 - pc / pu) if pc is not None and pu else None
    ok = same and (saved is None or saved > 0.5 * prefix / (prefix + tail))
    return {"scenario": "kvcache", "cached": res["cached"], "uncached": res["uncached"], "outputs_equal": same,
            "prefill_saved_fraction": saved, "passed": ok}


def soak(make: Make, seconds: float = 5.0, concurrency: int = 4, seed: int = 0, vocab: int = 32000,
         input_len: int = 48, out_tokens: int = 8) -> Dict:
    """Closed-loop traffic for a fixed time on ONE target: throughput of the last third must stay
    within 30 % of the first third and every KV block must be back in the pool at the end."""
    t = make()
    thirds: List[float] = []
    total = 0
    try:
        free0 = t.free_blocks() if hasattr(t, "free_blocks") else None
        t_end = time.perf_counter() + seconds
        round_i = 0
        marks = []
        while time.perf_counter() < t_end:
            wl = standard("interactive", Arrival.closed_loop(concurrency), 4 * concurrency, seed + round_i, vocab)
            wl.classes[0].input, wl.classes[0].output = Lengths.fixed(input_len), Lengths.fixed(out_tokens)
            r = drive(t, wl)
            s = Summary.build(r.records, r.wall_s, wl.classes[0].slo)
            marks.append((time.perf_counter(), s.output_artifacts, r.wall_s))
            total += s.completed
            round_i += 1
        free1 = t.free_blocks() if hasattr(t, "free_blocks") else None
    finally:
        t.close()
    k = max(len(marks) // 3, 1)
    rate = lambda ms: sum(m[1] for m in ms) / max(sum(m[2] for m in ms), 1e-9)
    first, last = rate(marks[:k]), rate(marks[-k:])
    ok = last >= 0.7 * first and (free0 is None or free0 == free1)
    return {"scenario": "soak", "rounds": len(marks), "completed": total, "first_third_per_s": first,
            "last_third_per_s": last, "blocks_before": free0, "blocks_after": free1, "passed": ok}


TIER1 = ("latency", "throughput", "serve", "sweep", "startup")
TIER2 = ("mixed", "overload", "cancel", "kvcache", "soak", "faults", "residency", "placement", "frontend")
