"""The measurement loop (reference: crates/perf/src/driver.rs:29-140): submit requests as the
arrival process allows, step the target, fold emissions into per-request records; wall time runs
from the first measured submission to the last measured completion."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List

from .metrics import ReqRecord
from .targets import Emission, PerfTarget
from .workload import Workload


@dataclass
class Run:
    records: List[ReqRecord]
    wall_s: float
    ids: List[int]


def drive(target: PerfTarget, wl: Workload, max_seconds: float = 3600.0) -> Run:
    reqs = wl.requests()
    delays = wl.arrival_delays()
    records: List[ReqRecord] = []
    by_id: Dict[int, int] = {}
    nxt = in_flight = 0
    conc = wl.arrival.concurrency if wl.arrival.kind == "closed_loop" else 1 << 60
    t_start = time.perf_counter()
    due_at = delays[0] if delays else 0.0
    m_start = m_end = None
    ems: List[Emission] = []
    while True:
        while nxt < len(reqs):
            if wl.arrival.kind == "closed_loop":
                due = in_flight < conc
            elif wl.arrival.kind == "saturated":
                due = True
            else:
                due = time.perf_counter() - t_start >= due_at
            if not due:
                break
            warm = nxt < wl.warmup_requests
            now = time.perf_counter()
            try:
                rid = target.submit(reqs[nxt])
            except Exception as e:  # noqa: BLE001 - a refused submission is a rejected request
                rec = ReqRecord(-1 - nxt, reqs[nxt].cls, reqs[nxt].input_artifacts, warm, now)
                rec.rejected, rec.done, rec.error = True, now, str(e)
                records.append(rec)
                nxt += 1
                continue
            by_id[rid] = len(records)
            records.append(ReqRecord(rid, reqs[nxt].cls, reqs[nxt].input_artifacts, warm, now))
            if not warm and m_start is None:
                m_start = now
            nxt += 1
            in_flight += 1
            if nxt < len(delays):
                due_at += delays[nxt]
        ems.clear()
        busy = target.step(ems)
        for e in ems:
            idx = by_id.get(e.id)
            if idx is None:
                continue
            r = records[idx]
            if e.kind == "admitted":
                r.admit = e.at
            elif e.kind == "artifact":
                if r.first is None:
                    r.first = e.at
                r.artifacts.append(e.at)
                r.counts.append(e.count)
            else:
                r.done = e.at
                r.failed = e.kind == "failed"
                r.rejected = e.kind == "rejected"
                r.error = e.error
                in_flight = max(in_flight - 1, 0)
                if not r.warmup:
                    m_end = e.at
        if nxt >= len(reqs) and not busy and in_flight == 0:
            break
        if time.perf_counter() - t_start > max_seconds:
            break
        if not busy and nxt < len(reqs) and wl.arrival.kind in ("rate", "ramp"):
            time.sleep(min(max(due_at - (time.perf_counter() - t_start), 0.0), 0.01))
    wall = (m_end - m_start) if m_start is not None and m_end is not None else time.perf_counter() - t_start
    return Run(records, wall, [r.id for r in records])
