"""Stats snapshot (reference: crates/stats/src/snapshot.rs:27-175 — accelerators, models,
instances, executor, requests, connections as one JSON document; the reference streams it over
D-Bus at 2 Hz, here it is served at ``GET /stats`` and printed by ``brain serve -v 2``)."""
from __future__ import annotations

import time
from typing import Dict, Optional


def accelerators() -> list:
    import torch
    out = []
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            free, total = torch.cuda.mem_get_info(i)
            out.append({"index": i, "name": p.name, "memory_total": total, "memory_used": total - free,
                        "allocated": torch.cuda.memory_allocated(i), "reserved": torch.cuda.memory_reserved(i)})
    return out


def snapshot(executor=None, surfaces: Optional[Dict] = None) -> Dict:
    snap = {"ts": time.time(), "accelerators": accelerators(), "models": [], "executor": {}, "requests": {},
            "connections": {}}
    if executor is not None:
        snap["uptime_s"] = time.time() - executor.started
        snap["executor"] = executor.stats()
        snap["connections"] = {"in_flight": executor.in_flight(), "limit": executor.edge_limit}
        for mid, m in executor.models().items():
            entry = {"id": mid, "context_length": m.context_length(), "actions": [a.name for a in m.manifest().actions]}
            if hasattr(m, "stats"):
                entry["scheduler"] = m.stats()
            snap["models"].append(entry)
    for name, s in (surfaces or {}).items():
        snap["requests"][name] = s.acct.snapshot()
    return snap
