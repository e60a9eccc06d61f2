"""Structured tracing with per-family levels (reference: crates/trace/src/registry.rs:43-62 family
table, crates/trace/src/init.rs:115 install; flags ``--trace-<family> 0-5``, ``--trace name=level``,
``--trace-format text|json``, ``--trace-output -|path``, env ``BRAIN_TRACE``).

Library code calls :func:`event`; nothing is printed until the binary calls :func:`install`."""
from __future__ import annotations

import json
import os
import sys
import threading
import time
from typing import Dict, List, Optional, TextIO, Tuple

LEVELS = ["off", "error", "warn", "info", "debug", "trace"]
FAMILIES = ["cli", "train", "serve", "sched", "engine", "kernel", "comm", "checkpoint", "data", "api",
            "executor", "perf", "federated", "optim", "parallel"]

_levels: Dict[str, int] = {}
_fmt = "text"
_out: Optional[TextIO] = None
_lock = threading.Lock()
_t0 = time.time()


def _parse_level(s: str) -> int:
    s = s.strip().lower()
    if s.isdigit():
        return max(0, min(5, int(s)))
    if s in LEVELS:
        return LEVELS.index(s)
    raise ValueError(f"bad trace level {s!r} (0-5 or {'|'.join(LEVELS)})")


def parse_spec(spec: str) -> Dict[str, int]:
    """``"serve=4,comm=debug,3"`` -> per-family levels; a bare level applies to every family."""
    out: Dict[str, int] = {}
    for part in filter(None, (p.strip() for p in spec.split(","))):
        if "=" in part:
            name, lvl = part.split("=", 1)
            if name not in FAMILIES:
                raise ValueError(f"unknown trace family {name!r}; known: {' '.join(FAMILIES)}")
            out[name] = _parse_level(lvl)
        else:
            for f in FAMILIES:
                out.setdefault(f, _parse_level(part))
    return out


def take_flags(argv: List[str]) -> Tuple[List[str], Dict[str, int], str, str]:
    """Strip the global trace flags out of ``argv``; returns (rest, levels, format, output)."""
    rest, levels, fmt, output = [], {}, "text", "-"
    i = 0
    while i < len(argv):
        a = argv[i]
        nxt = argv[i + 1] if i + 1 < len(argv) else None
        if a == "--trace" and nxt is not None:
            levels.update(parse_spec(nxt)); i += 2
        elif a == "--trace-format" and nxt is not None:
            if nxt not in ("text", "json"):
                raise ValueError("--trace-format text|json")
            fmt = nxt; i += 2
        elif a == "--trace-output" and nxt is not None:
            output = nxt; i += 2
        elif a.startswith("--trace-") and a[8:] in FAMILIES and nxt is not None:
            levels[a[8:]] = _parse_level(nxt); i += 2
        else:
            rest.append(a); i += 1
    return rest, levels, fmt, output


def install(levels: Optional[Dict[str, int]] = None, fmt: str = "text", output: str = "-") -> None:
    global _fmt, _out
    env = os.environ.get("BRAIN_TRACE")
    merged = parse_spec(env) if env else {}
    merged.update(levels or {})
    _levels.clear()
    _levels.update(merged)
    _fmt = fmt
    _out = sys.stderr if output in ("-", "") else open(output, "a", buffering=1)


def enabled(family: str, level: int = 3) -> bool:
    return _out is not None and _levels.get(family, 0) >= level


def event(family: str, level: int, message: str, **fields) -> None:
    if not enabled(family, level):
        return
    if _fmt == "json":
        rec = {"ts": round(time.time(), 6), "level": LEVELS[level], "target": family, "message": message}
        rec.update(fields)
        line = json.dumps(rec, default=str)
    else:
        kv = " ".join(f"{k}={v}" for k, v in fields.items())
        line = f"{time.time() - _t0:10.4f} {LEVELS[level].upper():5} {family}: {message}" + (f" {kv}" if kv else "")
    with _lock:
        print(line, file=_out)


class span:
    """``with span('train', 'step', step=3):`` emits enter/exit events with the elapsed time."""

    def __init__(self, family: str, name: str, level: int = 4, **fields):
        self.family, self.name, self.level, self.fields = family, name, level, fields

    def __enter__(self):
        self.t = time.perf_counter()
        event(self.family, self.level, f"{self.name} begin", **self.fields)
        return self

    def __exit__(self, *exc):
        event(self.family, self.level, f"{self.name} end",
              ms=round((time.perf_counter() - self.t) * 1e3, 3), **self.fields)
        return False
