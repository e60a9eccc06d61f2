"""``brain top``: a refreshing text view of a running server's stats snapshot (reference:
crates/braintop — accelerators, resident models with their schedulers, executor lanes, request
accounting; the reference reads the snapshot over D-Bus, here it is ``GET /stats`` of any HTTP
surface)."""
from __future__ import annotations

import json
import sys
import time
import urllib.request
from typing import Dict, List

from .args import Args


def fetch(url: str, key: str, timeout: float = 5.0) -> Dict:
    req = urllib.request.Request(url.rstrip("/") + "/stats", headers={"Authorization": f"Bearer {key}"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read().decode())


def _gb(x) -> str:
    return f"{x / 2**30:6.1f}G"


def render(snap: Dict) -> str:
    out: List[str] = []
    up = snap.get("uptime_s")
    out.append(f"brain top — uptime {up:.0f}s" if up is not None else "brain top")
    acc = snap.get("accelerators") or []
    if acc:
        out.append("accelerators")
        for a in acc:
            out.append(f"  [{a['index']}] {a['name']:<24} used {_gb(a['memory_used'])} / {_gb(a['memory_total'])}"
                       f"   torch allocated {_gb(a['allocated'])} reserved {_gb(a['reserved'])}")
    out.append("models")
    for m in snap.get("models") or []:
        line = f"  {m['id']:<40} ctx {m.get('context_length') or '-':>6}  actions {','.join(m.get('actions', []))}"
        sch = m.get("scheduler")
        if sch:
            line += "   " + "  ".join(f"{k} {v}" for k, v in sch.items())
        out.append(line)
    ex = snap.get("executor") or {}
    if ex:
        out.append("executor  " + "  ".join(f"{k} {v}" for k, v in ex.items() if not isinstance(v, (dict, list))))
    con = snap.get("connections") or {}
    if con:
        out.append(f"connections  in flight {con.get('in_flight', 0)} / {con.get('limit', '-')}")
    for name, r in (snap.get("requests") or {}).items():
        out.append(f"requests[{name}]  " + "  ".join(f"{k} {v}" for k, v in r.items() if not isinstance(v, (dict, list))))
    return "\n".join(out)


def run_top(argv: List[str]) -> int:
    a = Args(argv)
    url = a.str_or("--url", "http://127.0.0.1:8788")
    key = a.str_or("--key", "")
    keys_file = a.take_str("--api-keys")
    interval = a.float_or("--interval", 0.5)
    once = a.take_flag("--once")
    as_json = a.take_flag("--json")
    a.finish()
    if not key and keys_file:
        ks = json.loads(open(keys_file).read())
        key = next(iter(ks.values())) if isinstance(ks, dict) else ks[0]
    if not key:
        print("usage: brain top --url http://HOST:PORT (--key sk-brain-… | --api-keys keys.json) [--interval S --once --json]",
              file=sys.stderr)
        return 2
    try:
        while True:
            snap = fetch(url, key)
            text = json.dumps(snap, indent=1) if as_json else render(snap)
            if once:
                print(text)
                return 0
            sys.stdout.write("\x1b[2J\x1b[H" + text + "\n")
            sys.stdout.flush()
            time.sleep(max(interval, 0.05))
    except KeyboardInterrupt:
        return 0
    except Exception as e:  # noqa: BLE001
        print(f"brain top: {e}", file=sys.stderr)
        return 1
