"""Device enumeration for ``brain devices`` (reference: crates/cli/src/devices_cli.rs — one line per
adapter with name, memory and whether it is the selected one; selection by ``BRAIN_DEVICE`` /
``BRAIN_GPU_INDEX`` / ``--device``)."""
from __future__ import annotations

import os
from typing import Dict, List

import torch


def list_devices() -> List[Dict]:
    out = [{"index": -1, "kind": "cpu", "name": "CPU (fp32 reference backend)", "memory_gb": None,
            "sm": None, "cc": None}]
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            out.append({"index": i, "kind": "cuda", "name": p.name, "memory_gb": p.total_memory / 2**30,
                        "sm": p.multi_processor_count, "cc": f"{p.major}.{p.minor}"})
    return out


def selected(device_flag: str = "") -> str:
    want = device_flag or os.environ.get("BRAIN_DEVICE", "")
    if want in ("cpu",):
        return "cpu"
    idx = os.environ.get("BRAIN_GPU_INDEX")
    if want.startswith("cuda"):
        return want if ":" in want else f"cuda:{idx or 0}"
    if want == "gpu" or want == "":
        return f"cuda:{idx or 0}" if torch.cuda.is_available() else "cpu"
    return want


def peer_matrix() -> List[List[bool]]:
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]


def render(device_flag: str = "") -> str:
    sel = selected(device_flag)
    lines = []
    for d in list_devices():
        name = "cpu" if d["kind"] == "cpu" else f"cuda:{d['index']}"
        mark = "*" if name == sel else " "
        if d["kind"] == "cpu":
            lines.append(f"{mark} {name:<8} {d['name']}")
        else:
            native = "sm_100a kernels" if d["cc"] == "10.0" else "unsupported (kernels target sm_100a)"
            lines.append(f"{mark} {name:<8} {d['name']}  {d['memory_gb']:.0f} GiB  {d['sm']} SMs  cc {d['cc']}  {native}")
    pm = peer_matrix()
    if len(pm) > 1:
        lines.append("peer access: " + ("all pairs" if all(all(r) for r in pm) else
                                         "; ".join(f"{i}->{[j for j, ok in enumerate(r) if ok and j != i]}"
                                                   for i, r in enumerate(pm))))
    return "\n".join(lines)
