"""Device enumeration and selection (reference: crates/cli/src/devices_cli.rs — one line per adapter
with name, memory and whether it is the selected one; crates/gpu-core/src/devices.rs — canonical GPU
indices sorted by PCI bus id; the ``--device`` grammar of crates/cli/src/main.rs:113-131):

    (omitted)      every device            cpu           CPU only, all cores
    gpu            every GPU               gpu0          only physical GPU 0
    gpu0,gpu1      those two cards         cpu21         only CPU core 21
    cpu0-7         CPU cores 0..=7         gpu1,cpu0-3   one card plus four cores
    cuda / cuda:N  torch spellings of gpu / gpuN

Indexed CPU selections pin the process affinity and size the thread pool to match.  ``npu`` and
``vulkan`` name back ends that do not exist here and are refused."""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class Selection:
    gpus: Optional[List[int]] = None       # None: every GPU; []: no GPU
    cpu: bool = True                        # CPU schedulable
    cores: Optional[List[int]] = None       # None: all cores
    spec: str = ""

    def first(self) -> torch.device:
        """Where single-device work runs: the first selected GPU, else the CPU."""
        if self.gpus is None:
            return torch.device("cuda:0") if torch.cuda.is_available() else torch.device("cpu")
        if self.gpus:
            return torch.device("cuda", canonical_to_torch(self.gpus[0]))
        return torch.device("cpu")


def _pci_key(i: int):
    p = torch.cuda.get_device_properties(i)
    return (getattr(p, "pci_domain_id", 0), getattr(p, "pci_bus_id", i), getattr(p, "pci_device_id", 0))


def canonical_order() -> List[int]:
    """torch device indices sorted by PCI bus id: position = canonical index."""
    if not torch.cuda.is_available():
        return []
    return sorted(range(torch.cuda.device_count()), key=_pci_key)


def canonical_to_torch(idx: int) -> int:
    order = canonical_order()
    if not order:
        return idx
    if idx < 0 or idx >= len(order):
        raise ValueError(f"gpu{idx}: this machine has GPUs 0..{len(order) - 1}")
    return order[idx]


def parse_selection(spec: str) -> Selection:
    spec = (spec or "").strip()
    if spec in ("", "auto"):
        return Selection(spec=spec)
    gpus: Optional[List[int]] = []
    cores: Optional[List[int]] = None
    cpu = False
    for part in spec.split(","):
        part = part.strip()
        if part in ("gpu", "cuda"):
            gpus = None
        elif part == "cpu":
            cpu = True
        elif part in ("npu", "vulkan"):
            raise ValueError(f"--device {part}: that back end does not exist in this build (CUDA and CPU only)")
        elif part.startswith("cuda:") and part[5:].isdigit():
            if gpus is not None:
                gpus.append(int(part[5:]))
        elif part.startswith("gpu") and part[3:].isdigit():
            if gpus is not None:
                gpus.append(int(part[3:]))
        elif part.startswith("cpu"):
            rng = part[3:]
            lo, sep, hi = rng.partition("-")
            if not lo.isdigit() or (sep and not hi.isdigit()):
                raise ValueError(f"--device {part}: expected cpuN or cpuA-B")
            a, b = int(lo), int(hi) if sep else int(lo)
            if b < a:
                raise ValueError(f"--device {part}: empty core range")
            cpu = True
            cores = sorted(set((cores or []) + list(range(a, b + 1))))
        else:
            raise ValueError(f"--device {part!r}: expected cpu | gpu | gpuN | cpuN | cpuA-B (comma separated)")
    if gpus is not None:
        gpus = sorted(set(gpus))
    return Selection(gpus, cpu or not (gpus is None or gpus), cores, spec)


def apply_selection(sel: Selection) -> Selection:
    """Pin affinity / size the thread pool for an indexed CPU selection (no-op otherwise)."""
    if sel.cores:
        avail = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else set(range(os.cpu_count() or 1))
        want = [c for c in sel.cores if c in avail]
        if not want:
            raise ValueError(f"--device {sel.spec}: none of the cores {sel.cores} is available to this process")
        if hasattr(os, "sched_setaffinity"):
            os.sched_setaffinity(0, want)
        torch.set_num_threads(len(want))
    return sel


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
    if want and not want.startswith("cuda") and want not in ("gpu", "cpu"):
        try:
            d = parse_selection(want).first()
            return "cpu" if d.type == "cpu" else f"cuda:{d.index}"
        except ValueError:
            return want
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
