"""Flat parameter store: every parameter of a module becomes a view into one contiguous working-
weight buffer (bf16 on the GPU, fp32 on the CPU backend) and gets a ``main_grad`` view into one
contiguous fp32 gradient buffer.  The flat layout is what the fused reduce-scatter + AdamW kernel,
the global gradient norm and the sharded optimiser state operate on.

Reference: crates/paramstore/src/lib.rs:21-81 (named weight/grad/adam buffers and roles),
:114-205 (construction), :210-218 (gradient-norm partial layout)."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, List, Optional

import torch
import torch.nn as nn


class Role(str, Enum):
    TRAINABLE = "trainable"   # weight + grad + optimiser moments on the device
    FROZEN = "frozen"         # weight only
    OFFLOAD = "offload"       # grad on device, fp32 master + moments in host RAM (OffloadAdam)


@dataclass
class Slot:
    name: str
    offset: int
    numel: int
    shape: tuple
    role: Role
    decay: bool


ALIGN = 64  # elements; keeps every view 128-byte aligned in bf16 and 256-byte aligned in fp32


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class ParamStore:
    def __init__(self, module: nn.Module, device=None, dtype: Optional[torch.dtype] = None,
                 pad_to: int = 1, decay_fn=None, roles: Optional[Dict[str, Role]] = None, select=None):
        """``select(name) -> bool`` restricts the store to a subset of the module's parameters (a
        model may keep e.g. its replicated and its expert-parallel tensors in two stores with two
        different optimiser/collective treatments)."""
        params = [(n, p) for n, p in module.named_parameters() if select is None or select(n)]
        if device is None:
            device = params[0][1].device
        device = torch.device(device)
        if dtype is None:
            dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
        self.device, self.dtype = device, dtype
        self.slots: List[Slot] = []
        self.by_name: Dict[str, Slot] = {}
        roles = roles or {}
        # trainable params first (they are what gradients / optimiser shards cover), frozen after
        train = [(n, p) for n, p in params if p.requires_grad]
        frozen = [(n, p) for n, p in params if not p.requires_grad]
        off = 0
        for n, p in train:
            role = roles.get(n, Role.TRAINABLE)
            s = Slot(n, off, p.numel(), tuple(p.shape), role, bool(decay_fn(n)) if decay_fn else True)
            self.slots.append(s)
            self.by_name[n] = s
            off = _round_up(off + p.numel(), ALIGN)
        self.n_train = _round_up(off, max(pad_to, 1) * ALIGN)
        off = self.n_train
        for n, p in frozen:
            s = Slot(n, off, p.numel(), tuple(p.shape), Role.FROZEN, False)
            self.slots.append(s)
            self.by_name[n] = s
            off = _round_up(off + p.numel(), ALIGN)
        self.n_total = off
        self.weights = torch.zeros(self.n_total, device=device, dtype=dtype)
        self.grads = torch.zeros(self.n_train, device=device, dtype=torch.float32)
        self.params: Dict[str, nn.Parameter] = {}
        with torch.no_grad():
            for n, p in params:
                s = self.by_name[n]
                view = self.weights[s.offset:s.offset + s.numel].view(s.shape)
                view.copy_(p.detach().to(device=device, dtype=dtype))
                p.data = view
                if s.role != Role.FROZEN:
                    p.main_grad = self.grads[s.offset:s.offset + s.numel].view(s.shape)
                self.params[n] = p

    # ---- access by name (reference ParamStore::read_weight / write_weight / read_grad) ----
    def read_weight(self, name: str) -> torch.Tensor:
        s = self.by_name[name]
        return self.weights[s.offset:s.offset + s.numel].float().cpu()

    def write_weight(self, name: str, data) -> None:
        s = self.by_name[name]
        t = torch.as_tensor(data, dtype=torch.float32).reshape(-1)
        self.weights[s.offset:s.offset + s.numel].copy_(t.to(self.device, self.dtype))

    def read_grad(self, name: str) -> torch.Tensor:
        s = self.by_name[name]
        return self.grads[s.offset:s.offset + s.numel].clone().cpu()

    def zero_grads(self) -> None:
        self.grads.zero_()

    def collect_autograd_grads(self) -> None:
        """CPU backend: autograd leaves gradients in ``p.grad``; fold them into the flat buffer."""
        for n, p in self.params.items():
            if p.grad is not None:
                s = self.by_name[n]
                self.grads[s.offset:s.offset + s.numel].add_(p.grad.reshape(-1).float())
                p.grad = None

    def names(self, role: Optional[Role] = None) -> List[str]:
        return [s.name for s in self.slots if role is None or s.role == role]

    def decay_mask(self) -> Optional[torch.Tensor]:
        """fp32 0/1 per element of the trainable range, or None when every slot decays."""
        if all(s.decay for s in self.slots if s.role != Role.FROZEN):
            return None
        m = torch.zeros(self.n_train, device=self.device, dtype=torch.float32)
        for s in self.slots:
            if s.role != Role.FROZEN and s.decay:
                m[s.offset:s.offset + s.numel] = 1.0
        return m
