"""LoRA adapters for the Qwen3 blocks: ``y += (alpha/r) * (x A^T) B^T`` on the targeted projections
with the base weights frozen (crates/qwen3/src/model.rs:1103-1150 forward/backward,
crates/model/src/lora.rs:30-153 host pair, :196-306 adapter files: ``save_adapter`` /
``fold_adapter_into``).  ``A`` [r, in] ~ N(0, 0.02), ``B`` [out, r] = 0, so training starts at the
base model.  Adapter tensors are named ``<target>.lora_a`` / ``<target>.lora_b``."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import functional as F
from .config import LoraCfg

#: target name -> (fused projection it lives in, (row_start, row_end) resolver)
_TARGETS = ("wq", "wk", "wv", "wo", "gate", "up", "down")


class BlockLora(nn.Module):
    def __init__(self, blk, cfg: LoraCfg, gen: torch.Generator):
        super().__init__()
        c = blk.cfg
        d, q, kv, ff = c.d_model, c.q_dim, c.kv_dim, c.d_ff
        self.scale = cfg.alpha / cfg.rank
        self.rank = cfg.rank
        # (fused name, row offset, rows, input dim)
        self.slices = {
            "wq": ("qkv", 0, q, d), "wk": ("qkv", q, kv, d), "wv": ("qkv", q + kv, kv, d),
            "wo": ("wo", 0, d, q), "gate": ("gate_up", 0, ff, d), "up": ("gate_up", ff, ff, d),
            "down": ("down", 0, d, ff),
        }
        self.targets: List[str] = [t for t in _TARGETS if t in cfg.targets]
        self.a = nn.ParameterDict()
        self.b = nn.ParameterDict()
        for t in self.targets:
            _, _, rows, din = self.slices[t]
            self.a[t] = nn.Parameter(torch.randn(cfg.rank, din, generator=gen) * 0.02)
            self.b[t] = nn.Parameter(torch.zeros(rows, cfg.rank))

    def add(self, blk, fused: str, x, y):
        """Add the adapter deltas of every target that lives in the fused projection ``fused``."""
        out = None
        for t in self.targets:
            f, r0, rows, _ = self.slices[t]
            if f != fused:
                continue
            a, b = self.a[t].to(x.dtype), self.b[t].to(x.dtype)
            delta = F.linear(F.linear(x, a), b) * self.scale
            if out is None:
                out = y.clone()
            out[:, r0:r0 + rows] += delta
        return y if out is None else out

    def reference_state(self, prefix: str) -> Dict[str, torch.Tensor]:
        names = {"wq": "attn.wq", "wk": "attn.wk", "wv": "attn.wv", "wo": "attn.wo",
                 "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}
        out = {}
        for t in self.targets:
            out[f"{prefix}.{names[t]}.lora_a"] = self.a[t]
            out[f"{prefix}.{names[t]}.lora_b"] = self.b[t]
        return out


def attach_lora(model, cfg: LoraCfg, seed: int = 1234, freeze_base: bool = True):
    """Give every block adapters for ``cfg.targets`` and freeze everything else."""
    if freeze_base:
        for p in model.parameters():
            p.requires_grad_(False)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    for blk in model.blocks:
        blk.lora = BlockLora(blk, cfg, gen)
    model.cfg.lora = cfg
    return model


def adapter_state(model) -> Dict[str, torch.Tensor]:
    return {n: t for n, t in model.reference_state().items()
            if n.endswith(".lora_a") or n.endswith(".lora_b")}


def save_adapter(path: str, model, base_id: str = "brain/qwen3", dataset_id: Optional[str] = None,
                 adapter_id: Optional[str] = None):
    """Write only the adapter tensors, config ``{rank, alpha, targets}``, and a card whose
    ``variant_of`` names the base (crates/model/src/lora.rs:196-240)."""
    from ..checkpoint import st
    from ..checkpoint.card import Adapter, ModelCard
    l = model.cfg.lora
    card = ModelCard(id=adapter_id or f"{base_id}-lora", family="qwen", variant_of=base_id,
                     adapter=Adapter("lora", l.rank, base_id, l.alpha, list(l.targets), dataset_id),
                     capabilities=["generate"])
    st.save(path, adapter_state(model), {"rank": l.rank, "alpha": l.alpha, "targets": list(l.targets)},
            card)


@torch.no_grad()
def fold_adapter_into(model, adapter_tensors: Dict[str, torch.Tensor], rank: int, alpha: float):
    """base += (alpha/rank) * B @ A for every adapted projection; returns the number folded."""
    ref = model.reference_state()
    n = 0
    scale = alpha / rank
    for name, a in adapter_tensors.items():
        if not name.endswith(".lora_a"):
            continue
        stem = name[: -len(".lora_a")]
        b = adapter_tensors[stem + ".lora_b"]
        w = ref[stem + ".weight"]
        A = a.reshape(rank, -1).float()
        B = b.reshape(-1, rank).float()
        w.add_((scale * (B @ A)).to(w.dtype).reshape(w.shape))
        n += 1
    return n


@torch.no_grad()
def fold_attached(model):
    """Fold a model's own attached adapters into its base weights and detach them."""
    st = adapter_state(model)
    l = model.cfg.lora
    n = fold_adapter_into(model, {k: v.detach() for k, v in st.items()}, l.rank, l.alpha)
    for blk in model.blocks:
        blk.lora = None
    model.cfg.lora = None
    return n
