"""The library arm of the benchmarks: the SAME Qwen3 architecture written with stock PyTorch only —
``F.linear`` (cuBLAS), ``F.scaled_dot_product_attention`` (cuDNN / flash), ``F.rms_norm``,
``F.cross_entropy``, ``torch.optim.AdamW(fused=True)``, ``clip_grad_norm_`` and, on several GPUs,
``DistributedDataParallel`` over NCCL.  fp32 parameters under ``torch.autocast(bfloat16)``.

None of this repository's kernels, its parameter store or its engine are on this path.  It is NOT the
reference project (a Rust / wgpu workspace that cannot be built on this box); it is the anchor a
PyTorch user would compare against on the same GPU, reported beside the native numbers."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def _rope_tables(T: int, hd: int, theta: float, device):
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))
    ang = torch.arange(T, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def _rope(x, cos, sin):
    # x [B, H, T, hd], NeoX layout: (first half, second half) pairs
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    c, s = cos[None, None].to(x.dtype), sin[None, None].to(x.dtype)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


class Block(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        d, hq, hk, hd = cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        self.hq, self.hk, self.hd, self.eps = hq, hk, hd, cfg.rms_eps
        self.ln1 = nn.Parameter(torch.ones(d))
        self.ln2 = nn.Parameter(torch.ones(d))
        self.wqkv = nn.Linear(d, (hq + 2 * hk) * hd, bias=False)
        self.wo = nn.Linear(hq * hd, d, bias=False)
        self.q_norm = nn.Parameter(torch.ones(hd))
        self.k_norm = nn.Parameter(torch.ones(hd))
        self.gate_up = nn.Linear(d, 2 * cfg.d_ff, bias=False)
        self.down = nn.Linear(cfg.d_ff, d, bias=False)

    def forward(self, x, cos, sin):
        B, T, d = x.shape
        hq, hk, hd = self.hq, self.hk, self.hd
        h = F.rms_norm(x, (d,), self.ln1.to(x.dtype), self.eps)
        qkv = self.wqkv(h)
        q, k, v = qkv.split([hq * hd, hk * hd, hk * hd], dim=-1)
        q = F.rms_norm(q.view(B, T, hq, hd), (hd,), self.q_norm.to(q.dtype), self.eps).transpose(1, 2)
        k = F.rms_norm(k.view(B, T, hk, hd), (hd,), self.k_norm.to(k.dtype), self.eps).transpose(1, 2)
        v = v.view(B, T, hk, hd).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + self.wo(o.transpose(1, 2).reshape(B, T, hq * hd))
        h = F.rms_norm(x, (d,), self.ln2.to(x.dtype), self.eps)
        g, u = self.gate_up(h).chunk(2, dim=-1)
        return x + self.down(F.silu(g) * u)


class TorchQwen3(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.tok = nn.Embedding(cfg.vocab, cfg.d_model)
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(cfg.n_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.d_model))
        nn.init.normal_(self.tok.weight, std=0.02)
        for p in self.parameters():
            if p.dim() == 2 and p is not self.tok.weight:
                nn.init.normal_(p, std=0.02)

    def loss(self, tokens, targets, scale: float):
        """sum of token losses * scale (tied LM head), as the native model's ``loss``."""
        cfg = self.cfg
        B, T = tokens.shape
        cos, sin = _rope_tables(T, cfg.head_dim, cfg.rope_theta, tokens.device)
        x = self.tok(tokens.long())
        for blk in self.blocks:
            x = blk(x, cos, sin)
        x = F.rms_norm(x, (cfg.d_model,), self.norm.to(x.dtype), cfg.rms_eps)
        logits = F.linear(x, self.tok.weight)
        return F.cross_entropy(logits.view(B * T, -1).float(), targets.long().view(-1), reduction="sum") * scale


class TorchlibTrainer:
    """train_step(tokens, targets, lr, micro_batch, global_count) with the native Trainer's signature."""

    def __init__(self, cfg, device, world: int = 1, betas=(0.9, 0.95), weight_decay=0.1, grad_clip=1.0):
        torch.manual_seed(0)
        self.device = device
        self.model = TorchQwen3(cfg).to(device)
        self.net = self.model
        self.world = world
        if world > 1:
            from torch.nn.parallel import DistributedDataParallel as DDP
            self.ddp = DDP(self.model, device_ids=[device.index] if device.type == "cuda" else None,
                           gradient_as_bucket_view=True)
        else:
            self.ddp = None
        decay = [p for p in self.model.parameters() if p.dim() == 2]
        rest = [p for p in self.model.parameters() if p.dim() != 2]
        self.opt = torch.optim.AdamW([{"params": decay, "weight_decay": weight_decay},
                                      {"params": rest, "weight_decay": 0.0}], lr=1e-3, betas=betas,
                                     fused=device.type == "cuda")
        self.clip = grad_clip

    def _loss(self, tok, tgt, scale):
        # through DDP's forward (= the module's loss) so its gradient hooks are armed for this backward
        with torch.autocast(self.device.type, dtype=torch.bfloat16):
            return (self.ddp if self.ddp is not None else self.model)(tok, tgt, scale)

    def train_step(self, tokens, targets, lr, micro_batch=None, global_count=None):
        B = tokens.shape[0]
        micro_batch = micro_batch or B
        if global_count is None:
            global_count = int((targets >= 0).sum()) * self.world
        # DDP averages over ranks: scale so that the summed, averaged gradient is the global mean's
        scale = (self.world if self.ddp is not None else 1) / max(global_count, 1)
        for g in self.opt.param_groups:
            g["lr"] = lr
        self.opt.zero_grad(set_to_none=False)
        total = None
        n_micro = (B + micro_batch - 1) // micro_batch
        for i, r0 in enumerate(range(0, B, micro_batch)):
            tok = tokens[r0:r0 + micro_batch].to(self.device, non_blocking=True)
            tgt = targets[r0:r0 + micro_batch].to(self.device, non_blocking=True)
            if self.ddp is not None and i != n_micro - 1:
                with self.ddp.no_sync():
                    loss = self._loss(tok, tgt, scale)
                    loss.backward()
            else:
                loss = self._loss(tok, tgt, scale)
                loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if self.clip:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.clip, foreach=True)
        self.opt.step()
        return total / (self.world if self.ddp is not None else 1)


TorchQwen3.forward = TorchQwen3.loss    # DDP calls forward(); the module's forward IS the loss
