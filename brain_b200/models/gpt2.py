"""nanoGPT-parity GPT-2: token + learned position embeddings, pre-LayerNorm blocks with fused
qkv(+bias) causal multi-head attention and a tanh-GELU MLP, final LayerNorm, untied ``lm_head``.
Reference: crates/gpt2/src/model.rs:275-302 (parameters), :561-614 (forward), :666-742 (backward),
crates/gpt2/src/init.rs:18-43 (init)."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn

from ..ops import functional as F
from ..ops.attention import flash_attention
from .config import GptConfig


class GptBlock(nn.Module):
    def __init__(self, cfg: GptConfig):
        super().__init__()
        d, ff = cfg.d_model, cfg.d_ff
        self.cfg = cfg
        self.ln1_w = nn.Parameter(torch.ones(d))
        self.ln1_b = nn.Parameter(torch.zeros(d))
        self.qkv_w = nn.Parameter(torch.empty(3 * d, d))
        self.qkv_b = nn.Parameter(torch.zeros(3 * d))
        self.out_w = nn.Parameter(torch.empty(d, d))
        self.out_b = nn.Parameter(torch.zeros(d))
        self.ln2_w = nn.Parameter(torch.ones(d))
        self.ln2_b = nn.Parameter(torch.zeros(d))
        self.fc_w = nn.Parameter(torch.empty(ff, d))
        self.fc_b = nn.Parameter(torch.zeros(ff))
        self.proj_w = nn.Parameter(torch.empty(d, ff))
        self.proj_b = nn.Parameter(torch.zeros(d))

    def forward(self, x, B, T):
        cfg = self.cfg
        d, H = cfg.d_model, cfg.n_heads
        hd = d // H
        h = F.layernorm(x, self.ln1_w, self.ln1_b, 1e-5)
        qkv = F.linear(h, self.qkv_w, self.qkv_b)
        o = flash_attention(qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:], B, T, H, H, hd, causal=True)
        x = x + F.linear(o, self.out_w, self.out_b)
        h = F.layernorm(x, self.ln2_w, self.ln2_b, 1e-5)
        x = x + F.linear(F.gelu(F.linear(h, self.fc_w, self.fc_b)), self.proj_w, self.proj_b)
        return x


class Gpt2(nn.Module):
    family = "gpt"

    def __init__(self, cfg: GptConfig, layers: Optional[range] = None, first: bool = True,
                 last: bool = True):
        super().__init__()
        self.cfg = cfg
        self.layer_ids = list(layers) if layers is not None else list(range(cfg.n_layers))
        self.first, self.last = first, last
        d = cfg.d_model
        if first:
            self.tok = nn.Parameter(torch.empty(cfg.vocab, d))
            self.pos = nn.Parameter(torch.empty(cfg.block_size, d))
        else:
            self.tok = self.pos = None
        self.blocks = nn.ModuleList([GptBlock(cfg) for _ in self.layer_ids])
        if last:
            self.ln_w = nn.Parameter(torch.ones(d))
            self.ln_b = nn.Parameter(torch.zeros(d))
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab, d))
        else:
            self.ln_w = self.ln_b = self.lm_head = None
        self.ce_chunk_rows = 8192

    @torch.no_grad()
    def init_weights(self, seed: int = 1337):
        g = torch.Generator(device="cpu").manual_seed(seed)
        std, pstd = 0.02, 0.02 / math.sqrt(2.0 * self.cfg.n_layers)

        def normal_(p, s):
            p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * s).to(p.dtype))

        if self.tok is not None:
            normal_(self.tok, std)
            normal_(self.pos, std)
        for b in self.blocks:
            for w in (b.qkv_w, b.fc_w):
                normal_(w, std)
            for w in (b.out_w, b.proj_w):
                normal_(w, pstd)
            for z in (b.qkv_b, b.out_b, b.fc_b, b.proj_b, b.ln1_b, b.ln2_b):
                z.zero_()
            b.ln1_w.fill_(1.0)
            b.ln2_w.fill_(1.0)
        if self.lm_head is not None:
            self.ln_w.fill_(1.0)
            self.ln_b.zero_()
            normal_(self.lm_head, std)
        return self

    def hidden(self, tokens=None, x_in=None, B=None, T=None):
        if self.first:
            B, T = tokens.shape
            x = F.embedding(tokens.reshape(-1), self.tok, self.pos, T).reshape(B * T, -1)
        else:
            x = x_in
        for blk in self.blocks:
            x = blk(x, B, T)
        if self.last:
            x = F.layernorm(x, self.ln_w, self.ln_b, 1e-5)
        return x

    def forward(self, tokens, targets=None, loss_scale=None):
        B, T = tokens.shape
        h = self.hidden(tokens)
        if targets is None:
            return F.linear(h, self.lm_head).reshape(B, T, -1)
        return F.lm_head_ce(h, self.lm_head, targets.reshape(-1), loss_scale, self.ce_chunk_rows)

    def loss(self, tokens, targets, loss_scale=None):
        return self.forward(tokens, targets, loss_scale)

    def head_weight(self):
        return self.lm_head

    # ---- checkpoint names (crates/gpt2/src/model.rs:275-302) ----
    def reference_state(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        if self.tok is not None:
            out["tok.weight"] = self.tok
            out["pos.weight"] = self.pos
        for lid, b in zip(self.layer_ids, self.blocks):
            p = f"blocks.{lid}"
            out.update({
                f"{p}.ln1.weight": b.ln1_w, f"{p}.ln1.bias": b.ln1_b,
                f"{p}.attn.qkv.weight": b.qkv_w, f"{p}.attn.qkv.bias": b.qkv_b,
                f"{p}.attn.out.weight": b.out_w, f"{p}.attn.out.bias": b.out_b,
                f"{p}.ln2.weight": b.ln2_w, f"{p}.ln2.bias": b.ln2_b,
                f"{p}.mlp.fc.weight": b.fc_w, f"{p}.mlp.fc.bias": b.fc_b,
                f"{p}.mlp.proj.weight": b.proj_w, f"{p}.mlp.proj.bias": b.proj_b,
            })
        if self.lm_head is not None:
            out["ln.weight"] = self.ln_w
            out["ln.bias"] = self.ln_b
            out["lm_head.weight"] = self.lm_head
        return out

    @torch.no_grad()
    def load_reference_state(self, state, strict: bool = True):
        missing = []
        for name, dst in self.reference_state().items():
            if name not in state:
                missing.append(name)
                continue
            dst.copy_(state[name].reshape(dst.shape).to(dst.dtype))
        if strict and missing:
            raise KeyError(f"checkpoint is missing {len(missing)} tensors, e.g. {missing[:4]}")
        return missing

    def config_json(self) -> dict:
        return self.cfg.to_json()

    def flops_per_token(self, T: int, train: bool = True) -> float:
        cfg = self.cfg
        per_layer = 2 * (4 * cfg.d_model * cfg.d_model + 2 * cfg.d_model * cfg.d_ff)
        attn = 4 * cfg.d_model * T / 2
        total = len(self.layer_ids) * (per_layer + attn) + 2 * cfg.d_model * cfg.vocab
        return total * (3 if train else 1)
