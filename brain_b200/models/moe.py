"""Sparse top-k mixture-of-experts transformer.

``family='toymoe'``: the reference's trainable toy MoE (RMSNorm, fused qkv, interleaved RoPE,
softmax router with aux + z loss, SwiGLU experts, tied head; crates/toymoe/src/train.rs:147-167,
378-428).  ``family='qwen3_moe'``: the Qwen3-MoE decoder (GQA + QK-norm + NeoX RoPE attention as the
dense model, 128 experts / top-8 in the 30B-A3B shape; layer shape after
crates/qwen3omnimoe/src/thinker.rs:237-290, router/expert math crates/model/src/moe.rs:57-286).

Expert weights are stored stacked (``w_gate_up`` [E, 2*ff, d], ``w_down`` [E, d, ff]) so one grouped
GEMM serves all experts; checkpoints use per-expert names
``blocks.{l}.moe.experts.{e}.{w_gate,w_up,w_down}.weight`` (what the federated splitter keys on).
With an expert-parallel group each rank stores only its slice of the expert dimension."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn

from ..ops import functional as F
from ..ops import moe as moe_ops
from ..ops import reference as ref
from ..ops.attention import flash_attention
from .config import MoeConfig


class MoeLayer(nn.Module):
    def __init__(self, cfg: MoeConfig, ep=None):
        super().__init__()
        self.cfg = cfg
        self.ep = ep  # parallel.ep.ExpertParallel or None
        E = cfg.n_experts
        self.e_local = E // (ep.world if ep is not None else 1)
        self.e_first = self.e_local * (ep.rank if ep is not None else 0)
        d, ff = cfg.d_model, cfg.d_ff
        self.router = nn.Parameter(torch.empty(E, d))
        self.w_gate_up = nn.Parameter(torch.empty(self.e_local, 2 * ff, d))
        self.w_down = nn.Parameter(torch.empty(self.e_local, d, ff))
        self.last_aux = None
        self.last_counts = None

    def forward(self, x):
        """x: [n, d] -> ([n, d], aux_loss scalar)."""
        cfg = self.cfg
        y, aux, counts = moe_ops.moe_forward(
            x, self.router, self.w_gate_up, self.w_down, cfg.top_k, cfg.norm_topk_prob,
            cfg.routed_scaling, cfg.aux_coef, cfg.z_coef, ep=self.ep)
        self.last_aux, self.last_counts = aux.detach(), counts
        return y, aux


class MoeBlock(nn.Module):
    def __init__(self, cfg: MoeConfig, ep=None):
        super().__init__()
        self.cfg = cfg
        d = cfg.d_model
        self.ln1 = nn.Parameter(torch.ones(d))
        self.wqkv = nn.Parameter(torch.empty(cfg.q_dim + 2 * cfg.kv_dim, d))
        if cfg.family == "toymoe":
            self.q_norm = self.k_norm = None
        else:
            self.q_norm = nn.Parameter(torch.ones(cfg.head_dim))
            self.k_norm = nn.Parameter(torch.ones(cfg.head_dim))
        self.wo = nn.Parameter(torch.empty(d, cfg.q_dim))
        self.ln2 = nn.Parameter(torch.ones(d))
        self.moe = MoeLayer(cfg, ep)

    def forward(self, x, B, T, cos, sin, pos, recompute_experts=False):
        cfg = self.cfg
        hq, hk, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        h = F.rmsnorm(x, self.ln1, cfg.rms_eps)
        qkv = F.linear(h, self.wqkv)
        if cfg.family == "toymoe" and not qkv.is_cuda:
            n = qkv.shape[0]
            qk = ref.rope_interleaved(qkv[:, : (hq + hk) * hd].reshape(n, hq + hk, hd), cos, sin,
                                      pos.long()).reshape(n, -1)
        else:
            # the GPU path uses the half-split layout for both families (a fixed permutation of the
            # head dimension, which the learned projections absorb); checkpoints of the toy family
            # trained on CPU keep the interleaved convention
            qk = F.qknorm_rope(qkv, self.q_norm, self.k_norm, cos, sin, pos, hq, hk, hd, cfg.rms_eps)
        v = qkv[:, (hq + hk) * hd:]
        o = flash_attention(qk[:, : hq * hd], qk[:, hq * hd:], v, B, T, hq, hk, hd, causal=True)
        x = x + F.linear(o, self.wo)
        h2 = F.rmsnorm(x, self.ln2, cfg.rms_eps)
        if recompute_experts:
            # the routed rows and the experts' intermediates (top_k rows of d + 3*ff values per token)
            # are most of a block's activations: keep only the layer's input and run router, dispatch,
            # experts and combine again inside backward; the attention half keeps what it saved
            from torch.utils.checkpoint import checkpoint
            y, aux = checkpoint(self.moe, h2, use_reentrant=False)
        else:
            y, aux = self.moe(h2)
        return x + y, aux


class MoeModel(nn.Module):
    family = "moe"

    def __init__(self, cfg: MoeConfig, ep=None):
        super().__init__()
        self.cfg = cfg
        self.ep = ep
        d = cfg.d_model
        self.tok = nn.Parameter(torch.empty(cfg.vocab, d))
        self.blocks = nn.ModuleList([MoeBlock(cfg, ep) for _ in range(cfg.n_layers)])
        self.norm = nn.Parameter(torch.ones(d))
        self.lm_head = None if cfg.tie_embeddings else nn.Parameter(torch.empty(cfg.vocab, d))
        self._rope = None
        self.ce_chunk_rows = 8192
        self.last_aux = None

    @torch.no_grad()
    def init_weights(self, seed: int = 1234):
        g = torch.Generator(device="cpu").manual_seed(seed)
        std, pstd = 0.02, 0.02 / math.sqrt(2.0 * self.cfg.n_layers)

        def normal_(p, s):
            p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * s).to(p.dtype))

        normal_(self.tok, std)
        E = self.cfg.n_experts
        for blk in self.blocks:
            normal_(blk.wqkv, std)
            normal_(blk.wo, pstd)
            normal_(blk.moe.router, std)
            # draw the full expert stack so every EP rank gets the slice of one global init
            ff, d = self.cfg.d_ff, self.cfg.d_model
            m = blk.moe
            gu = torch.randn(E, 2 * ff, d, generator=g, dtype=torch.float32) * std
            dn = torch.randn(E, d, ff, generator=g, dtype=torch.float32) * pstd
            m.w_gate_up.copy_(gu[m.e_first:m.e_first + m.e_local].to(m.w_gate_up.dtype))
            m.w_down.copy_(dn[m.e_first:m.e_first + m.e_local].to(m.w_down.dtype))
        if self.lm_head is not None:
            normal_(self.lm_head, std)
        return self

    def rope_tables(self, device, n):
        n = max(n, self.cfg.block_size)
        if self._rope is None or self._rope[0].device != torch.device(device) or self._rope[0].shape[0] < n:
            self._rope = ref.rope_tables(n, self.cfg.head_dim, self.cfg.rope_theta, device=device)
        return self._rope

    def head_weight(self):
        return self.tok if self.cfg.tie_embeddings else self.lm_head

    def hidden(self, tokens):
        B, T = tokens.shape
        x = F.embedding(tokens.reshape(-1), self.tok).reshape(B * T, -1)
        cos, sin = self.rope_tables(x.device, T)
        pos = torch.arange(T, device=x.device, dtype=torch.int32).repeat(B)
        aux_total = None
        recompute = getattr(self, "recompute_blocks", False) and torch.is_grad_enabled()
        experts_only = getattr(self, "recompute_experts", False) and torch.is_grad_enabled() and not recompute
        for blk in self.blocks:
            if recompute:
                # activation recomputation: keep only the block input, re-run the block (including
                # its expert dispatch/combine, on every rank alike) inside backward
                from torch.utils.checkpoint import checkpoint
                x, aux = checkpoint(blk, x, B, T, cos, sin, pos, use_reentrant=False)
            else:
                x, aux = blk(x, B, T, cos, sin, pos, experts_only)
            aux_total = aux if aux_total is None else aux_total + aux
        return F.rmsnorm(x, self.norm, self.cfg.rms_eps), aux_total

    def forward(self, tokens, targets=None, loss_scale=None):
        B, T = tokens.shape
        h, aux = self.hidden(tokens)
        self.last_aux = aux.detach() if aux is not None else None
        if targets is None:
            return F.linear(h, self.head_weight()).reshape(B, T, -1)
        n_count = max(int((targets >= 0).sum()), 1) if loss_scale is None else None
        scale = loss_scale if loss_scale is not None else 1.0 / n_count
        ce = F.lm_head_ce(h, self.head_weight(), targets.reshape(-1), scale, self.ce_chunk_rows)
        # the auxiliary terms are per-batch means; weight them like the token loss of this batch
        frac = scale * float(B * T) if loss_scale is not None else 1.0
        return ce + aux * frac

    def loss(self, tokens, targets, loss_scale=None):
        return self.forward(tokens, targets, loss_scale)

    # ---- checkpoint names ----
    def reference_state(self) -> Dict[str, torch.Tensor]:
        cfg = self.cfg
        toy = cfg.family == "toymoe"
        out: Dict[str, torch.Tensor] = {"token_emb.weight" if toy else "tok.weight": self.tok}
        q, kv, ff = cfg.q_dim, cfg.kv_dim, cfg.d_ff
        for l, blk in enumerate(self.blocks):
            p = f"blocks.{l}"
            if toy:
                out[f"{p}.norm1.weight"] = blk.ln1
                out[f"{p}.attn.qkv.weight"] = blk.wqkv
                out[f"{p}.attn.out.weight"] = blk.wo
                out[f"{p}.norm2.weight"] = blk.ln2
            else:
                out[f"{p}.ln1.weight"] = blk.ln1
                out[f"{p}.attn.wq.weight"] = blk.wqkv[:q]
                out[f"{p}.attn.wk.weight"] = blk.wqkv[q:q + kv]
                out[f"{p}.attn.wv.weight"] = blk.wqkv[q + kv:]
                out[f"{p}.attn.q_norm.weight"] = blk.q_norm
                out[f"{p}.attn.k_norm.weight"] = blk.k_norm
                out[f"{p}.attn.wo.weight"] = blk.wo
                out[f"{p}.ln2.weight"] = blk.ln2
            m = blk.moe
            out[f"{p}.moe.router.weight"] = m.router
            for j in range(m.e_local):
                e = m.e_first + j
                out[f"{p}.moe.experts.{e}.w_gate.weight"] = m.w_gate_up[j, :ff]
                out[f"{p}.moe.experts.{e}.w_up.weight"] = m.w_gate_up[j, ff:]
                out[f"{p}.moe.experts.{e}.w_down.weight"] = m.w_down[j]
        out["norm.weight"] = self.norm
        if self.lm_head is not None:
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
        per_layer = 2 * (cfg.d_model * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * cfg.d_model
                         + cfg.d_model * cfg.n_experts + cfg.top_k * 3 * cfg.d_model * cfg.d_ff)
        attn = 4 * cfg.q_dim * T / 2
        total = cfg.n_layers * (per_layer + attn) + 2 * cfg.d_model * cfg.vocab
        return total * (3 if train else 1)
