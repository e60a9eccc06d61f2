"""Dense Qwen3 / Qwen2 decoder: RMSNorm, GQA with per-head QK-RMSNorm, half-split RoPE, SwiGLU,
tied or untied LM head (reference: crates/qwen3/src/model.rs:1157-1313 forward, :1345-1471 backward,
crates/qwen3/src/config.rs:311-366 parameter list).

Projection weights are stored fused (``wqkv`` = [wq; wk; wv], ``gate_up`` = [gate; up]) so one
tcgen05 GEMM produces q|k|v and gate|up; ``to_reference_state`` / ``load_reference_state`` split and
join them so checkpoints use the reference's tensor names."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn

from ..ops import functional as F
from ..ops import reference as ref
from ..ops.attention import attention_qkv, flash_attention
from .config import QwenConfig


class QwenBlock(nn.Module):
    def __init__(self, cfg: QwenConfig, tp=None):
        """``tp`` (a ``parallel.tp.TensorParallel`` of degree w > 1) shards the block the Megatron
        way with sequence parallelism: qkv and gate_up by output rows (heads / ff columns), wo and
        down by input columns; the residual stream, norms and their gains act on S/w rows.  The
        gains are replicated and marked ``tp_replicated`` so their gradients get summed over the
        group before the optimiser step."""
        super().__init__()
        d = cfg.d_model
        self.cfg = cfg
        self.tp = tp if tp is not None and tp.world > 1 else None
        w = self.tp.world if self.tp is not None else 1
        assert cfg.n_heads % w == 0 and cfg.n_kv_heads % w == 0 and cfg.d_ff % w == 0, \
            "tensor-parallel degree must divide the head counts and d_ff"
        self.hq, self.hk = cfg.n_heads // w, cfg.n_kv_heads // w
        q_dim, kv_dim, d_ff = cfg.q_dim // w, cfg.kv_dim // w, cfg.d_ff // w
        self.ff_local = d_ff
        self.ln1 = nn.Parameter(torch.ones(d))
        self.wqkv = nn.Parameter(torch.empty(q_dim + 2 * kv_dim, d))
        self.bqkv = nn.Parameter(torch.zeros(q_dim + 2 * kv_dim)) if cfg.attn_bias else None
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(cfg.head_dim))
            self.k_norm = nn.Parameter(torch.ones(cfg.head_dim))
        else:
            self.q_norm = self.k_norm = None
        self.wo = nn.Parameter(torch.empty(d, q_dim))
        self.ln2 = nn.Parameter(torch.ones(d))
        self.gate_up = nn.Parameter(torch.empty(2 * d_ff, d))
        self.down = nn.Parameter(torch.empty(d, d_ff))
        self.lora = None  # set by models.lora.attach
        if self.tp is not None:
            assert not cfg.attn_bias, "tensor-parallel blocks do not carry a qkv bias yet"
            for p in (self.ln1, self.ln2, self.q_norm, self.k_norm):
                if p is not None:
                    p.tp_replicated = True

    def attn(self, h, B, T, cos, sin, pos):
        cfg = self.cfg
        hq, hk, hd = self.hq, self.hk, cfg.head_dim
        if self.tp is not None:
            from ..parallel.tp import column_parallel_linear, row_parallel_linear
            qkv = column_parallel_linear(h, self.wqkv, self.tp)        # all-gather rows -> GEMM
            o = attention_qkv(qkv, self.q_norm, self.k_norm, cos, sin, pos, B, T, hq, hk, hd, cfg.rms_eps)
            return row_parallel_linear(o, self.wo, self.tp)            # GEMM -> reduce-scatter rows
        qkv = F.linear(h, self.wqkv, self.bqkv)
        if self.lora is not None:
            qkv = self.lora.add(self, "qkv", h, qkv)
        o = attention_qkv(qkv, self.q_norm, self.k_norm, cos, sin, pos, B, T, hq, hk, hd, cfg.rms_eps)
        y = F.linear(o, self.wo)
        if self.lora is not None:
            y = self.lora.add(self, "wo", o, y)
        return y

    def mlp(self, h):
        if self.tp is not None:
            from ..parallel.tp import column_parallel_linear, row_parallel_linear
            gu = column_parallel_linear(h, self.gate_up, self.tp)
            return row_parallel_linear(F.swiglu(gu), self.down, self.tp)
        gu = F.linear(h, self.gate_up)
        if self.lora is not None:
            gu = self.lora.add(self, "gate_up", h, gu)
        a = F.swiglu(gu)
        y = F.linear(a, self.down)
        if self.lora is not None:
            y = self.lora.add(self, "down", a, y)
        return y

    def forward(self, x, delta, B, T, cos, sin, pos):
        """x: residual stream, delta: pending branch output (added inside the fused norm)."""
        eps = self.cfg.rms_eps
        if delta is None:
            h = F.rmsnorm(x, self.ln1, eps)
        else:
            h, x = F.rmsnorm(delta, self.ln1, eps, residual=x)
        a = self.attn(h, B, T, cos, sin, pos)
        h2, x = F.rmsnorm(a, self.ln2, eps, residual=x)
        return x, self.mlp(h2)


class Qwen3(nn.Module):
    family = "qwen"

    def __init__(self, cfg: QwenConfig, layers: Optional[range] = None, first: bool = True,
                 last: bool = True, tp=None):
        """``layers``/``first``/``last`` select a pipeline stage (crates/qwen3/src/shard.rs:27-82):
        the first stage owns the embedding, the last owns the final norm and head (and a replica of
        ``tok.weight`` when embeddings are tied)."""
        super().__init__()
        self.cfg = cfg
        self.layer_ids = list(layers) if layers is not None else list(range(cfg.n_layers))
        self.first, self.last = first, last
        d = cfg.d_model
        if first or (last and cfg.tie_embeddings):
            self.tok = nn.Parameter(torch.empty(cfg.vocab, d))
        else:
            self.tok = None
        self.tp = tp if tp is not None and tp.world > 1 else None
        self.blocks = nn.ModuleList([QwenBlock(cfg, self.tp) for _ in self.layer_ids])
        if last:
            self.norm = nn.Parameter(torch.ones(d))
            self.lm_head = None if cfg.tie_embeddings else nn.Parameter(torch.empty(cfg.vocab, d))
        else:
            self.norm = None
            self.lm_head = None
        if self.tp is not None:
            # embedding, final norm and head are replicated inside the tensor-parallel group; each
            # rank applies them to its S/w rows, so their gradients are partial sums
            for p in (self.tok, self.norm, self.lm_head):
                if p is not None:
                    p.tp_replicated = True
        self._rope = None
        self.ce_chunk_rows = 8192

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def init_weights(self, seed: int = 1234):
        """N(0, 0.02); residual projections 0.02/sqrt(2L); norm gains 1
        (crates/qwen3/src/init.rs)."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        # sharded tensors draw from a per-rank stream, replicated ones from the shared stream
        gs = torch.Generator(device="cpu").manual_seed(seed + 7919 * (1 + self.tp.rank)) if self.tp is not None else g
        std = 0.02
        pstd = 0.02 / math.sqrt(2.0 * self.cfg.n_layers)

        def normal_(p, s, gen=None):
            gen = gen or g
            if p.is_cuda and p.numel() > (1 << 24):    # large tensors: draw on the device
                gd = torch.Generator(device=p.device).manual_seed(int(gen.initial_seed()) + p.numel() % 9973)
                p.normal_(0.0, s, generator=gd)
                return
            p.copy_((torch.randn(p.shape, generator=gen, dtype=torch.float32) * s).to(p.dtype))

        if self.tok is not None:
            normal_(self.tok, std)
        for blk in self.blocks:
            blk.ln1.fill_(1.0)
            blk.ln2.fill_(1.0)
            normal_(blk.wqkv, std, gs)
            if blk.bqkv is not None:
                blk.bqkv.zero_()
            if blk.q_norm is not None:
                blk.q_norm.fill_(1.0)
                blk.k_norm.fill_(1.0)
            normal_(blk.wo, pstd, gs)
            normal_(blk.gate_up, std, gs)
            normal_(blk.down, pstd, gs)
        if self.norm is not None:
            self.norm.fill_(1.0)
        if self.lm_head is not None:
            normal_(self.lm_head, std)
        return self

    # ------------------------------------------------------------------ forward
    def rope_tables(self, device, max_pos=None):
        n = max_pos or max(self.cfg.block_size, self.cfg.max_position_embeddings)
        if self._rope is None or self._rope[0].device != torch.device(device) or self._rope[0].shape[0] < n:
            self._rope = ref.rope_tables(n, self.cfg.head_dim, self.cfg.rope_theta, device=device)
        return self._rope

    def head_weight(self):
        return self.tok if self.cfg.tie_embeddings else self.lm_head

    def embed(self, tokens):
        B, T = tokens.shape
        return F.embedding(tokens.reshape(-1), self.tok).reshape(B * T, -1)

    def local_rows(self, t):
        """This rank's slice of a per-token tensor ``[B*T, ...]`` under tensor parallelism."""
        if self.tp is None:
            return t
        rows = t.shape[0] // self.tp.world
        return t[self.tp.rank * rows:(self.tp.rank + 1) * rows]

    def run_blocks(self, x, B, T, pos=None):
        """x: [B*T, d] (or this rank's [B*T/w, d] rows under tensor parallelism) -> (residual,
        pending delta)."""
        dev = x.device
        cos, sin = self.rope_tables(dev, T)
        if pos is None:
            pos = torch.arange(T, device=dev, dtype=torch.int32).repeat(B)
        delta = None
        recompute = getattr(self, "recompute_blocks", False) and torch.is_grad_enabled()
        for blk in self.blocks:
            if recompute:
                # activation re-materialisation (the pipeline of crates/model/src/shard.rs:551-652 keeps
                # only stage inputs and re-runs the forward in backward): keep the block's inputs only
                from torch.utils.checkpoint import checkpoint
                if delta is None:
                    x, delta = checkpoint(lambda a, blk=blk: blk(a, None, B, T, cos, sin, pos), x, use_reentrant=False)
                else:
                    x, delta = checkpoint(lambda a, d, blk=blk: blk(a, d, B, T, cos, sin, pos), x, delta, use_reentrant=False)
            else:
                x, delta = blk(x, delta, B, T, cos, sin, pos)
        return x, delta

    def hidden(self, tokens=None, x_in=None, B=None, T=None):
        """Stage forward: returns the residual stream [B*T, d] after this stage's blocks (final norm
        applied on the last stage)."""
        if self.first:
            B, T = tokens.shape
            if self.tp is not None:
                rows = (B * T) // self.tp.world
                assert rows * self.tp.world == B * T and rows % 128 == 0, \
                    "tensor parallel: B*T must split into multiples of 128 rows per rank"
                flat = tokens.reshape(-1)[self.tp.rank * rows:(self.tp.rank + 1) * rows]
                x = F.embedding(flat, self.tok).reshape(rows, -1)
            else:
                x = self.embed(tokens)
        else:
            x = x_in
        x, delta = self.run_blocks(x, B, T)
        if self.last:
            if delta is None:
                return F.rmsnorm(x, self.norm, self.cfg.rms_eps)
            h, _ = F.rmsnorm(delta, self.norm, self.cfg.rms_eps, residual=x)
            return h
        return x + delta if delta is not None else x

    def forward(self, tokens, targets=None, loss_scale=None, weights=None):
        """tokens [B,T] -> logits [B,T,V] (targets None) or the summed token loss * loss_scale
        (default 1/#counted targets, i.e. the mean); ``weights`` [B,T] multiplies each position's
        loss (weighted-loss training)."""
        B, T = tokens.shape
        h = self.hidden(tokens)
        w = self.head_weight()
        if targets is None:
            assert self.tp is None, "logits of a tensor-parallel model: use hidden() and gather the rows"
            return F.linear(h, w).reshape(B, T, -1)
        # under tensor parallelism h holds this rank's rows: the loss is this rank's partial sum
        wl = self.local_rows(weights.reshape(-1)) if weights is not None else None
        return F.lm_head_ce(h, w, self.local_rows(targets.reshape(-1)), loss_scale, self.ce_chunk_rows, wl)

    def loss(self, tokens, targets, loss_scale=None, weights=None):
        return self.forward(tokens, targets, loss_scale, weights)

    # ------------------------------------------------------------------ checkpoint naming
    def reference_state(self) -> Dict[str, torch.Tensor]:
        """Tensors under the reference's names (crates/qwen3/src/config.rs:311-366); fused
        projections are split into views."""
        cfg = self.cfg
        if self.tp is not None:
            raise RuntimeError("a tensor-parallel model holds slices: gather with parallel.trainer3d.gather_state")
        out: Dict[str, torch.Tensor] = {}
        if self.tok is not None:
            out["tok.weight"] = self.tok
        for lid, blk in zip(self.layer_ids, self.blocks):
            p = f"blocks.{lid}"
            q, kv = cfg.q_dim, cfg.kv_dim
            out[f"{p}.ln1.weight"] = blk.ln1
            out[f"{p}.attn.wq.weight"] = blk.wqkv[:q]
            out[f"{p}.attn.wk.weight"] = blk.wqkv[q:q + kv]
            out[f"{p}.attn.wv.weight"] = blk.wqkv[q + kv:]
            if blk.bqkv is not None:
                out[f"{p}.attn.wq.bias"] = blk.bqkv[:q]
                out[f"{p}.attn.wk.bias"] = blk.bqkv[q:q + kv]
                out[f"{p}.attn.wv.bias"] = blk.bqkv[q + kv:]
            if blk.q_norm is not None:
                out[f"{p}.attn.q_norm.weight"] = blk.q_norm
                out[f"{p}.attn.k_norm.weight"] = blk.k_norm
            out[f"{p}.attn.wo.weight"] = blk.wo
            out[f"{p}.ln2.weight"] = blk.ln2
            out[f"{p}.mlp.gate.weight"] = blk.gate_up[: cfg.d_ff]
            out[f"{p}.mlp.up.weight"] = blk.gate_up[cfg.d_ff:]
            out[f"{p}.mlp.down.weight"] = blk.down
            if blk.lora is not None:
                out.update(blk.lora.reference_state(p))
        if self.norm is not None:
            out["norm.weight"] = self.norm
        if self.lm_head is not None:
            out["lm_head.weight"] = self.lm_head
        return out

    @torch.no_grad()
    def load_reference_state(self, state: Dict[str, torch.Tensor], strict: bool = True):
        mine = self.reference_state()
        missing = []
        for name, dst in mine.items():
            if name not in state:
                missing.append(name)
                continue
            src = state[name]
            dst.copy_(src.reshape(dst.shape).to(dst.dtype))
        if strict and missing:
            raise KeyError(f"checkpoint is missing {len(missing)} tensors, e.g. {missing[:4]}")
        return missing

    @torch.no_grad()
    def load_full_state(self, state: Dict[str, torch.Tensor]):
        """Load this stage's (and, under tensor parallelism, this rank's) slice of a FULL model's
        tensors (reference names): q/k/v rows by head range, wo and down by input columns, gate/up
        by ff rows; replicated tensors whole."""
        cfg = self.cfg
        w = self.tp.world if self.tp is not None else 1
        r = self.tp.rank if self.tp is not None else 0
        d, q, kv, ff = cfg.d_model, cfg.q_dim, cfg.kv_dim, cfg.d_ff
        ql, kl, fl = q // w, kv // w, ff // w

        def get(name, shape):
            return state[name].reshape(shape)
        if self.tok is not None:
            self.tok.copy_(get("tok.weight", (cfg.vocab, d)))
        for lid, blk in zip(self.layer_ids, self.blocks):
            p = f"blocks.{lid}"
            blk.ln1.copy_(state[f"{p}.ln1.weight"].reshape(-1))
            blk.ln2.copy_(state[f"{p}.ln2.weight"].reshape(-1))
            blk.wqkv[:ql].copy_(get(f"{p}.attn.wq.weight", (q, d))[r * ql:(r + 1) * ql])
            blk.wqkv[ql:ql + kl].copy_(get(f"{p}.attn.wk.weight", (kv, d))[r * kl:(r + 1) * kl])
            blk.wqkv[ql + kl:].copy_(get(f"{p}.attn.wv.weight", (kv, d))[r * kl:(r + 1) * kl])
            if blk.q_norm is not None:
                blk.q_norm.copy_(state[f"{p}.attn.q_norm.weight"].reshape(-1))
                blk.k_norm.copy_(state[f"{p}.attn.k_norm.weight"].reshape(-1))
            blk.wo.copy_(get(f"{p}.attn.wo.weight", (d, q))[:, r * ql:(r + 1) * ql])
            blk.gate_up[:fl].copy_(get(f"{p}.mlp.gate.weight", (ff, d))[r * fl:(r + 1) * fl])
            blk.gate_up[fl:].copy_(get(f"{p}.mlp.up.weight", (ff, d))[r * fl:(r + 1) * fl])
            blk.down.copy_(get(f"{p}.mlp.down.weight", (d, ff))[:, r * fl:(r + 1) * fl])
        if self.norm is not None:
            self.norm.copy_(state["norm.weight"].reshape(-1))
        if self.lm_head is not None:
            self.lm_head.copy_(get("lm_head.weight", (cfg.vocab, d)))
        return self

    def config_json(self) -> dict:
        return self.cfg.to_json()

    def decayed(self, name: str) -> bool:
        """Weight decay applies to matrices, not to norm gains or biases."""
        return not (name.endswith("ln1") or name.endswith("ln2") or name.endswith("norm")
                    or name.endswith("q_norm") or name.endswith("k_norm") or "bqkv" in name)

    def flops_per_token(self, T: int, train: bool = True) -> float:
        """Model FLOPs per token (GEMMs + causal attention), x3 for fwd+bwd."""
        cfg = self.cfg
        per_layer = 2 * (cfg.d_model * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * cfg.d_model
                         + 3 * cfg.d_model * cfg.d_ff)
        attn = 4 * cfg.q_dim * T / 2
        total = len(self.layer_ids) * (per_layer + attn) + 2 * cfg.d_model * cfg.vocab
        return total * (3 if train else 1)
