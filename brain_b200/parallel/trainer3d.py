"""Training over a tensor x pipeline (x data) grid: one process per GPU, each holding one pipeline
stage's layers sliced over its tensor-parallel group.

Step: zero the fp32 gradient bucket -> pipeline schedule (1F1B or GPipe) over the micro-batches,
with the fused all-gather->GEMM / GEMM->reduce-scatter kernels inside every block -> sum the
gradients of the tensors that are replicated inside a tensor-parallel group (embedding, head, norm
gains) and of a tied embedding across the first and last stage -> global gradient norm over the
whole model (each distinct value counted once) -> clip + AdamW on the local slice.

Reference: crates/model/src/shard.rs:355-652 (Pipeline with fused host AdamW, tied-weight sum) and
crates/model/tests/tensor_parallel.rs (the tensor-parallel primitives, which the reference never
wires into a full model); crates/model/src/grid.rs for the rank layout."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..optim.adamw import AdamW
from ..paramstore import ParamStore
from .grid import Grid, ProcessGroups
from .pipeline import PipelineStage
from .plan import ShardCost, plan_balanced


def even_bounds(n_layers: int, pp: int) -> List[int]:
    return [s * n_layers // pp for s in range(pp + 1)]


class Trainer3D:
    def __init__(self, cfg, grid: Grid, device, model_cls=None, impl: str = "fused", schedule: str = "1f1b",
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.1, grad_clip: Optional[float] = 1.0,
                 seed: int = 1234, dtype: Optional[torch.dtype] = None, full_state=None, arena_mb: int = 1024,
                 recompute: bool = False):
        from ..models.qwen3 import Qwen3
        from .tp import TensorParallel
        model_cls = model_cls or Qwen3
        self.grid = grid
        self.device = torch.device(device)
        cuda = self.device.type == "cuda"
        self.pgs = ProcessGroups(grid)
        self.rank = dist.get_rank()
        self.tp = None
        if grid.tp > 1:
            self.tp = TensorParallel(group=self.pgs.group("tp"), impl=impl if cuda else "nccl", device=self.device if cuda else None,
                                     arena_mb=arena_mb)
        # tied embeddings live on the first and the last stage: one 2-rank group per (tp, dp) column
        self.tied_group = None
        if grid.pp > 1 and cfg.tie_embeddings:
            for r in range(grid.world):
                t, p, d_ = grid.coord_of(r)
                if p == 0:
                    pair = [r, grid.rank_of(t, grid.pp - 1, d_)]
                    g = dist.new_group(pair)
                    if self.rank in pair:
                        self.tied_group = g
        stage = self.pgs.pp_coord
        bounds = even_bounds(cfg.n_layers, grid.pp)
        self.stage, self.bounds = stage, bounds
        dt = dtype or (torch.bfloat16 if cuda else torch.float32)
        if full_state is None and cuda:
            prev = torch.get_default_dtype()
            torch.set_default_dtype(dt)
            try:
                with torch.device(self.device):
                    model = model_cls(cfg, layers=range(bounds[stage], bounds[stage + 1]), first=stage == 0,
                                      last=stage == grid.pp - 1, tp=self.tp)
            finally:
                torch.set_default_dtype(prev)
            model.init_weights(seed)
        else:
            model = model_cls(cfg, layers=range(bounds[stage], bounds[stage + 1]), first=stage == 0,
                              last=stage == grid.pp - 1, tp=self.tp)
            if full_state is not None:
                model.load_full_state(full_state)
            else:
                model.init_weights(seed)
        self.model = model
        model.recompute_blocks = bool(recompute)    # keep block inputs only, re-run blocks in backward
        self.store = ParamStore(model, device=self.device, dtype=dt)
        self.opt = AdamW(self.store, betas=betas, eps=eps)
        self.wd, self.clip = weight_decay, grad_clip
        pp_ranks = self.pgs.ranks("pp")
        prev_r = pp_ranks[stage - 1] if stage > 0 else None
        next_r = pp_ranks[stage + 1] if stage < grid.pp - 1 else None
        self.pipe = PipelineStage(model, stage, grid.pp, prev_r, next_r, group=None, tied_group=self.tied_group,
                                  schedule=schedule, act_dtype=dt, row_div=grid.tp,
                                  group_fwd=self.pgs.group("pp_fwd"), group_bwd=self.pgs.group("pp_bwd"))
        self._replicated = [p for p in model.parameters() if getattr(p, "tp_replicated", False)]
        self.step_count = 0
        self.last_grad_norm = None

    # ------------------------------------------------------------------ pieces
    def _grad(self, p):
        g = getattr(p, "main_grad", None)
        return g if g is not None else p.grad

    def _sync_replicated(self):
        """Sum the partial gradients of tensor-parallel-replicated tensors over the group (one
        flattened all-reduce for the small ones, in place for the large ones)."""
        if self.tp is None or not self._replicated:
            return
        group = self.pgs.group("tp")
        small = [self._grad(p) for p in self._replicated if p.numel() < (1 << 20) and self._grad(p) is not None]
        big = [self._grad(p) for p in self._replicated if p.numel() >= (1 << 20) and self._grad(p) is not None]
        if small:
            flat = torch.cat([g.reshape(-1) for g in small])
            dist.all_reduce(flat, group=group)
            off = 0
            for g in small:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
        for g in big:
            dist.all_reduce(g, group=group)

    def _global_sumsq(self) -> torch.Tensor:
        """Sum of squares of every DISTINCT gradient value of the whole model: a tensor replicated
        over w tensor-parallel ranks (and a tied embedding held by two stages) counts once."""
        g = self.store.grads[: self.store.n_train]
        total = (g.double() ** 2).sum() if g.device.type == "cpu" else self.opt.grad_sumsq(g).double().clone().reshape(())
        w = self.grid.tp
        for p in self._replicated:
            gr = self._grad(p)
            if gr is None:
                continue
            copies = w * (2 if (p is self.model.tok and self.tied_group is not None) else 1)
            total = total - (gr.double() ** 2).sum() * (1.0 - 1.0 / copies)
        if self.tp is None and self.tied_group is not None and self.model.tok is not None:
            gr = self._grad(self.model.tok)
            total = total - (gr.double() ** 2).sum() * 0.5
        t = total.float().reshape(1)
        if dist.get_world_size() > 1:
            dist.all_reduce(t)
        # after the data-parallel reduction every replica holds the same gradients: count them once
        return t / float(self.grid.dp)

    # ------------------------------------------------------------------ step
    def train_step(self, micro_tokens: List[torch.Tensor], micro_targets: List[torch.Tensor], lr: float,
                   global_count: Optional[int] = None):
        """One optimiser step over the micro-batches (every rank passes the same lists; data-parallel
        replica r of ``dp`` takes micro-batches r, r+dp, ...).  Returns the mean loss (all ranks
        receive the same value)."""
        if global_count is None:
            global_count = sum(int((t >= 0).sum()) for t in micro_targets)
        dp = self.grid.dp
        if dp > 1:
            assert len(micro_tokens) % dp == 0, "the number of micro-batches must be a multiple of the dp degree"
            micro_tokens = micro_tokens[self.pgs.dp_coord::dp]
            micro_targets = micro_targets[self.pgs.dp_coord::dp]
        self.store.zero_grads()
        loss = self.pipe.forward_backward(micro_tokens, micro_targets, 1.0 / max(global_count, 1))
        if self.device.type == "cpu":
            self.store.collect_autograd_grads()
        self.pipe.sync_tied_embeddings()
        self._sync_replicated()
        if dp > 1:
            dist.all_reduce(self.store.grads[: self.store.n_train], group=self.pgs.group("dp"))
        ss = self._global_sumsq() if self.clip else None
        self.opt.step(lr, self.wd, self.clip, sumsq=ss)
        if self.opt.store.device.type == "cuda":
            from ..ops import _cuda
            _cuda.poll_error()
        if ss is not None:
            self.last_grad_norm = ss.sqrt()
        self.step_count += 1
        out = (loss if loss is not None else torch.zeros((), device=self.device)).detach().float().reshape(1).clone()
        if dist.get_world_size() > 1:
            dist.all_reduce(out)          # last-stage ranks hold partial sums over their rows; others zero
        return out


@torch.no_grad()
def gather_state(trainer: Trainer3D):
    """Full-model tensors under the reference names on rank 0 (None elsewhere): tensor-parallel
    slices are concatenated back, pipeline stages contribute their layers."""
    model, cfg = trainer.model, trainer.model.cfg
    w = trainer.grid.tp
    tp_group = trainer.pgs.group("tp")
    q, kv, ff, d = cfg.q_dim, cfg.kv_dim, cfg.d_ff, cfg.d_model
    ql, kl, fl = q // w, kv // w, ff // w
    local = {}

    def cat_tp(t, dim):
        if w == 1:
            return t.detach().float().cpu()
        parts = [torch.empty_like(t) for _ in range(w)]
        dist.all_gather(parts, t.detach().contiguous(), group=tp_group)
        return torch.cat(parts, dim=dim).float().cpu()
    if model.tok is not None:
        local["tok.weight"] = model.tok.detach().float().cpu()
    for lid, blk in zip(model.layer_ids, model.blocks):
        p = f"blocks.{lid}"
        local[f"{p}.ln1.weight"] = blk.ln1.detach().float().cpu()
        local[f"{p}.attn.wq.weight"] = cat_tp(blk.wqkv[:ql], 0)
        local[f"{p}.attn.wk.weight"] = cat_tp(blk.wqkv[ql:ql + kl], 0)
        local[f"{p}.attn.wv.weight"] = cat_tp(blk.wqkv[ql + kl:], 0)
        if blk.q_norm is not None:
            local[f"{p}.attn.q_norm.weight"] = blk.q_norm.detach().float().cpu()
            local[f"{p}.attn.k_norm.weight"] = blk.k_norm.detach().float().cpu()
        local[f"{p}.attn.wo.weight"] = cat_tp(blk.wo, 1)
        local[f"{p}.ln2.weight"] = blk.ln2.detach().float().cpu()
        local[f"{p}.mlp.gate.weight"] = cat_tp(blk.gate_up[:fl], 0)
        local[f"{p}.mlp.up.weight"] = cat_tp(blk.gate_up[fl:], 0)
        local[f"{p}.mlp.down.weight"] = cat_tp(blk.down, 1)
    if model.norm is not None:
        local["norm.weight"] = model.norm.detach().float().cpu()
    if model.lm_head is not None:
        local["lm_head.weight"] = model.lm_head.detach().float().cpu()
    gathered = [None] * dist.get_world_size()
    mine = local if trainer.pgs.tp_coord == 0 else {}
    dist.all_gather_object(gathered, mine)
    if dist.get_rank() != 0:
        return None
    out = {}
    for part in gathered:
        for k, v in part.items():
            out.setdefault(k, v)
    return {n: out[n].reshape(-1) for n, _ in cfg.param_list() if n in out}
