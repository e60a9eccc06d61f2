"""Training with expert parallelism: every rank is a data-parallel replica of the shared layers
(attention, norms, router, embedding) and owns E/world experts of every MoE layer; tokens travel to
their experts and back through the fused peer-memory dispatch/combine kernels inside the model.

Two parameter stores with two treatments:
  shared tensors  — gradients are summed over the ranks (one collective over the flat bucket),
  expert tensors  — gradients are already complete on the owner (every rank's tokens were
                    dispatched to it), nothing to reduce.
The gradient norm counts each distinct value once (shared bucket once, expert buckets summed over
ranks); one clip coefficient drives both AdamW instances.

The reference has no distributed expert parallelism (closest: checkpoint-level federated expert
shards, crates/federated/src/shard.rs); the layer math follows crates/model/src/moe.rs."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..optim.adamw import AdamW
from ..paramstore import ParamStore


def is_expert_param(name: str) -> bool:
    return ".moe.w_gate_up" in name or ".moe.w_down" in name


class TrainerEP:
    def __init__(self, model, device, group=None, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1,
                 grad_clip: Optional[float] = 1.0, dtype: Optional[torch.dtype] = None):
        self.model = model
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = torch.device(device)
        self.shared = ParamStore(model, device=self.device, dtype=dtype, select=lambda n: not is_expert_param(n))
        self.expert = ParamStore(model, device=self.device, dtype=dtype, select=is_expert_param)
        self.opt_shared = AdamW(self.shared, betas=betas, eps=eps)
        self.opt_expert = AdamW(self.expert, betas=betas, eps=eps)
        self.wd, self.clip = weight_decay, grad_clip
        self.cuda = self.device.type == "cuda"
        self.step_count = 0
        self.last_grad_norm = None

    def zero_grads(self):
        self.shared.zero_grads()
        self.expert.zero_grads()

    def forward_backward(self, tokens, targets, micro_batch: int, loss_scale: float):
        total = None
        for r0 in range(0, tokens.shape[0], micro_batch):
            tok = tokens[r0:r0 + micro_batch].to(self.device, non_blocking=True)
            tgt = targets[r0:r0 + micro_batch].to(self.device, non_blocking=True)
            loss = self.model.loss(tok, tgt, loss_scale)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if not self.cuda:
            self.shared.collect_autograd_grads()
            self.expert.collect_autograd_grads()
        return total

    def optimizer_step(self, lr: float):
        if self.world > 1:
            dist.all_reduce(self.shared.grads, group=self.group)
        ss = None
        if self.clip:
            gs, ge = self.shared.grads[: self.shared.n_train], self.expert.grads[: self.expert.n_train]
            if self.cuda:
                s_sh = self.opt_shared.grad_sumsq(gs).clone()
                s_ex = self.opt_expert.grad_sumsq(ge).clone()
            else:
                s_sh = (gs.double() ** 2).sum().float().reshape(1)
                s_ex = (ge.double() ** 2).sum().float().reshape(1)
            if self.world > 1:
                dist.all_reduce(s_ex, group=self.group)
            ss = s_sh + s_ex
            self.last_grad_norm = ss.sqrt()
        self.opt_shared.step(lr, self.wd, self.clip, sumsq=ss)
        self.opt_expert.step(lr, self.wd, self.clip, sumsq=ss)
        self.step_count += 1

    def train_step(self, tokens, targets, lr: float, micro_batch: Optional[int] = None,
                   global_count: Optional[int] = None):
        """One optimiser step on this rank's sequences; ``global_count`` = counted targets over all
        ranks (default: this rank's count x world)."""
        micro_batch = micro_batch or tokens.shape[0]
        if global_count is None:
            global_count = int((targets >= 0).sum()) * self.world
        self.zero_grads()
        loss = self.forward_backward(tokens, targets, micro_batch, 1.0 / max(global_count, 1))
        self.optimizer_step(lr)
        return loss
