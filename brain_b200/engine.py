"""Training step engine: flat parameter store + (sharded) AdamW + micro-batched forward/backward.

One process per GPU.  A step is: zero the fp32 main-grad bucket, run the micro-batches (inputs are
copied from pinned host memory on a side stream), then the optimiser: on one GPU a gradient-norm +
AdamW pass; on N GPUs the ZeRO-style path in ``parallel.zero`` (reduce-scatter of the gradient
bucket, sharded AdamW, all-gather of the bf16 weights) — either the fused NVLink kernel or the
NCCL baseline.

Reference call stack: crates/model/src/train.rs:250-300 (per-step loop) and
crates/model/src/parallel.rs:114-240 (data-parallel forward_backward + adamw_step)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .optim.adamw import AdamW
from .paramstore import ParamStore


class Trainer:
    def __init__(self, model: nn.Module, device=None, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=0.1, grad_clip: Optional[float] = 1.0, dp=None, decay_fn=None,
                 dtype: Optional[torch.dtype] = None, offload_adam: Optional[bool] = None):
        """``dp``: a ``parallel.zero.ZeroDP`` (or None for a single replica).  ``offload_adam``
        keeps fp32 master weights and moments in host memory (default: env ``BRAIN_OFFLOAD_ADAM=1``)."""
        self.model = model
        self.dp = dp
        world = dp.world if dp is not None else 1
        self.store = ParamStore(model, device=device, dtype=dtype, pad_to=world, decay_fn=decay_fn)
        self.device = self.store.device
        shard = (dp.rank, world) if dp is not None else None
        if offload_adam is None:
            import os
            offload_adam = os.environ.get("BRAIN_OFFLOAD_ADAM") == "1"
        if offload_adam and dp is None:
            from .optim.offload import OffloadAdam
            self.opt = OffloadAdam(self.store, betas=betas, eps=eps)
        else:
            self.opt = AdamW(self.store, betas=betas, eps=eps, shard=shard,
                             group=dp.group if dp is not None else None)
        if dp is not None:
            dp.attach(self.store, self.opt)
        self.wd = weight_decay
        self.clip = grad_clip
        self.cuda = self.device.type == "cuda"
        self._copy_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.step_count = 0

    # ------------------------------------------------------------------ pieces
    def zero_grads(self):
        self.store.zero_grads()

    def _to_device(self, t):
        if not self.cuda or t.is_cuda:
            return t
        return t.to(self.device, non_blocking=True)

    def forward_backward(self, tokens, targets, micro_batch: int, loss_scale: float, weights=None):
        """Accumulate gradients of sum(token losses) * loss_scale over the rows of ``tokens``
        (``weights``: per-position loss weights, models that take them).  Returns the accumulated
        (device) loss."""
        B = tokens.shape[0]
        total = None
        for r0 in range(0, B, micro_batch):
            if r0 + micro_batch >= B and self.dp is not None and hasattr(self.dp, "arm"):
                self.dp.arm()       # last micro-batch: finished gradient buckets may be reduced under backward
            tok = self._to_device(tokens[r0:r0 + micro_batch])
            tgt = self._to_device(targets[r0:r0 + micro_batch])
            if weights is not None:
                loss = self.model.loss(tok, tgt, loss_scale, self._to_device(weights[r0:r0 + micro_batch]))
            else:
                loss = self.model.loss(tok, tgt, loss_scale)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if not self.cuda:
            self.store.collect_autograd_grads()
        return total

    def optimizer_step(self, lr: float, extra_scale: float = 1.0):
        if self.dp is not None:
            self.dp.step(lr, self.wd, self.clip, extra_scale)
        else:
            self.opt.step(lr, self.wd, self.clip, extra_scale)
        self.step_count += 1
        if self.cuda:
            # a kernel whose bounded wait ran out skipped its work: stop instead of training on
            # garbage (non-blocking; reports the previous step's kernels)
            from .ops import _cuda
            _cuda.poll_error()

    def train_step(self, tokens, targets, lr: float, micro_batch: Optional[int] = None,
                   global_count: Optional[int] = None):
        """One optimiser step on this rank's rows.  ``global_count`` = number of counted targets in
        the whole (all ranks) batch; defaults to this rank's count times the DP world size."""
        if micro_batch is None:
            micro_batch = tokens.shape[0]
        if global_count is None:
            local = int((targets >= 0).sum())
            global_count = local * (self.dp.world if self.dp is not None else 1)
        self.zero_grads()
        loss = self.forward_backward(tokens, targets, micro_batch, 1.0 / max(global_count, 1))
        self.optimizer_step(lr)
        return loss
