"""ZeRO-style data parallelism: every rank holds the full bf16 working weights and an fp32 gradient
bucket; optimiser state (fp32 master, m, v) is sharded.  A step's communication is

    reduce-scatter(fp32 grads) -> global-norm clip -> sharded AdamW -> all-gather(bf16 weights)

``impl='nccl'`` is the baseline built from ``torch.distributed`` collectives and separate kernels;
``impl='fused'`` runs the hand-written NVLink kernels of ``csrc/comm/rs_adamw.cu`` over symmetric
peer memory (reduce-scatter by P2P loads fused with the cast/scale + AdamW update, weights pushed to
every peer by the same kernel).  CPU ranks (gloo) use the baseline path with the PyTorch optimiser.

Replaces the reference's host-staged data parallelism (crates/model/src/parallel.rs:152-240:
D2H every replica's grads, host sum, one host AdamW, H2D weights to every replica; and
crates/model/src/distributed.rs:58-89 ``FlatAdam::step`` = all-reduce + identical AdamW per rank)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class ZeroDP:
    def __init__(self, group=None, impl: str = "nccl"):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.impl = impl
        self.store = None
        self.opt = None
        self._fused = None

    def attach(self, store, opt):
        self.store, self.opt = store, opt
        if store.device.type == "cuda":
            self._shard_g = torch.empty(opt.shard_len, device=store.device, dtype=torch.float32)
        if self.impl == "fused":
            from .fused_dp import FusedDP
            self._fused = FusedDP(self, store, opt)

    def arm(self):
        """The trainer calls this right before the last micro-batch of a step: from here on every
        finished gradient may start its bucket's reduce-scatter (fused engine only)."""
        if self._fused is not None:
            self._fused.arm()

    def step(self, lr, wd, clip, extra_scale=1.0):
        st, opt = self.store, self.opt
        if self.world == 1:
            opt.step(lr, wd, clip, extra_scale)
            return
        if self._fused is not None:
            self._fused.step(lr, wd, clip, extra_scale)
            return
        n = st.n_train
        if st.device.type == "cuda":
            dist.reduce_scatter_tensor(self._shard_g, st.grads[:n], op=dist.ReduceOp.SUM,
                                       group=self.group)
            shard_g = self._shard_g
        else:
            # gloo has no reduce_scatter: all-reduce the bucket and slice this rank's shard
            dist.all_reduce(st.grads[:n], op=dist.ReduceOp.SUM, group=self.group)
            shard_g = st.grads[opt.lo:opt.hi]
        sumsq = opt.grad_sumsq(shard_g) if (clip is not None and clip > 0) else None
        opt.step(lr, wd, clip, extra_scale, grads=shard_g, sumsq=sumsq)
        w = st.weights[:n]
        if st.device.type == "cuda":
            dist.all_gather_into_tensor(w, w[opt.lo:opt.hi], group=self.group)
        else:
            parts = [torch.empty(opt.shard_len, dtype=w.dtype) for _ in range(self.world)]
            dist.all_gather(parts, w[opt.lo:opt.hi].clone(), group=self.group)
            for r, p in enumerate(parts):
                w[r * opt.shard_len:(r + 1) * opt.shard_len].copy_(p)
