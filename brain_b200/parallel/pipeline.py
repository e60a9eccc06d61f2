"""Pipeline parallelism: contiguous layer stages, micro-batched, point-to-point activations.

Each rank of the pipeline group holds one stage (a model built with ``layers=range(lo, hi)``,
``first``/``last`` flags).  ``train_step`` runs the per-stage op list of the chosen schedule
(``1f1b`` — warm-up forwards, then one-forward-one-backward, then drain — or ``gpipe``, the
reference's all-forward-then-all-backward): forward receives the residual stream ``[mb*T, d]`` from
the previous stage and sends its own on; backward receives the gradient of what it sent and sends
the gradient of what it received.  Transfers are ``torch.distributed`` p2p (NCCL on GPUs, gloo on
CPU ranks) on one communicator per direction; sends are asynchronous, and with ``BRAIN_PP_PREFETCH=1`` the
receive of the NEXT op of the schedule is posted before the current op computes, so a stage's transfers
run under its compute instead of in front of it (off by default: nothing to hide at the sizes measured).  Stage inputs are kept
for the backward; with ``model.recompute_blocks`` only block inputs are kept inside a stage and the
blocks are re-run in backward (the reference's re-materialisation).  With tied embeddings the first and last stage both hold
``tok.weight`` and sum its gradient before the optimiser step.

Reference: crates/model/src/shard.rs:355-652 (Pipeline, GPipe with recompute, fused host AdamW and
tied-weight sum); the 1F1B schedule is new here."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .plan import schedule as make_schedule


class PipelineStage:
    def __init__(self, model, stage: int, n_stages: int, prev_rank: Optional[int], next_rank: Optional[int],
                 group=None, tied_group=None, schedule: str = "1f1b", act_dtype=None, row_div: int = 1,
                 group_fwd=None, group_bwd=None):
        self.model, self.stage, self.n_stages = model, stage, n_stages
        self.prev, self.next = prev_rank, next_rank
        self.group, self.tied_group = group, tied_group
        # activations travel on group_fwd, gradients on group_bwd (both default to ``group``)
        self.group_fwd = group_fwd if group_fwd is not None else group
        self.group_bwd = group_bwd if group_bwd is not None else group
        self.schedule = schedule
        p = next(model.parameters())
        self.device = p.device
        self.act_dtype = act_dtype or p.dtype
        self.d_model = model.cfg.d_model
        self.row_div = row_div      # tensor-parallel degree: stages exchange [B*T/row_div, d] row shards
        self._pending: List = []
        # Receives are posted one op ahead (see forward_backward).  On NCCL a posted receive is a
        # kernel that spins until its data arrives, and two host-side events can then close a cycle
        # between neighbouring stages: (1) the first send/recv between two ranks on a communicator
        # blocks the HOST until the peer makes its first call too; (2) the first launch of a kernel
        # loads its module, which waits for running kernels -- such as that spinning receive.  So the
        # connections are made here, up front, and the first call of forward_backward (which launches
        # every kernel of the step for the first time) posts its receives only where it needs them.
        import os
        # Off by default: a stage-to-stage hop is ~10 MB (tens of microseconds on NVLink) against ~100 ms of
        # compute per micro-batch, and posting ahead measured 194.0k against 198.2k tok/s (0.6 B, PP=2).
        self.prefetch = os.environ.get("BRAIN_PP_PREFETCH", "0") == "1"
        self._warmed = False
        if self.device.type == "cuda" and dist.is_initialized():
            self._connect()

    def _connect(self):
        """One tiny exchange per neighbour and direction, so that no later p2p call sets up a connection."""
        one = torch.zeros(1, device=self.device, dtype=self.act_dtype)
        got = torch.empty_like(one)
        works = []
        if not self.last:
            works.append(dist.isend(one, dst=self.next, group=self.group_fwd))
        if not self.first:
            works.append(dist.irecv(got, src=self.prev, group=self.group_fwd))
        for w in works:
            w.wait()
        works = []
        if not self.first:
            works.append(dist.isend(one, dst=self.prev, group=self.group_bwd))
        if not self.last:
            works.append(dist.irecv(got, src=self.next, group=self.group_bwd))
        for w in works:
            w.wait()
        torch.cuda.synchronize(self.device)

    @property
    def first(self):
        return self.stage == 0

    @property
    def last(self):
        return self.stage == self.n_stages - 1

    def _post_recv(self, shape, src, group):
        """Start a receive; returns (work, buffer).  The caller waits right before the data is used."""
        buf = torch.empty(shape, device=self.device, dtype=self.act_dtype)
        return dist.irecv(buf, src=src, group=group), buf

    def _send(self, t, dst, group):
        self._pending.append((dist.isend(t.contiguous(), dst=dst, group=group), t))

    def _drain(self):
        for w, _ in self._pending:
            w.wait()
        self._pending.clear()

    def forward_backward(self, micro_tokens: List[torch.Tensor], micro_targets: List[torch.Tensor],
                         loss_scale: float):
        """Run this stage's schedule over the micro-batches.  ``micro_tokens`` is needed on the first
        stage (and for shapes everywhere), ``micro_targets`` on the last.  Returns the summed loss
        on the last stage (None elsewhere)."""
        n_micro = len(micro_tokens)
        ops = make_schedule(self.schedule, self.stage, self.n_stages, n_micro)

        def recv_spec(op):
            """(shape, source, group) of the transfer op needs before it can run, or None."""
            B, T = micro_tokens[abs(op) - 1].shape
            shape = (B * T // self.row_div, self.d_model)
            if op > 0:
                return None if self.first else (shape, self.prev, self.group_fwd)
            return None if self.last else (shape, self.next, self.group_bwd)

        posted = {}

        def post(i):
            if i < len(ops) and i not in posted:
                spec = recv_spec(ops[i])
                posted[i] = self._post_recv(*spec) if spec is not None else None

        def take(i):
            post(i)
            r = posted.pop(i)
            if r is None:
                return None
            r[0].wait()
            return r[1]

        stash = {}
        total = None
        ahead = self.prefetch and self._warmed
        self._warmed = True
        if ahead:
            post(0)
        for i, op in enumerate(ops):
            m = abs(op) - 1
            B, T = micro_tokens[m].shape
            got = take(i)
            if ahead:
                post(i + 1)      # the next op's input arrives while this op computes
            if op > 0:
                if self.first:
                    x_in = None
                    out = self.model.hidden(tokens=micro_tokens[m].to(self.device))
                else:
                    x_in = got.requires_grad_()
                    out = self.model.hidden(x_in=x_in, B=B, T=T)
                if self.last:
                    from ..ops import functional as F
                    tgt = micro_targets[m].to(self.device).reshape(-1)
                    if self.row_div > 1:
                        tgt = self.model.local_rows(tgt)
                    loss = F.lm_head_ce(out, self.model.head_weight(), tgt, loss_scale,
                                        self.model.ce_chunk_rows)
                    stash[m] = (x_in, loss)
                    total = loss.detach() if total is None else total + loss.detach()
                else:
                    self._send(out.detach(), self.next, self.group_fwd)
                    stash[m] = (x_in, out)
            else:
                x_in, out = stash.pop(m)
                if self.last:
                    out.backward()
                else:
                    out.backward(got)
                if not self.first:
                    self._send(x_in.grad, self.prev, self.group_bwd)
        self._drain()
        return total

    def sync_tied_embeddings(self):
        """Sum the gradient of ``tok.weight`` between the first and last stage (tied head)."""
        if self.tied_group is None or not self.model.cfg.tie_embeddings:
            return
        if not (self.first or self.last) or self.model.tok is None:
            return
        g = getattr(self.model.tok, "main_grad", None)
        if g is None:
            g = self.model.tok.grad
        if g is not None:
            dist.all_reduce(g, group=self.tied_group)


def build_stage_model(model_cls, cfg, stage: int, n_stages: int, bounds: List[int]):
    """Instantiate the stage's slice: layers [bounds[stage], bounds[stage+1])."""
    return model_cls(cfg, layers=range(bounds[stage], bounds[stage + 1]), first=stage == 0,
                     last=stage == n_stages - 1)
