"""Replicated data parallelism on the CPU backend, ranks as threads of one process.

``DataParallel``: one model replica per worker thread; ``forward_backward`` deals the
micro-batches round-robin (replica r takes r, r+n, ...), ``adamw_step`` all-reduces the flat
gradient through the native ``HostCollective`` (fixed rank order, bit-reproducible), runs ONE
AdamW on replica 0's flat buffers and broadcasts the new weights to every replica
(reference: crates/model/src/parallel.rs:69-134, 152-240).

``FlatAdam`` / ``DdpOptimizer``: the SPMD form — every rank all-reduces its flat gradient over any
``Collective`` and applies an identical AdamW; ``federated_average`` = FedAvg weighted by sample
count (crates/model/src/distributed.rs:33-101, 120-178)."""
from __future__ import annotations

import threading
from typing import Callable, List, Optional, Sequence

import torch

from ..optim.adamw import AdamW
from ..paramstore import ParamStore
from .collective import HostCollective


class DataParallel:
    def __init__(self, make_model: Callable[[], torch.nn.Module], n_workers: int = 2,
                 betas=(0.9, 0.999), eps: float = 1e-8):
        self.n = n_workers
        self.models = [make_model() for _ in range(n_workers)]
        # identical replicas: copy replica 0's weights into the rest
        sd = self.models[0].state_dict()
        for m in self.models[1:]:
            m.load_state_dict(sd)
        self.stores = [ParamStore(m, device="cpu") for m in self.models]
        self.coll = HostCollective.group(n_workers)
        self.opt = AdamW(self.stores[0], betas=betas, eps=eps)
        self.n_micro = 0
        self.last_losses: List[float] = []
        # the native CPU GEMM runs a worker pool per calling thread: give every replica its share of
        # the cores unless the user fixed the count, and so does PyTorch's own thread team (set per
        # replica thread in forward_backward): two teams of 8 on 8 cores cost a third of the throughput
        import os
        from ..ops import cpu_native
        self.threads_per_replica = max(1, (os.cpu_count() or 1) // n_workers)
        if cpu_native.enabled() and "BRAIN_CPU_THREADS" not in os.environ:
            cpu_native.threads = self.threads_per_replica

    def forward_backward(self, micro_batches: Sequence, loss_scale: Optional[float] = None) -> float:
        """``micro_batches``: list of (tokens, targets).  Gradients accumulate in each replica's
        flat buffer; returns the mean micro-batch loss."""
        for s in self.stores:
            s.zero_grads()
        losses = [0.0] * len(micro_batches)
        errors: List[BaseException] = []

        def work(r: int):
            try:
                torch.set_num_threads(self.threads_per_replica)   # per calling thread: this replica's share
                m, st = self.models[r], self.stores[r]
                for i in range(r, len(micro_batches), self.n):
                    tok, tgt = micro_batches[i]
                    loss = m.loss(tok, tgt, loss_scale)
                    loss.backward()
                    losses[i] = float(loss.detach())
                st.collect_autograd_grads()
            except BaseException as e:  # a failing replica must not leave the others waiting
                errors.append(e)
                self.coll[r].abort()

        ths = [threading.Thread(target=work, args=(r,)) for r in range(self.n)]
        for t in ths:
            t.start()
        for t in ths:
            t.join()
        if errors:
            raise errors[0]
        self.n_micro = len(micro_batches)
        self.last_losses = losses
        return sum(losses) / max(len(losses), 1)

    def adamw_step(self, lr: float, wd: float = 0.0, clip: Optional[float] = None):
        """sum gradients over replicas -> mean over micro-batches -> clip -> AdamW -> broadcast."""
        errors: List[BaseException] = []

        def reduce(r: int):
            try:
                self.coll[r].all_reduce(self.stores[r].grads)
            except BaseException as e:
                errors.append(e)

        ths = [threading.Thread(target=reduce, args=(r,)) for r in range(self.n)]
        for t in ths:
            t.start()
        for t in ths:
            t.join()
        if errors:
            raise errors[0]
        scale = 1.0 / max(self.n_micro, 1)
        self.opt.step(lr, wd, clip, extra_scale=scale)
        w0 = self.stores[0].weights
        for s in self.stores[1:]:
            s.weights.copy_(w0)

    def train_step(self, micro_batches, lr, wd=0.0, clip=None) -> float:
        loss = self.forward_backward(micro_batches)
        self.adamw_step(lr, wd, clip)
        return loss


class FlatAdam:
    """all-reduce(sum) -> mean -> clip -> AdamW on a flat fp32 vector; every rank runs it with the
    same inputs and gets the same weights."""

    def __init__(self, n: int, betas=(0.9, 0.999), eps=1e-8):
        self.m = torch.zeros(n)
        self.v = torch.zeros(n)
        self.t = 0
        self.betas, self.eps = betas, eps

    def step(self, coll, weights: torch.Tensor, grads: torch.Tensor, lr: float, wd: float = 0.0,
             clip: Optional[float] = None):
        from ..ops import reference as ref
        g = grads.clone()
        coll.all_reduce(g)
        g /= coll.world_size
        coef = 1.0
        if clip:
            coef = min(1.0, clip / (float(g.norm()) + 1e-6))
        self.t += 1
        ref.adamw_(weights, self.m, self.v, g, lr, self.betas[0], self.betas[1], self.eps, wd, self.t, coef)
        return weights


class DdpOptimizer:
    """Per-rank wrapper: flatten the model's gradients, ``FlatAdam.step``, scatter weights back."""

    def __init__(self, model: torch.nn.Module, coll, betas=(0.9, 0.999)):
        self.store = ParamStore(model, device="cpu")
        self.coll = coll
        self.adam = FlatAdam(self.store.n_train, betas)

    def zero_grads(self):
        self.store.zero_grads()

    def step(self, lr: float, wd: float = 0.0, clip: Optional[float] = None):
        self.store.collect_autograd_grads()
        self.adam.step(self.coll, self.store.weights[: self.store.n_train], self.store.grads, lr, wd, clip)


def fed_avg_flat(coll, weights: torch.Tensor, n_samples: float) -> torch.Tensor:
    """In-place FedAvg of a flat weight vector: sum_r n_r w_r / sum_r n_r (two all-reduces)."""
    w = weights * float(n_samples)
    coll.all_reduce(w)
    tot = torch.tensor([float(n_samples)])
    coll.all_reduce(tot)
    weights.copy_(w / tot)
    return weights


def federated_average(models: Sequence[torch.nn.Module], samples: Sequence[float]):
    """Weighted average of replicas' parameters, written back to every model."""
    total = float(sum(samples))
    with torch.no_grad():
        for ps in zip(*[m.parameters() for m in models]):
            avg = sum(p * (n / total) for p, n in zip(ps, samples))
            for p in ps:
                p.copy_(avg)
