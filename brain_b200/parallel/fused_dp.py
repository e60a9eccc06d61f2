"""Driver of the fused ZeRO step (csrc/comm/rs_adamw.cu): no NCCL call in the step.

    backward of the last micro-batch ──► per bucket, as soon as its parameters are complete:
        side stream: dp_bucket_kernel   every rank stages its bf16 copy of the bucket, the bucket's
                                        owner sums own fp32 + peers' bf16 over NVLink (rank order)
    after backward ──► dp_publish_norm  each rank's shard sum of squares to every peer
                       dp_adamw_ag      global clip coefficient, AdamW on the shard, new bf16 weights
                                        stored straight into every rank's weight buffer

Buckets never cross a rank's optimiser shard, so each has one owner and the optimiser state keeps its
contiguous per-rank layout.  Which parameters feed a bucket, and how many times each is accumulated
per backward (a tied embedding: twice), is learnt from the first step, which runs every bucket after
backward; later steps launch a bucket when its last expected accumulation of the last micro-batch
was issued.  A bucket that turns out to have been launched too early (an accumulation arrives after
it) is simply run again after backward.

``wire='fp32'`` keeps the first form: one reduce kernel over fp32 peer loads after backward,
bit-identical on every rank count to a rank-ordered fp32 sum.

The bf16 weights, the bf16 staging array (or, for fp32, the gradient bucket) and the signal words
live in a symmetric arena; the ParamStore's flat buffers are moved there when the engine is
attached."""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from ..ops import _cuda
from ..ops import functional as F
from ..ops._cuda import L, call, stream_ptr
from .symm import SymmArena, default_wait_seconds


def make_buckets(n: int, world: int, bucket_elems: int) -> List[Tuple[int, int, int]]:
    """[(owner, start, end)] covering [0, n): every rank's shard cut into pieces of at most
    ``bucket_elems`` elements (multiples of 8), listed from the END of the flat range to its start,
    which is the order backward completes them in."""
    assert n % (8 * world) == 0
    shard = n // world
    piece = max(8, bucket_elems // 8 * 8)
    out = []
    for r in range(world):
        a = r * shard
        while a < (r + 1) * shard:
            b = min(a + piece, (r + 1) * shard)
            out.append((r, a, b))
            a = b
    out.reverse()
    return out


class BucketTracker:
    """Decides, from the stream of "gradient of parameter p accumulated" notifications of the last
    micro-batch, when a bucket can be reduced.  Pure host logic (unit-tested on CPU)."""

    def __init__(self, buckets: List[Tuple[int, int, int]], slots: List[Tuple[int, int, int]]):
        """``slots``: (key, offset, numel) of every trainable parameter."""
        self.buckets = buckets
        self.of_param: Dict[int, List[int]] = {}
        for key, off, numel in slots:
            self.of_param[key] = [i for i, (_, a, b) in enumerate(buckets) if off < b and off + numel > a]
        self.expected: Dict[int, int] = {}      # accumulations per backward, learnt
        self.learnt = False
        self.begin()

    def begin(self):
        self.seen: Dict[int, int] = {}
        self.launched: List[int] = []
        self.late: set = set()
        self._pending = None
        if self.learnt:
            self._pending = [0] * len(self.buckets)
            for key, bs in self.of_param.items():
                for b in bs:
                    self._pending[b] += self.expected.get(key, 0)

    def notify(self, key: int) -> List[int]:
        """Buckets that became complete with this accumulation (in launch order)."""
        self.seen[key] = self.seen.get(key, 0) + 1
        ready = []
        if key not in self.of_param:
            return ready
        if not self.learnt:
            return ready
        over = self.seen[key] > self.expected.get(key, 0)
        for b in self.of_param[key]:
            if over:
                if b in self.launched:
                    self.late.add(b)        # reduced before this accumulation: run it again later
                continue
            self._pending[b] -= 1
            if self._pending[b] == 0 and b not in self.launched:
                ready.append(b)
        # keep the global launch order identical on every rank: buckets go out in list order only
        out = []
        for b in sorted(ready):
            out.append(b)
        self.launched.extend(out)
        return out

    def finish(self) -> List[int]:
        """Buckets still to run after backward (never launched, or launched too early), in list
        order; also folds what was seen into the expectations for the next step."""
        rest = [b for b in range(len(self.buckets)) if b not in self.launched or b in self.late]
        changed = (not self.learnt) or any(self.seen.get(k, 0) != self.expected.get(k, 0) for k in self.of_param)
        if changed:
            self.expected = {k: self.seen.get(k, 0) for k in self.of_param}
            self.learnt = True
        return rest


class FusedDP:
    def __init__(self, dp, store, opt, wait_seconds: float = None, wire: str = None,
                 bucket_mb: float = None, overlap_ctas: int = None):
        self.dp, self.store, self.opt = dp, store, opt
        self.world, self.rank = dp.world, dp.rank
        dev = store.device
        n = store.n_train
        assert n % (8 * self.world) == 0
        self.wire = (wire or os.environ.get("BRAIN_DP_WIRE", "bf16")).lower()
        assert self.wire in ("bf16", "fp32")
        lib = _cuda.lib()
        sig_bytes = int(lib.bb_dp_signal_bytes(self.world))
        need = (n * 2 if self.wire == "bf16" else n * 4) + store.n_total * 2 + sig_bytes + 8192
        self.arena = SymmArena(need, dev, dp.group)
        w = self.arena.alloc(store.n_total, store.dtype)
        self.sig = self.arena.alloc(sig_bytes // 8, torch.int64)
        w.copy_(store.weights)
        store.weights = w
        U64 = ctypes.c_uint64 * self.world
        if self.wire == "fp32":
            g = self.arena.alloc(n, torch.float32)
            g.copy_(store.grads)
            store.grads = g
            self.grad_ptrs = U64(*self.arena.peer_ptrs(g))
        else:
            self.stage = self.arena.alloc(n, torch.bfloat16)
            self.stage_ptrs = U64(*self.arena.peer_ptrs(self.stage))
        g = store.grads
        for name, p in store.params.items():
            s = store.by_name[name]
            p.data = w[s.offset:s.offset + s.numel].view(s.shape)
            if hasattr(p, "main_grad"):
                p.main_grad = g[s.offset:s.offset + s.numel].view(s.shape)
        self.w_ptrs = U64(*self.arena.peer_ptrs(w))
        self.sig_ptrs = U64(*self.arena.peer_ptrs(self.sig))
        self.scratch = torch.zeros(int(lib.bb_dp_scratch_floats()), device=dev, dtype=torch.float32)
        self.shard_g = torch.empty(opt.shard_len, device=dev, dtype=torch.float32)
        self.norm = torch.zeros(1, device=dev, dtype=torch.float32)
        self.decay_mask = None
        m = store.decay_mask()
        if m is not None:
            self.decay_mask = m[opt.lo:opt.hi].contiguous()
        self.epoch = 0
        self.wait_seconds = default_wait_seconds() if wait_seconds is None else float(wait_seconds)
        # ---- buckets (bf16 wire)
        if bucket_mb is None:
            bucket_mb = float(os.environ.get("BRAIN_DP_BUCKET_MB", "128"))
        self.buckets = make_buckets(n, self.world, int(bucket_mb * (1 << 20) / 4))
        owned = [i for i, (o, _, _) in enumerate(self.buckets) if o == self.rank]
        self.sumsq_slot = {b: k for k, b in enumerate(owned)}
        self.bucket_sumsq = torch.zeros(max(len(owned), 1), device=dev, dtype=torch.float32)
        from ..paramstore import Role
        slots = [(id(store.params[s.name]), s.offset, s.numel) for s in store.slots
                 if s.role != Role.FROZEN and s.name in store.params]
        self.tracker = BucketTracker(self.buckets, slots)
        self.seq = 0
        self.overlap_ctas = int(os.environ.get("BRAIN_DP_CTAS", "32")) if overlap_ctas is None else overlap_ctas
        self.side = torch.cuda.Stream(device=dev)
        # Overlap with backward pays when the reduce is long enough to be worth hiding: the bucket
        # kernels under backward are held to ``overlap_ctas`` CTAs and every bucket costs two event
        # hand-offs.  For a 0.6 B-parameter model the whole bf16 reduce-scatter is ~1 ms at 4 ranks:
        # there is nothing to hide, and the overlapped form measured 1 % behind the unfused NCCL arm at
        # 2 and 4 ranks.  ``auto`` turns the overlap on from 4 GB of fp32 gradients upwards.
        mode = os.environ.get("BRAIN_DP_OVERLAP", "auto").lower()
        self.overlap = mode in ("1", "on", "true") or (mode == "auto" and n * 4 >= (4 << 30))
        self._armed = False
        self.overlapped = 0          # buckets launched under backward in the last step (for reports)
        torch.cuda.synchronize(dev)
        dist.barrier(group=dp.group)

    # ------------------------------------------------------------------ overlap with backward
    def arm(self):
        """Called by the trainer right before the LAST micro-batch's forward/backward."""
        if self.wire != "bf16" or not self.overlap:
            return
        self.tracker.begin()
        self.overlapped = 0
        self._armed = True
        F.grad_ready_hook = self._on_grad

    def _on_grad(self, p):
        for b in self.tracker.notify(id(p)):
            # the accumulation kernels were issued on the current stream: the side stream starts
            # the bucket once they are done, while the current stream continues with backward
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self.side.wait_event(ev)
            with torch.cuda.stream(self.side):
                self._launch_bucket(b, self.overlap_ctas)
            self.overlapped += 1

    def _launch_bucket(self, b: int, max_ctas: int):
        owner, a, e = self.buckets[b]
        self.seq += 1
        opt = self.opt
        slot = self.sumsq_slot.get(b, 0)
        call("dp_bucket_reduce", self.store.grads, self.stage_ptrs, self.sig_ptrs, self.shard_g,
             self.bucket_sumsq[slot:], self.scratch, L(a), L(e - a), L(opt.lo), self.rank, self.world, owner,
             ctypes.c_ulonglong(self.seq), max_ctas, ctypes.c_double(self.wait_seconds), stream_ptr())

    # ------------------------------------------------------------------ the step
    def step(self, lr, wd, clip, extra_scale=1.0):
        opt = self.opt
        self.epoch += 1
        opt.t += 1
        if self.wire == "fp32":
            s = stream_ptr()
            call("dp_reduce", self.grad_ptrs, self.sig_ptrs, self.shard_g, self.scratch, L(opt.lo),
                 L(opt.shard_len), self.rank, self.world, ctypes.c_uint(self.epoch),
                 ctypes.c_double(self.wait_seconds), s)
        else:
            if F.grad_ready_hook is not None and self._armed:
                F.grad_ready_hook = None
            if not self._armed:
                self.tracker.begin()        # a step without arm(): everything runs now
            self._armed = False
            rest = self.tracker.finish()
            main = torch.cuda.current_stream()
            if rest:
                # same stream order on every rank: the leftovers follow the overlapped buckets
                ev = torch.cuda.Event()
                ev.record(main)
                self.side.wait_event(ev)
                with torch.cuda.stream(self.side):
                    for b in rest:
                        self._launch_bucket(b, 0)
            done = torch.cuda.Event()
            done.record(self.side)
            main.wait_event(done)
            s = stream_ptr()
            call("dp_publish_norm", self.sig_ptrs, self.bucket_sumsq, len(self.sumsq_slot), self.rank, self.world,
                 ctypes.c_uint(self.epoch), s)
        s = stream_ptr()
        call("dp_adamw_allgather", self.w_ptrs, self.sig_ptrs, opt.master, opt.m, opt.v,
             self.shard_g, self.decay_mask, self.norm, self.scratch, L(opt.lo), L(opt.shard_len),
             self.rank, self.world, ctypes.c_uint(self.epoch), float(lr), opt.beta1, opt.beta2,
             opt.eps, float(wd), opt.t, float(clip or 0.0), float(extra_scale),
             ctypes.c_double(self.wait_seconds), s)
        opt.last_grad_norm = self.norm
