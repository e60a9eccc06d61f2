"""Driver of the fused ZeRO step (csrc/comm/rs_adamw.cu): two kernels per optimiser step, no NCCL
call — peer-load reduce-scatter + norm exchange, then clip + AdamW + peer-store all-gather.

The gradient bucket, the bf16 weights and the signal words live in a symmetric arena; the
ParamStore's flat buffers are moved there when the engine is attached."""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _cuda
from ..ops._cuda import L, call, stream_ptr
from .symm import SymmArena


from .symm import default_wait_seconds


class FusedDP:
    def __init__(self, dp, store, opt, wait_seconds: float = None):
        self.dp, self.store, self.opt = dp, store, opt
        self.world, self.rank = dp.world, dp.rank
        dev = store.device
        n = store.n_train
        assert n % (8 * self.world) == 0
        lib = _cuda.lib()
        sig_bytes = int(lib.bb_dp_signal_bytes(self.world))
        need = n * 4 + store.n_total * 2 + sig_bytes + 4096
        self.arena = SymmArena(need, dev, dp.group)
        # move the flat buffers into the arena and re-point every parameter view
        g = self.arena.alloc(n, torch.float32)
        w = self.arena.alloc(store.n_total, store.dtype)
        self.sig = self.arena.alloc(sig_bytes // 8, torch.int64)
        g.copy_(store.grads)
        w.copy_(store.weights)
        store.grads, store.weights = g, w
        for name, p in store.params.items():
            s = store.by_name[name]
            p.data = w[s.offset:s.offset + s.numel].view(s.shape)
            if hasattr(p, "main_grad"):
                p.main_grad = g[s.offset:s.offset + s.numel].view(s.shape)
        U64 = ctypes.c_uint64 * self.world
        self.grad_ptrs = U64(*self.arena.peer_ptrs(g))
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
        torch.cuda.synchronize(dev)
        dist.barrier(group=dp.group)

    def step(self, lr, wd, clip, extra_scale=1.0):
        opt = self.opt
        self.epoch += 1
        opt.t += 1
        s = stream_ptr()
        call("dp_reduce", self.grad_ptrs, self.sig_ptrs, self.shard_g, self.scratch, L(opt.lo),
             L(opt.shard_len), self.rank, self.world, ctypes.c_uint(self.epoch),
             ctypes.c_double(self.wait_seconds), s)
        call("dp_adamw_allgather", self.w_ptrs, self.sig_ptrs, opt.master, opt.m, opt.v,
             self.shard_g, self.decay_mask, self.norm, self.scratch, L(opt.lo), L(opt.shard_len),
             self.rank, self.world, ctypes.c_uint(self.epoch), float(lr), opt.beta1, opt.beta2,
             opt.eps, float(wd), opt.t, float(clip or 0.0), float(extra_scale),
             ctypes.c_double(self.wait_seconds), s)
        opt.last_grad_norm = self.norm
