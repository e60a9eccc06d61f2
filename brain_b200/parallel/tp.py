"""Tensor parallelism in the sequence-parallel Megatron layout.

Activations between layers are sharded by rows (``[S/tp, d]`` per rank); a column-parallel linear
all-gathers its input, a row-parallel linear reduce-scatters its output:

    column-parallel   Y[S, N/tp]  = all_gather(X[S/tp, K]) @ W_r^T        (AG -> GEMM)
    row-parallel      Y[S/tp, N]  = reduce_scatter(X[S, K/tp] @ W_r^T)    (GEMM -> RS)

``impl='fused'`` runs each of these as ONE tcgen05 GEMM launch whose collective half happens inside
the kernel over NVLink peer memory (``bb_gemm_bf16_tp``: data-mover CTAs + per-tile flags for the
all-gather side, per-destination TMA stores + a landed handshake for the reduce-scatter side; every
load is issued per CTA).  ``impl='nccl'`` is the baseline made of ``torch.distributed`` collectives and
separate GEMMs; CPU (gloo) ranks use the same baseline with PyTorch matmuls.

Reference: the column-/row-parallel MLP and attention-by-heads primitives of
crates/model/tests/tensor_parallel.rs:164-379 (one all-reduce per column->row pair) and the planner
crates/model/src/plan.rs:26-127."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as F


from .symm import default_wait_seconds


class TensorParallel:
    def __init__(self, group=None, impl: str = "nccl", device=None, arena_mb: int = 512,
                 wait_seconds: float = None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.impl = impl if self.world > 1 else "none"
        self.wait_seconds = default_wait_seconds() if wait_seconds is None else float(wait_seconds)
        self.epoch = 0
        self._slots = {}
        if self.impl == "fused":
            from ..ops import _cuda
            from .symm import SymmArena
            self.device = torch.device(device if device is not None else torch.cuda.current_device())
            self.arena = SymmArena(arena_mb << 20, self.device, group)
            self.sig = self.arena.alloc(2 * self.world, torch.int64)
            self.ar_sig = self.arena.alloc(self.world, torch.int64)
            self._U64 = ctypes.c_uint64 * self.world
            self.sig_ptrs = self._U64(*self.arena.peer_ptrs(self.sig))
            self.ar_sig_ptrs = self._U64(*self.arena.peer_ptrs(self.ar_sig))
            self.counter = torch.zeros(4, device=self.device, dtype=torch.int32)
            self.row_flags = torch.zeros(1 << 16, device=self.device, dtype=torch.int32)
            self.ar_epoch = 0
            self._cmaps = {}
            # two-shot all-reduce state: device-resident epoch (graph capture safe), own flags
            self.ar2_sig = self.arena.alloc(self.world, torch.int64)
            self.ar2_sig_ptrs = self._U64(*self.arena.peer_ptrs(self.ar2_sig))
            self.ar2_state = torch.zeros(4, device=self.device, dtype=torch.int32)   # [0] epoch, [1..3] counters
            self._ar2 = None
            self.ar2_calls = 0
            # in-switch (NVLS multimem) form of the same all-reduce: used when the arena is bound to
            # an NVLink multicast object and BRAIN_TP_NVLS=1; own flags and epoch word
            import os
            self.ag_copy_ctas = int(os.environ.get("BRAIN_TP_COPY_CTAS", "0"))   # 0: the kernel default (four per rank)
            self.nvls = os.environ.get("BRAIN_TP_NVLS") == "1" and self.arena.multicast_ptr(self.sig) != 0
            self.mm_sig = self.arena.alloc(self.world, torch.int64)
            self.mm_sig_ptrs = self._U64(*self.arena.peer_ptrs(self.mm_sig))
            self.mm_state = torch.zeros(4, device=self.device, dtype=torch.int32)

    # ------------------------------------------------------------------ symmetric slots
    def _slot(self, kind: str, numel: int, dtype, parity: int) -> torch.Tensor:
        key = (kind, numel, dtype, parity)
        t = self._slots.get(key)
        if t is None:
            t = self.arena.alloc(numel, dtype)
            self._slots[key] = t
        return t

    # ------------------------------------------------------------------ collectives (baseline)
    def all_gather_rows(self, x):
        if self.world == 1:
            return x
        out = torch.empty(self.world * x.shape[0], *x.shape[1:], device=x.device, dtype=x.dtype)
        if x.is_cuda:
            dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        else:
            parts = [torch.empty_like(x) for _ in range(self.world)]
            dist.all_gather(parts, x.contiguous(), group=self.group)
            out = torch.cat(parts)
        return out

    def reduce_scatter_rows(self, x):
        if self.world == 1:
            return x
        rows = x.shape[0] // self.world
        if x.is_cuda:
            out = torch.empty(rows, *x.shape[1:], device=x.device, dtype=x.dtype)
            dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
            return out
        y = x.clone()
        dist.all_reduce(y, group=self.group)
        return y[self.rank * rows:(self.rank + 1) * rows].contiguous()

    def all_reduce(self, x):
        """Sum over the TP group (serving: small activations -> one-shot peer kernel when fused)."""
        if self.world == 1:
            return x
        if self.impl == "fused" and x.is_cuda and x.dtype == torch.bfloat16 and \
                x.numel() % (8 * self.world) == 0:
            return self._all_reduce2(x)
        if self.impl == "fused" and x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
            from ..ops._cuda import L, call, stream_ptr
            self.ar_epoch += 1
            n = x.numel()
            buf = self._slot("ar", max(n, 1 << 16), torch.bfloat16, self.ar_epoch & 1)
            y = torch.empty_like(x)
            xc = x.contiguous()
            call("tp_allreduce", self._U64(*self.arena.peer_ptrs(buf)), self.ar_sig_ptrs, xc, y, L(n),
                 self.rank, self.world, ctypes.c_uint(self.ar_epoch), self.counter[1:],
                 ctypes.c_double(self.wait_seconds), stream_ptr())
            return y
        y = x.clone()
        dist.all_reduce(y, group=self.group)
        return y

    def ensure_ar2(self, n: int):
        """Symmetric staging + two result buffers of the two-shot all-reduce, holding >= ``n``
        elements (collective: every rank calls it with the same ``n``)."""
        if self._ar2 is None or self._ar2["cap"] < n:
            # grow by powers of two: the arena never frees, so a capacity that crept up with every
            # slightly longer prompt would eat it
            cap = max(1 << (int(n) - 1).bit_length(), 1 << 22)
            stage = self.arena.alloc(cap, torch.bfloat16)
            res = [self.arena.alloc(cap, torch.bfloat16) for _ in range(2)]
            self._ar2 = {"cap": cap, "stage": stage, "res": res,
                         "stage_ptrs": self._U64(*self.arena.peer_ptrs(stage)),
                         "res_ptrs": [self._U64(*self.arena.peer_ptrs(r)) for r in res]}
            if dist.is_initialized():
                dist.barrier(group=self.group)      # nobody signals into buffers that do not exist yet
        return self._ar2

    def _all_reduce2(self, x):
        """Two-shot peer-memory all-reduce; the result is a view of this rank's symmetric result
        buffer (two alternate, so a result stays valid across ONE later all-reduce)."""
        from ..ops._cuda import L, call, stream_ptr
        n = x.numel()
        st = self.ensure_ar2(n)
        which = self.ar2_calls & 1
        self.ar2_calls += 1
        xc = x.contiguous()
        if self.nvls:
            # the switch sums the ranks' staging buffers and writes the result into every rank's buffer
            call("tp_allreduce_mm", st["stage"], ctypes.c_void_p(self.arena.multicast_ptr(st["stage"])),
                 ctypes.c_void_p(self.arena.multicast_ptr(st["res"][which])), self.mm_sig_ptrs, xc, L(n), self.rank,
                 self.world, self.mm_state, self.mm_state[1:], ctypes.c_double(self.wait_seconds), stream_ptr())
            return st["res"][which][:n].view(x.shape)
        call("tp_allreduce2", st["stage_ptrs"], st["res_ptrs"][which], self.ar2_sig_ptrs, xc, L(n), self.rank,
             self.world, self.ar2_state, self.ar2_state[1:], ctypes.c_double(self.wait_seconds), stream_ptr())
        return st["res"][which][:n].view(x.shape)

    # ------------------------------------------------------------------ fused GEMM + collective
    def ag_gemm(self, x_shard, w):
        """(Y[S, N_local], X_full[S, K]) = all_gather(x_shard) @ w^T, w: [N_local, K]."""
        if self.world == 1:
            return F.linear(x_shard, w) if not x_shard.requires_grad else F.gemm(x_shard, w), x_shard
        rows, K = x_shard.shape
        if self.impl == "fused" and x_shard.is_cuda and rows % 128 == 0:
            from ..ops._cuda import call, stream_ptr
            self.epoch += 1
            send = self._slot("ag_send", rows * K, x_shard.dtype, self.epoch & 1).view(rows, K)
            send.copy_(x_shard)
            M = rows * self.world
            x_full = torch.empty(M, K, device=x_shard.device, dtype=x_shard.dtype)
            y = torch.empty(M, w.shape[0], device=x_shard.device, dtype=x_shard.dtype)
            call("gemm_bf16_tp", 1, x_full, w, y, M, w.shape[0], K, K, w.stride(0), y.stride(0),
                 self.rank, self.world, rows, self._U64(*self.arena.peer_ptrs(send)), self.row_flags,
                 self.ag_copy_ctas, self.sig_ptrs, ctypes.c_uint(self.epoch), None, None,
                 ctypes.c_double(self.wait_seconds), stream_ptr())
            return y, x_full
        x_full = self.all_gather_rows(x_shard)
        y = F.gemm(x_full, w) if x_full.is_cuda else x_full @ w.t()
        return y, x_full

    def gemm_rs(self, x, w, residual=None):
        """Y[S/tp, N] = reduce_scatter(x @ w^T) (+ residual); x: [S, K_local], w: [N, K_local]."""
        if self.world == 1:
            y = F.gemm(x, w) if x.is_cuda else x @ w.t()
            return y + residual if residual is not None else y
        M, K = x.shape
        N = w.shape[0]
        rows = M // self.world
        if self.impl == "fused" and x.is_cuda and rows % 128 == 0 and N % 8 == 0:
            from ..ops._cuda import L, call, stream_ptr
            self.epoch += 1
            par = self.epoch & 1
            recv = self._slot("rs_recv", M * N, x.dtype, par)
            key = (M, N, par)
            cm = self._cmaps.get(key)
            if cm is None:
                cm = torch.empty(128 * self.world, device=x.device, dtype=torch.uint8)
                call("tp_make_cmaps", cm, self._U64(*self.arena.peer_ptrs(recv)), self.world, M, N, N)
                self._cmaps[key] = cm
            call("gemm_bf16_tp", 2, x, w, None, M, N, K, x.stride(0), w.stride(0), N, self.rank,
                 self.world, rows, None, None, 0, self.sig_ptrs, ctypes.c_uint(self.epoch), cm,
                 self.counter, ctypes.c_double(self.wait_seconds), stream_ptr())
            y = torch.empty(rows, N, device=x.device, dtype=x.dtype)
            res = residual.contiguous() if residual is not None else None
            call("tp_sum_slots", recv, self.world, L(rows * N), res, y, stream_ptr())
            return y
        part = F.gemm(x, w) if x.is_cuda else x @ w.t()
        y = self.reduce_scatter_rows(part)
        return y + residual if residual is not None else y


# ------------------------------------------------------------------------------------ autograd
class _ColumnParallel(torch.autograd.Function):
    """Y[S, N/tp] = all_gather(X[S/tp, K]) W^T ; backward: dX = reduce_scatter(dY W), dW = dY^T X."""

    @staticmethod
    def forward(ctx, x_shard, w, tp):
        y, x_full = tp.ag_gemm(x_shard.detach(), w.detach())
        ctx.save_for_backward(x_full, w)
        ctx.tp, ctx.w_ref = tp, w
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        # dX_full = dy @ W  ->  reduce-scatter over rows; W^T as the "weight" of a row-parallel GEMM
        wt = w.t().contiguous()   # [K, N_local]: dX = dy . (W^T)^T
        dx = tp.gemm_rs(dy, wt)
        wp = ctx.w_ref
        mg = getattr(wp, "main_grad", None)
        if dy.is_cuda:
            if mg is not None:
                F.gemm(dy, x_full, a_mn=True, b_mn=True, out=mg, accumulate=True)
                F._notify(wp)
                dw = None
            else:
                dw = F.gemm(dy, x_full, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)
        else:
            dw = dy.t() @ x_full
        return dx, dw, None


class _RowParallel(torch.autograd.Function):
    """Y[S/tp, N] = reduce_scatter(X[S, K/tp] W^T); backward: dX = all_gather(dY) W, dW = dY_full^T X."""

    @staticmethod
    def forward(ctx, x, w, tp):
        y = tp.gemm_rs(x.detach(), w.detach())
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.w_ref = tp, w
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        wt = w.t().contiguous()   # [K_local, N]: dX = dY_full . W = dY_full . (W^T)^T
        dx, dy_full = tp.ag_gemm(dy_shard.contiguous(), wt)
        wp = ctx.w_ref
        mg = getattr(wp, "main_grad", None)
        if dy_full.is_cuda:
            if mg is not None:
                F.gemm(dy_full, x, a_mn=True, b_mn=True, out=mg, accumulate=True)
                F._notify(wp)
                dw = None
            else:
                dw = F.gemm(dy_full, x, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)
        else:
            dw = dy_full.t() @ x
        return dx, dw, None


def column_parallel_linear(x_shard, w, tp: TensorParallel):
    return _ColumnParallel.apply(x_shard, w, tp)


def row_parallel_linear(x, w, tp: TensorParallel):
    return _RowParallel.apply(x, w, tp)
