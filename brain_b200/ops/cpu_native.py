"""Native part of the CPU backend (csrc/cpu/gemm.cpp): an AVX2 + FMA fp32 GEMM threaded over row
panels, used for the three products of a linear layer (forward x W^T, dX = dY W, dW = dY^T X) and a
row-parallel RMSNorm.  ``BRAIN_CPU_NATIVE=1`` routes the CPU path of ``ops.functional.linear``
through it; the PyTorch restatement in ``ops/reference.py`` stays the oracle the tests compare both
with.  Reference: crates/backend-cpu/src/fast_ops.rs, par.rs:27-83."""
from __future__ import annotations

import ctypes as c
import os

import torch

from .. import _host

_host.register({
    "bbh_cpu_gemm": (c.c_int, [c.c_void_p, c.c_void_p, c.c_void_p] + [c.c_int] * 8 + [c.c_float, c.c_float, c.c_int]),
    "bbh_cpu_rmsnorm": (c.c_int, [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_float, c.c_int]),
})

#: worker threads per call (0 = all hardware threads); thread data-parallel workers set this to their share
threads = int(os.environ.get("BRAIN_CPU_THREADS", "0"))


def enabled() -> bool:
    return os.environ.get("BRAIN_CPU_NATIVE") == "1"


def gemm(a: torch.Tensor, b: torch.Tensor, ta: bool = False, tb: bool = False, out=None, alpha: float = 1.0,
         beta: float = 0.0) -> torch.Tensor:
    """C = alpha * op(a) @ op(b) + beta * C for fp32 CPU matrices (rows may be strided)."""
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if ta else a.shape
    Kb, N = (b.shape[1], b.shape[0]) if tb else b.shape
    assert K == Kb, (a.shape, b.shape, ta, tb)
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32)
    rc = _host.lib().bbh_cpu_gemm(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                  out.stride(0), int(ta), int(tb), alpha, beta, threads)
    if rc != 0:
        raise RuntimeError(f"bbh_cpu_gemm failed ({rc})")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    y = torch.empty_like(x2)
    _host.lib().bbh_cpu_rmsnorm(x2.data_ptr(), w.contiguous().data_ptr(), y.data_ptr(), x2.shape[0], x2.shape[1],
                                float(eps), threads)
    return y.view(x.shape)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = gemm(x2, w.contiguous(), tb=True)
        if bias is not None:
            y += bias
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = gemm(dy2, w.contiguous()).view(ctx.shape) if ctx.needs_input_grad[0] else None
        dw = gemm(dy2, x2, ta=True) if ctx.needs_input_grad[1] else None
        db = dy2.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db


def linear(x, w, bias=None):
    return _Linear.apply(x, w, bias)
