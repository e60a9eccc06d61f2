"""Native part of the CPU backend: an fp32 GEMM (csrc/cpu/gemm.cpp; AVX2 + FMA, or the AVX-512 tile
chosen at run time) threaded over row blocks, used for the three products of a linear layer (forward
x W^T, dX = dY W, dW = dY^T X); a row-parallel RMSNorm; and softmax attention with grouped KV heads,
forward and backward (csrc/cpu/attention.cpp).  ``BRAIN_CPU_NATIVE=1`` routes the CPU paths of
``ops.functional.linear`` and ``ops.attention.flash_attention`` through them; the PyTorch restatement
in ``ops/reference.py`` stays the oracle the tests compare both with.
Reference: crates/backend-cpu/src/fast_ops.rs, par.rs:27-83."""
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


# ----------------------------------------------------------------------------------- attention
_host.register({
    "bbh_cpu_attn_fwd": (c.c_int, [c.c_void_p, c.c_int64] * 4 + [c.c_void_p] + [c.c_int] * 6 + [c.c_float, c.c_int, c.c_int]),
    "bbh_cpu_attn_bwd": (c.c_int, [c.c_void_p, c.c_int64] * 5 + [c.c_void_p] + [c.c_void_p, c.c_int64] * 3 + [c.c_int] * 6 +
                         [c.c_float, c.c_int, c.c_int]),
})


def attention_supported(q: torch.Tensor, hd: int, S: int = 0) -> bool:
    """fp32 and a head dimension that is a multiple of 8 (the kernels' vector width)."""
    return q.dtype == torch.float32 and hd % 8 == 0 and hd > 0


class _Attention(torch.autograd.Function):
    """Softmax attention with grouped KV heads on the native CPU kernels (csrc/cpu/attention.cpp):
    tiled with a running softmax, so no T x S score matrix exists at any point; backward recomputes
    the probabilities from the saved log-sum-exp."""

    @staticmethod
    def forward(ctx, q, k, v, B, T, S, hq, hk, hd, causal, scale):
        q2, k2, v2 = (t if t.stride(-1) == 1 and t.dim() == 2 else t.reshape(-1, t.shape[-1]).contiguous()
                      for t in (q, k, v))
        o = torch.empty(B * T, hq * hd, dtype=torch.float32)
        lse = torch.empty(B, hq, T, dtype=torch.float32)
        rc = _host.lib().bbh_cpu_attn_fwd(q2.data_ptr(), q2.stride(0), k2.data_ptr(), k2.stride(0), v2.data_ptr(),
                                          v2.stride(0), o.data_ptr(), o.stride(0), lse.data_ptr(), B, T, S, hq, hk,
                                          hd, float(scale), int(causal), threads)
        if rc != 0:
            raise RuntimeError(f"bbh_cpu_attn_fwd failed ({rc})")
        ctx.save_for_backward(q2, k2, v2, o, lse)
        ctx.dims = (B, T, S, hq, hk, hd, bool(causal), float(scale))
        return o

    @staticmethod
    def backward(ctx, do):
        q2, k2, v2, o, lse = ctx.saved_tensors
        B, T, S, hq, hk, hd, causal, scale = ctx.dims
        do2 = do if do.stride(-1) == 1 else do.contiguous()
        dq = torch.empty(B * T, hq * hd, dtype=torch.float32)
        dk = torch.empty(B * S, hk * hd, dtype=torch.float32)
        dv = torch.empty(B * S, hk * hd, dtype=torch.float32)
        rc = _host.lib().bbh_cpu_attn_bwd(q2.data_ptr(), q2.stride(0), k2.data_ptr(), k2.stride(0), v2.data_ptr(),
                                          v2.stride(0), o.data_ptr(), o.stride(0), do2.data_ptr(), do2.stride(0),
                                          lse.data_ptr(), dq.data_ptr(), dq.stride(0), dk.data_ptr(), dk.stride(0),
                                          dv.data_ptr(), dv.stride(0), B, T, S, hq, hk, hd, scale, int(causal), threads)
        if rc != 0:
            raise RuntimeError(f"bbh_cpu_attn_bwd failed ({rc})")
        return dq, dk, dv, None, None, None, None, None, None, None, None


def attention(q, k, v, B, T, S, hq, hk, hd, causal=True, scale=None):
    """q: [B*T, hq*hd]; k, v: [B*S, hk*hd] -> [B*T, hq*hd] (fp32, head dimension a multiple of 8)."""
    scale = 1.0 / (hd ** 0.5) if scale is None else scale
    return _Attention.apply(q, k, v, B, T, S, hq, hk, hd, causal, scale)
