"""Attention ops: flash attention for training/prefill (tcgen05 kernels) and the CPU reference.

Layout convention everywhere: activations are ``[tokens, heads*head_dim]`` rows (token-major), so
the q/k/v inputs may be column slices of one fused projection output (row pitch = ``stride(0)``).
"""
from __future__ import annotations

import math

import torch

from . import reference as ref
from ._cuda import call, stream_ptr


def _rows(x):
    assert x.dim() == 2 and x.stride(1) == 1
    return x


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, B, T, S, hq, hk, hd, causal, scale):
        q, k, v = _rows(q), _rows(k), _rows(v)
        out = torch.empty(B * T, hq * hd, device=q.device, dtype=q.dtype)
        lse = torch.empty(B, hq, T, device=q.device, dtype=torch.float32)
        call("flash_fwd", q, q.stride(0), k, k.stride(0), v, v.stride(0), out, out.stride(0), lse,
             B, T, S, hq, hk, hd, float(scale), int(causal), stream_ptr())
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.dims = (B, T, S, hq, hk, hd, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        B, T, S, hq, hk, hd, causal, scale = ctx.dims
        dout = dout.contiguous()
        dq = torch.empty(B * T, hq * hd, device=q.device, dtype=q.dtype)
        dk = torch.empty(B * S, hk * hd, device=q.device, dtype=q.dtype)
        dv = torch.empty(B * S, hk * hd, device=q.device, dtype=q.dtype)
        delta = torch.empty(B, hq, T, device=q.device, dtype=torch.float32)
        call("flash_bwd", q, q.stride(0), k, k.stride(0), v, v.stride(0), out, out.stride(0), dout,
             dout.stride(0), lse, delta, dq, dq.stride(0), dk, dk.stride(0), dv, dv.stride(0),
             B, T, S, hq, hk, hd, float(scale), int(causal), stream_ptr())
        return dq, dk, dv, None, None, None, None, None, None, None, None


class _AttnQKV(torch.autograd.Function):
    """QK-norm + RoPE + causal flash attention over one fused ``qkv`` buffer.  One autograd node
    instead of three slices, a rope op and an attention op: the backward kernels write dq/dk into
    one scratch buffer, dv straight into its columns of ``d_qkv``, and the rope backward fills the
    q|k columns of the same ``d_qkv`` — no zero fills, slice copies or gradient adds in between."""

    @staticmethod
    def forward(ctx, qkv, w_q, w_k, cos, sin, pos, B, T, hq, hk, hd, eps, scale):
        n = qkv.shape[0]
        qkw = (hq + hk) * hd
        qk = torch.empty(n, qkw, device=qkv.device, dtype=qkv.dtype)
        rstd = torch.empty(n * (hq + hk), device=qkv.device, dtype=torch.float32) \
            if w_q is not None else None
        call("qknorm_rope_fwd", qkv, qkv.stride(0), w_q, w_k, cos, sin, pos, qk, qkw, rstd, n, hq, hk,
             hd, float(eps), stream_ptr())
        q, k, v = qk[:, : hq * hd], qk[:, hq * hd:], qkv[:, qkw:]
        out = torch.empty(n, hq * hd, device=qkv.device, dtype=qkv.dtype)
        lse = torch.empty(B, hq, T, device=qkv.device, dtype=torch.float32)
        call("flash_fwd", q, qkw, k, qkw, v, qkv.stride(0), out, out.stride(0), lse,
             B, T, T, hq, hk, hd, float(scale), 1, stream_ptr())
        ctx.save_for_backward(qkv, qk, out, lse, w_q, w_k, rstd, cos, sin, pos)
        ctx.wq_ref, ctx.wk_ref = w_q, w_k
        ctx.dims = (B, T, hq, hk, hd, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        from .functional import _notify
        qkv, qk, out, lse, w_q, w_k, rstd, cos, sin, pos = ctx.saved_tensors
        B, T, hq, hk, hd, scale = ctx.dims
        n = qkv.shape[0]
        qkw = (hq + hk) * hd
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dqk = torch.empty(n, qkw, device=qkv.device, dtype=qkv.dtype)
        delta = torch.empty(B, hq, T, device=qkv.device, dtype=torch.float32)
        call("flash_bwd", qk[:, : hq * hd], qkw, qk[:, hq * hd:], qkw, qkv[:, qkw:], qkv.stride(0),
             out, out.stride(0), dout, dout.stride(0), lse, delta, dqk[:, : hq * hd], qkw,
             dqk[:, hq * hd:], qkw, dqkv[:, qkw:], dqkv.stride(0), B, T, T, hq, hk, hd, float(scale), 1,
             stream_ptr())
        dwq = dwk = tq = tk = None
        if w_q is not None:
            mgq = getattr(ctx.wq_ref, "main_grad", None)
            mgk = getattr(ctx.wk_ref, "main_grad", None)
            tq = mgq if mgq is not None else torch.zeros(hd, device=qkv.device, dtype=torch.float32)
            tk = mgk if mgk is not None else torch.zeros(hd, device=qkv.device, dtype=torch.float32)
        call("qknorm_rope_bwd", dqk, qkw, qkv, qkv.stride(0), w_q, w_k, rstd, cos, sin, pos, dqkv,
             dqkv.stride(0), tq, tk, n, hq, hk, hd, stream_ptr())
        if w_q is not None:
            if getattr(ctx.wq_ref, "main_grad", None) is None:
                dwq = tq.to(w_q.dtype)
            else:
                _notify(ctx.wq_ref)
            if getattr(ctx.wk_ref, "main_grad", None) is None:
                dwk = tk.to(w_k.dtype)
            else:
                _notify(ctx.wk_ref)
        return (dqkv, dwq, dwk) + (None,) * 10


def attention_qkv(qkv, w_q, w_k, cos, sin, pos, B, T, hq, hk, hd, eps=1e-6, scale=None):
    """Causal self-attention from a fused projection ``qkv`` [B*T, (hq+2hk)*hd] with optional
    per-head RMSNorm gains and NeoX RoPE on q and k -> [B*T, hq*hd]."""
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    if not qkv.is_cuda:
        from . import functional as F
        qkw = (hq + hk) * hd
        qk = F.qknorm_rope(qkv, w_q, w_k, cos, sin, pos, hq, hk, hd, eps)
        return flash_attention(qk[:, : hq * hd], qk[:, hq * hd:], qkv[:, qkw:], B, T, hq, hk, hd, True, scale)
    return _AttnQKV.apply(qkv, w_q, w_k, cos, sin, pos, B, T, hq, hk, hd, eps, scale)


def flash_attention_into(out, q, k, v, B, T, hq, hk, hd, causal=True, scale=None, S=None, lse=None):
    """Inference form of :func:`flash_attention` on CUDA: no autograd node, rows may be strided views
    (last dimension contiguous) and the result is written into ``out`` [B*T, hq*hd]."""
    S = T if S is None else S
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    if lse is None:
        lse = torch.empty(B, hq, T, device=q.device, dtype=torch.float32)
    call("flash_fwd", q, q.stride(0), k, k.stride(0), v, v.stride(0), out, out.stride(0), lse,
         B, T, S, hq, hk, hd, float(scale), int(causal), stream_ptr())
    return out


def flash_attention(q, k, v, B, T, hq, hk, hd, causal=True, scale=None, S=None):
    """q: [B*T, hq*hd]; k, v: [B*S, hk*hd] (S defaults to T) -> [B*T, hq*hd]."""
    S = T if S is None else S
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    if not q.is_cuda:
        from . import cpu_native
        if cpu_native.enabled() and cpu_native.attention_supported(q, hd, S) and k.dtype == v.dtype == q.dtype:
            return cpu_native.attention(q, k, v, B, T, S, hq, hk, hd, causal, scale)
        o = ref.attention(q.reshape(B, T, hq, hd), k.reshape(B, S, hk, hd), v.reshape(B, S, hk, hd),
                          causal, scale)
        return o.reshape(B * T, hq * hd)
    return _FlashAttn.apply(q, k, v, B, T, S, hq, hk, hd, causal, scale)
