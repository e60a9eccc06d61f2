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


def flash_attention(q, k, v, B, T, hq, hk, hd, causal=True, scale=None, S=None):
    """q: [B*T, hq*hd]; k, v: [B*S, hk*hd] (S defaults to T) -> [B*T, hq*hd]."""
    S = T if S is None else S
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    if not q.is_cuda:
        o = ref.attention(q.reshape(B, T, hq, hd), k.reshape(B, S, hk, hd), v.reshape(B, S, hk, hd),
                          causal, scale)
        return o.reshape(B * T, hq * hd)
    return _FlashAttn.apply(q, k, v, B, T, S, hq, hk, hd, causal, scale)
