"""Differentiable ops of the framework.

CUDA tensors (bf16 activations/weights) run the hand-written sm_100a kernels through
``torch.autograd.Function`` wrappers; CPU tensors run the fp32 restatement in ``ops.reference``
(the CPU backend and oracle).  Weight gradients of the native path accumulate straight into
``param.main_grad`` (fp32, a view into the flat gradient bucket) when the parameter has one, the
way the GEMM's accumulate epilogue is meant to be used; otherwise they are returned to autograd.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch

from . import _cuda, reference as ref
from ..utils import tune as _tune
from ._cuda import L, call, stream_ptr

IGNORE_INDEX = ref.IGNORE_INDEX

#: called as fn(param) right after a native backward accumulated into ``param.main_grad``;
#: the ZeRO engine uses it to launch a bucket's fused reduce-scatter as soon as it is complete.
grad_ready_hook: Optional[Callable[[torch.Tensor], None]] = None


def _notify(p):
    if grad_ready_hook is not None:
        grad_ready_hook(p)


# --------------------------------------------------------------------------------------- GEMM
def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=torch.bfloat16, accumulate=False,
         bias=None, alpha=1.0, gelu=False, bn=0, max_ctas=0):
    """C[M,N] = alpha * A[M,K] @ B[N,K]^T (+bias) on tcgen05.

    ``a``: [M,K] (``a_mn=False``) or [K,M] (``a_mn=True``); ``b``: [N,K] or [K,N] likewise.
    Rows may be strided (last dim contiguous).  ``accumulate`` adds into fp32 ``out``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=out_dtype)
    assert out.stride(-1) == 1 and out.shape == (M, N)
    if accumulate:
        assert out.dtype == torch.float32
    mode = 3 if gelu else (0 if out.dtype == torch.bfloat16 else (2 if accumulate else 1))
    if M == 0 or N == 0:
        return out
    if bn == 0 and _tune._TUNER is not None and not accumulate and not torch.cuda.is_current_stream_capturing():
        # autotune (off by default): time the tile widths once per shape, then use the cached winner
        t = _tune._TUNER
        bn = t.pick(t.key("gemm_bf16", M, N, K, int(a_mn), int(b_mn), mode), _tune.GEMM_BN,
                    lambda c: call("gemm_bf16", a, b, out, bias, M, N, K, a.stride(0), b.stride(0), out.stride(0),
                                   int(a_mn), int(b_mn), mode, float(alpha), int(c), int(max_ctas), stream_ptr()))
    call("gemm_bf16", a, b, out, bias, M, N, K, a.stride(0), b.stride(0), out.stride(0),
         int(a_mn), int(b_mn), mode, float(alpha), int(bn), int(max_ctas), stream_ptr())
    return out


def gemm_i8(a_q, b_q, scale_m, scale_n, out=None, bn=0):
    """W8A8: bf16 C = (A_i8[M,K] @ B_i8[N,K]^T) * scale_m[:,None] * scale_n[None,:]."""
    M, K = a_q.shape
    N = b_q.shape[0]
    if out is None:
        out = torch.empty(M, N, device=a_q.device, dtype=torch.bfloat16)
    call("gemm_i8", a_q, b_q, out, scale_m, scale_n, M, N, K, a_q.stride(0), b_q.stride(0),
         out.stride(0), int(bn), 0, stream_ptr())
    return out


def unpack_q4(words, out=None):
    """int8 [n, 8*kw] operand of :func:`gemm_i8` from 4-bit storage ``words`` int32 [n, kw] (eight
    two's-complement nibbles per word, element b of a group in bits 4b..4b+3)."""
    n, kw = words.shape
    if not words.is_cuda:
        sh = (4 * torch.arange(8, dtype=torch.int64))[None, None, :]
        nib = ((words.to(torch.int64) & 0xFFFFFFFF)[:, :, None] >> sh) & 0xF
        return torch.where(nib >= 8, nib - 16, nib).reshape(n, kw * 8).to(torch.int8)
    if out is None:
        out = torch.empty(n, kw * 8, device=words.device, dtype=torch.int8)
    call("unpack_q4", words.contiguous(), out, L(n * kw), stream_ptr())
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        bias32 = bias.float() if bias is not None else None
        y = gemm(x2, w, bias=bias32)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.bias_ref = bias
        ctx.w_ref = w
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view(ctx.xshape)  # dy[M,N] . W[N,K]
        if ctx.needs_input_grad[1]:
            wp = ctx.w_ref
            mg = getattr(wp, "main_grad", None)
            if mg is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)  # dy^T . x
                _notify(wp)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            bp = ctx.bias_ref
            mg = getattr(bp, "main_grad", None)
            tgt = mg if mg is not None else torch.zeros(dy2.shape[1], device=dy.device,
                                                        dtype=torch.float32)
            call("colsum", dy2, None, None, None, tgt, dy2.shape[0], dy2.shape[1], dy2.stride(0), 0,
                 stream_ptr())
            if mg is None:
                db = tgt.to(bp.dtype)
            else:
                _notify(bp)
        return dx, dw, db


def linear(x, w, bias=None):
    if not x.is_cuda:
        if x.dtype == torch.float32 and w.dtype == torch.float32:
            from . import cpu_native
            if cpu_native.enabled():      # BRAIN_CPU_NATIVE=1: the AVX2 GEMM of csrc/cpu instead of PyTorch's
                return cpu_native.linear(x, w, bias)
        return ref.linear(x, w, bias)
    return _Linear.apply(x, w, bias)


# --------------------------------------------------------------------------------------- norms
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual):
        shape = x.shape
        d = shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        h = None
        if residual is not None:
            r2 = residual.reshape(-1, d).contiguous()
            h = torch.empty_like(x2)
            call("rmsnorm_fwd", x2, r2, w, y, h, rstd, rows, d, float(eps), stream_ptr())
            ctx.save_for_backward(h, w, rstd)
        else:
            call("rmsnorm_fwd", x2, None, w, y, None, rstd, rows, d, float(eps), stream_ptr())
            ctx.save_for_backward(x2, w, rstd)
        ctx.w_ref = w
        ctx.has_res = residual is not None
        ctx.shape = shape
        if h is not None:
            return y.view(shape), h.view(shape)
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        xin, w, rstd = ctx.saved_tensors
        d = xin.shape[1]
        rows = xin.shape[0]
        dy2 = dy.reshape(-1, d).contiguous()
        dres = dh.reshape(-1, d).contiguous() if (ctx.has_res and dh is not None) else None
        dx = torch.empty_like(xin)
        call("rmsnorm_bwd_dx", dy2, xin, w, rstd, dres, dx, rows, d, stream_ptr())
        wp = ctx.w_ref
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(wp, "main_grad", None)
            tgt = mg if mg is not None else torch.zeros(d, device=dy.device, dtype=torch.float32)
            call("colsum", dy2, xin, None, rstd, tgt, rows, d, d, 1, stream_ptr())
            if mg is None:
                dw = tgt.to(w.dtype)
            else:
                _notify(wp)
        dxv = dx.view(ctx.shape)
        return dxv, dw, None, (dxv if ctx.has_res else None)


def rmsnorm(x, w, eps=1e-6, residual=None):
    """y = w * h * rsqrt(mean(h^2)+eps) with h = x (+ residual). With ``residual`` returns (y, h)."""
    if not x.is_cuda:
        if residual is not None:
            h = x + residual
            return ref.rmsnorm(h, w, eps), h
        return ref.rmsnorm(x, w, eps)
    return _RMSNorm.apply(x, w, eps, residual)


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, b, eps):
        shape = x.shape
        d = shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, device=x.device, dtype=torch.float32)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        call("layernorm_fwd", x2, g, b, y, mean, rstd, rows, d, float(eps), stream_ptr())
        ctx.save_for_backward(x2, g, mean, rstd)
        ctx.g_ref, ctx.b_ref = g, b
        ctx.shape = shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, g, mean, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(-1, d).contiguous()
        dx = torch.empty_like(x2)
        call("layernorm_bwd_dx", dy2, x2, g, mean, rstd, None, dx, rows, d, stream_ptr())
        outs = []
        for p, mode in ((ctx.g_ref, 2), (ctx.b_ref, 0)):
            mg = getattr(p, "main_grad", None)
            tgt = mg if mg is not None else torch.zeros(d, device=dy.device, dtype=torch.float32)
            call("colsum", dy2, x2, mean, rstd, tgt, rows, d, d, mode, stream_ptr())
            if mg is None:
                outs.append(tgt.to(p.dtype))
            else:
                _notify(p)
                outs.append(None)
        return dx.view(ctx.shape), outs[0], outs[1], None


def layernorm(x, g, b, eps=1e-5):
    if not x.is_cuda:
        return ref.layernorm(x, g, b, eps)
    return _LayerNorm.apply(x, g, b, eps)


# --------------------------------------------------------------------------------------- rope
class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, w_q, w_k, cos, sin, pos, hq, hk, hd, eps):
        n = qkv.shape[0]
        out = torch.empty(n, (hq + hk) * hd, device=qkv.device, dtype=qkv.dtype)
        rstd = torch.empty(n * (hq + hk), device=qkv.device, dtype=torch.float32) \
            if w_q is not None else None
        call("qknorm_rope_fwd", qkv, qkv.stride(0), w_q, w_k, cos, sin, pos, out, out.stride(0),
             rstd, n, hq, hk, hd, float(eps), stream_ptr())
        ctx.save_for_backward(qkv, w_q, w_k, rstd, cos, sin, pos)
        ctx.wq_ref, ctx.wk_ref = w_q, w_k
        ctx.dims = (hq, hk, hd)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, w_q, w_k, rstd, cos, sin, pos = ctx.saved_tensors
        hq, hk, hd = ctx.dims
        n = qkv.shape[0]
        dout = dout.contiguous()
        # gradient wrt the whole qkv buffer: q|k part from this op, v part is zero here (the
        # attention op returns dv separately and the caller concatenates through autograd)
        dx = torch.zeros_like(qkv) if qkv.shape[1] != (hq + hk) * hd else torch.empty_like(qkv)
        dwq = dwk = None
        tq = tk = None
        if w_q is not None:
            mgq = getattr(ctx.wq_ref, "main_grad", None)
            mgk = getattr(ctx.wk_ref, "main_grad", None)
            tq = mgq if mgq is not None else torch.zeros(hd, device=qkv.device, dtype=torch.float32)
            tk = mgk if mgk is not None else torch.zeros(hd, device=qkv.device, dtype=torch.float32)
        call("qknorm_rope_bwd", dout, dout.stride(0), qkv, qkv.stride(0), w_q, w_k, rstd, cos, sin,
             pos, dx, dx.stride(0), tq, tk, n, hq, hk, hd, stream_ptr())
        if w_q is not None:
            if getattr(ctx.wq_ref, "main_grad", None) is None:
                dwq = tq.to(w_q.dtype)
            else:
                _notify(ctx.wq_ref)
            if getattr(ctx.wk_ref, "main_grad", None) is None:
                dwk = tk.to(w_k.dtype)
            else:
                _notify(ctx.wk_ref)
        return dx, dwq, dwk, None, None, None, None, None, None, None


def qknorm_rope(qkv, w_q, w_k, cos, sin, pos, hq, hk, hd, eps=1e-6):
    """Per-head RMSNorm (skipped when gains are None) + NeoX RoPE on the first (hq+hk) heads of
    ``qkv`` [n, >= (hq+hk)*hd]; returns [n, (hq+hk)*hd].  ``pos`` int32 [n]."""
    if not qkv.is_cuda:
        return ref.qknorm_rope(qkv[:, : (hq + hk) * hd], w_q, w_k, cos, sin, pos.long(), hq, hk, hd,
                               eps)
    return _QKNormRope.apply(qkv, w_q, w_k, cos, sin, pos, hq, hk, hd, eps)


# --------------------------------------------------------------------------------------- mlp acts
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        shape = gu.shape
        ff = shape[-1] // 2
        gu2 = gu.reshape(-1, 2 * ff).contiguous()
        h = torch.empty(gu2.shape[0], ff, device=gu.device, dtype=gu.dtype)
        call("swiglu_fwd", gu2, h, L(gu2.shape[0]), ff, stream_ptr())
        ctx.save_for_backward(gu2)
        ctx.shape = shape
        return h.view(*shape[:-1], ff)

    @staticmethod
    def backward(ctx, dh):
        (gu2,) = ctx.saved_tensors
        ff = gu2.shape[1] // 2
        dh2 = dh.reshape(-1, ff).contiguous()
        dgu = torch.empty_like(gu2)
        call("swiglu_bwd", dh2, gu2, dgu, L(gu2.shape[0]), ff, stream_ptr())
        return dgu.view(ctx.shape)


def swiglu(gu):
    if not gu.is_cuda:
        return ref.swiglu(gu)
    return _SwiGLU.apply(gu)


class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        call("gelu_fwd", xc, y, L(xc.numel()), stream_ptr())
        ctx.save_for_backward(xc)
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        call("gelu_bwd", dyc, xc, dx, L(xc.numel()), stream_ptr())
        return dx


def gelu(x):
    if not x.is_cuda:
        return ref.gelu_tanh(x)
    return _Gelu.apply(x)


# --------------------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tok, emb, pos_emb, T):
        tok32 = tok.reshape(-1).to(torch.int32)
        n = tok32.numel()
        d = emb.shape[1]
        out = torch.empty(n, d, device=emb.device, dtype=emb.dtype)
        call("embed_fwd", tok32, emb, pos_emb, int(T), out, L(n), d, emb.shape[0], stream_ptr())
        ctx.save_for_backward(tok32)
        ctx.emb_ref, ctx.pos_ref, ctx.T = emb, pos_emb, int(T)
        ctx.oshape = (*tok.shape, d)
        return out.view(ctx.oshape)

    @staticmethod
    def backward(ctx, dout):
        (tok32,) = ctx.saved_tensors
        emb, pos = ctx.emb_ref, ctx.pos_ref
        d = emb.shape[1]
        d2 = dout.reshape(-1, d).contiguous()
        mg = getattr(emb, "main_grad", None)
        te = mg if mg is not None else torch.zeros(emb.shape, device=emb.device, dtype=torch.float32)
        tp = None
        if pos is not None:
            mgp = getattr(pos, "main_grad", None)
            tp = mgp if mgp is not None else torch.zeros(pos.shape, device=emb.device,
                                                         dtype=torch.float32)
        call("embed_bwd", tok32, d2, te, tp, ctx.T, L(tok32.numel()), d, emb.shape[0], stream_ptr())
        de = dp = None
        if mg is None:
            de = te.to(emb.dtype)
        else:
            _notify(emb)
        if pos is not None:
            if getattr(pos, "main_grad", None) is None:
                dp = tp.to(pos.dtype)
            else:
                _notify(pos)
        return None, de, dp, None


def embedding(tok, emb, pos_emb=None, T=1):
    """emb[tok] (+ pos_emb[t % T] for learned absolute positions)."""
    if not emb.is_cuda:
        x = ref.embedding(tok, emb)
        if pos_emb is not None:
            n = tok.numel()
            idx = torch.arange(n, device=tok.device) % T
            x = x + pos_emb[idx].view(*tok.shape, -1)
        return x
    return _Embedding.apply(tok, emb, pos_emb, T)


# --------------------------------------------------------------------------------------- losses
class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        V = logits.shape[-1]
        lg = logits.reshape(-1, V)
        if not lg.is_contiguous():
            lg = lg.contiguous()
        n = lg.shape[0]
        t32 = targets.reshape(-1).to(torch.int32)
        loss = torch.empty(n, device=lg.device, dtype=torch.float32)
        lse = torch.empty(n, device=lg.device, dtype=torch.float32)
        call("cross_entropy", lg, L(lg.stride(0)), t32, loss, lse, n, V, 0, None, 1.0, stream_ptr())
        count = (t32 >= 0).sum().clamp_min(1).to(torch.float32)
        ctx.save_for_backward(lg, t32, lse, count)
        return loss.sum() / count

    @staticmethod
    def backward(ctx, dl):
        lg, t32, lse, count = ctx.saved_tensors
        # recompute softmax from saved lse in place of the logits copy
        n, V = lg.shape
        g = lg.clone()
        scale = (dl.float() / count).reshape(1)
        loss = torch.empty(n, device=lg.device, dtype=torch.float32)
        call("cross_entropy", g, L(g.stride(0)), t32, loss, None, n, V, 1, scale, 1.0, stream_ptr())
        return g, None


def cross_entropy(logits, targets):
    """Mean masked CE (targets < 0 ignored)."""
    if not logits.is_cuda:
        return ref.cross_entropy(logits, targets)
    return _CrossEntropy.apply(logits, targets)


class _LMHeadCE(torch.autograd.Function):
    """Fused LM head + masked CE in row chunks: logits never outlive a chunk, and the head's dX and
    dW are produced in the forward pass (the loss is the end of the graph).  ``scale`` is the factor
    the summed token losses are multiplied by (1/number of counted targets in the optimiser step);
    the upstream gradient multiplies dX in backward and must be 1 for the accumulated dW to be
    exact, which holds when the loss is what ``backward()`` is called on."""

    @staticmethod
    def forward(ctx, x, w, targets, scale, chunk_rows, weights=None):
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        n = x2.shape[0]
        V = w.shape[0]
        t32 = targets.reshape(-1).to(torch.int32)
        wts = weights.reshape(-1).float() if weights is not None else None
        loss_rows = torch.empty(n, device=x.device, dtype=torch.float32)
        need_grad = x.requires_grad or w.requires_grad
        dx = torch.empty_like(x2) if need_grad else None
        mg = getattr(w, "main_grad", None)
        dw_acc = None
        if need_grad and w.requires_grad:
            dw_acc = mg if mg is not None else torch.zeros(w.shape, device=w.device,
                                                           dtype=torch.float32)
        chunk = min(n, chunk_rows)
        logits = torch.empty(chunk, V, device=x.device, dtype=torch.bfloat16)
        for r0 in range(0, n, chunk):
            r1 = min(n, r0 + chunk)
            m = r1 - r0
            lg = logits[:m]
            gemm(x2[r0:r1], w, out=lg)
            call("cross_entropy", lg, L(lg.stride(0)), t32[r0:r1], loss_rows[r0:r1], None, m, V,
                 1 if need_grad else 0, None, float(scale), stream_ptr())
            if wts is not None and need_grad:
                # per-position weights: d(sum_i w_i CE_i)/d(logits) is the row gradient times w_i
                lg.mul_(wts[r0:r1, None].to(lg.dtype))
            if need_grad:
                gemm(lg, w, b_mn=True, out=dx[r0:r1])
                if dw_acc is not None:
                    gemm(lg, x2[r0:r1], a_mn=True, b_mn=True, out=dw_acc, accumulate=True)
        ctx.save_for_backward(dx)
        ctx.xshape = x.shape
        ctx.w_ref = w
        ctx.dw = None if (mg is not None or dw_acc is None) else dw_acc
        ctx.used_main = mg is not None and dw_acc is not None
        if wts is not None:
            return (loss_rows * wts).sum() * scale
        return loss_rows.sum() * scale

    @staticmethod
    def backward(ctx, dl):
        (dx,) = ctx.saved_tensors
        gx = (dx * dl.to(dx.dtype)).view(ctx.xshape) if dx is not None else None
        gw = None
        if ctx.dw is not None:
            gw = (ctx.dw * dl.float()).to(ctx.w_ref.dtype)
        if ctx.used_main:
            _notify(ctx.w_ref)
        return gx, gw, None, None, None, None


def lm_head_ce(x, w, targets, scale=None, chunk_rows=8192, weights=None):
    """sum over counted tokens of CE(x @ w^T, target) * scale  (scale defaults to 1/count).
    ``weights`` (one per position) turns it into sum_i w_i CE_i * scale — the reward / advantage
    weighted loss of crates/qwen3/src/model.rs:1320-1334."""
    if scale is None:
        scale = 1.0 / max(int((targets >= 0).sum().item()), 1)
    if not x.is_cuda:
        logits = ref.linear(x, w)
        if weights is not None:
            rows = ref.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), reduction="none")
            return (rows * weights.reshape(-1).to(rows.dtype)).sum() * scale
        return ref.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1),
                                 reduction="sum") * scale
    return _LMHeadCE.apply(x, w, targets, float(scale), int(chunk_rows), weights)


# --------------------------------------------------------------------------------------- misc
def quant_rows(x):
    """Per-row symmetric int8 quantisation -> (int8 [rows,k], fp32 scale [rows])."""
    if not x.is_cuda:
        return ref.quant_rows(x)
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    q = torch.empty(x2.shape, device=x.device, dtype=torch.int8)
    s = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
    dt = 0 if x2.dtype == torch.bfloat16 else 1
    if dt == 1:
        x2 = x2.float()
    call("quant_rows", x2, q, s, x2.shape[0], x2.shape[1], dt, stream_ptr())
    return q, s


def argmax_rows(logits):
    """Greedy head: int32 argmax per row of bf16 logits (lowest index on ties)."""
    if not logits.is_cuda:
        return logits.float().argmax(dim=-1).to(torch.int32)
    lg = logits.reshape(-1, logits.shape[-1])
    out = torch.empty(lg.shape[0], device=lg.device, dtype=torch.int32)
    call("argmax_rows", lg, L(lg.stride(0)), lg.shape[0], lg.shape[1], out, stream_ptr())
    return out


def topk_rows(logits, k: int):
    """The k largest logits of every row, descending (lowest index first among equals):
    (int32 indices [rows, k], fp32 values [rows, k])."""
    lg = logits.reshape(-1, logits.shape[-1])
    if not lg.is_cuda or lg.dtype != torch.bfloat16:
        vals, idx = torch.topk(lg.float(), k, dim=-1)
        return idx.to(torch.int32), vals
    idx = torch.empty(lg.shape[0], k, device=lg.device, dtype=torch.int32)
    vals = torch.empty(lg.shape[0], k, device=lg.device, dtype=torch.float32)
    call("topk_rows", lg, L(lg.stride(0)), lg.shape[0], lg.shape[1], int(k), idx, vals, stream_ptr())
    return idx, vals


def router_topk(logits, k, norm_topk_prob=True, scale=1.0, counts=None):
    """(probs, topk_idx, topk_w, lse) — see ``reference.router_topk``; CUDA path is one warp per token."""
    if not logits.is_cuda:
        return ref.router_topk(logits, k, norm_topk_prob, scale)
    lg = logits.float().contiguous()
    n, E = lg.shape
    probs = torch.empty_like(lg)
    lse = torch.empty(n, device=lg.device, dtype=torch.float32)
    idx = torch.empty(n, k, device=lg.device, dtype=torch.int32)
    w = torch.empty(n, k, device=lg.device, dtype=torch.float32)
    call("router_topk", lg, probs, lse, idx, w, counts, n, E, k, int(norm_topk_prob), float(scale),
         stream_ptr())
    return probs, idx.long(), w, lse
