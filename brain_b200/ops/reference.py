"""Plain PyTorch restatement of every op (fp32/fp64 math, any device).

This is the CPU backend of the framework and the oracle every sm_100a kernel is tested against.
It restates the reference's kernel contracts (crates/kernels/wgsl/*.wgsl, crates/model/src/hostmath.rs)
with ordinary differentiable tensor ops, so autograd provides the backward and the finite-difference
gate (brain_b200/gradcheck.py) validates it.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

IGNORE_INDEX = -1  # the reference's 0xFFFF_FFFF sentinel read as int32


def linear(x, w, bias=None):
    return F.linear(x, w, bias)


def rmsnorm(x, w, eps=1e-6):
    xf = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.to(xf.dtype)
    return y.to(x.dtype)


def layernorm(x, g, b, eps=1e-5):
    xf = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
    y = F.layer_norm(xf, (x.shape[-1],), g.to(xf.dtype), b.to(xf.dtype), eps)
    return y.to(x.dtype)


def gelu_tanh(x):
    return F.gelu(x, approximate="tanh")


def swiglu(gu):
    """gu = [gate | up] along the last dim -> silu(gate) * up."""
    g, u = gu.chunk(2, dim=-1)
    return F.silu(g) * u


def rope_tables(max_pos: int, head_dim: int, theta: float, device=None, dtype=torch.float32):
    """cos/sin tables [max_pos, head_dim/2]; angle = pos * theta^(-2m/hd) (rope_base.wgsl)."""
    half = head_dim // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / head_dim)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().to(dtype).to(device), ang.sin().to(dtype).to(device)


def rope_neox(x, cos, sin, pos):
    """Half-split RoPE. x: [n, heads, hd]; pos: int64 [n]; pairs (m, m + hd/2)."""
    half = x.shape[-1] // 2
    c = cos[pos].to(x.dtype)[:, None, :]
    s = sin[pos].to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def rope_interleaved(x, cos, sin, pos):
    """Interleaved RoPE (pairs (2m, 2m+1)) used by the toy MoE model (rope_train.wgsl)."""
    c = cos[pos].to(x.dtype)[:, None, :]
    s = sin[pos].to(x.dtype)[:, None, :]
    a, b = x[..., 0::2], x[..., 1::2]
    out = torch.stack([a * c - b * s, b * c + a * s], dim=-1)
    return out.flatten(-2)


def qknorm_rope(qk, w_q, w_k, cos, sin, pos, hq, hk, hd, eps=1e-6):
    """qk: [n, (hq+hk)*hd] -> per-head RMSNorm (gains w_q / w_k, skipped when None) then NeoX RoPE."""
    n = qk.shape[0]
    x = qk.reshape(n, hq + hk, hd)
    if w_q is not None:
        q = rmsnorm(x[:, :hq], w_q, eps)
        k = rmsnorm(x[:, hq:], w_k, eps)
        x = torch.cat([q, k], dim=1)
    return rope_neox(x, cos, sin, pos).reshape(n, (hq + hk) * hd)


def attention(q, k, v, causal=True, scale=None):
    """q: [B, T, Hq, hd], k/v: [B, S, Hkv, hd] -> [B, T, Hq, hd]. Materialised-scores GQA attention
    (gqa_scores/attn_softmax/gqa_apply.wgsl)."""
    B, T, Hq, hd = q.shape
    S, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    dt = torch.float32 if q.dtype in (torch.bfloat16, torch.float16) else q.dtype
    qf = q.to(dt).permute(0, 2, 1, 3).reshape(B, Hkv, g, T, hd)
    kf = k.to(dt).permute(0, 2, 1, 3)[:, :, None]
    vf = v.to(dt).permute(0, 2, 1, 3)[:, :, None]
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(T, S, dtype=torch.bool, device=q.device).tril(S - T)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf).reshape(B, Hq, T, hd).permute(0, 2, 1, 3)
    return o.to(q.dtype)


def cross_entropy(logits, targets, reduction="mean"):
    """Masked CE: rows whose target is negative are ignored; mean over counted rows."""
    lf = logits.float() if logits.dtype in (torch.bfloat16, torch.float16) else logits
    valid = targets >= 0
    t = targets.clamp_min(0).long()
    lse = torch.logsumexp(lf, dim=-1)
    per = (lse - lf.gather(-1, t[..., None]).squeeze(-1)) * valid
    if reduction == "none":
        return per
    if reduction == "sum":
        return per.sum()
    return per.sum() / valid.sum().clamp_min(1)


def embedding(tok, emb):
    return emb[tok.long()]


def router_topk(logits, k, norm_topk_prob=True, scale=1.0):
    """Softmax over experts, greedy top-k with ties to the lowest index, optional renormalisation.
    Returns (probs, topk_idx, topk_w, lse). Mirrors router_gate_train.wgsl."""
    lf = logits.float() if logits.dtype in (torch.bfloat16, torch.float16) else logits
    lse = torch.logsumexp(lf, dim=-1)
    probs = torch.softmax(lf, dim=-1)
    # torch.topk does not promise tie order: select greedily so ties resolve to the lowest index.
    work = probs.detach().clone()
    idxs = []
    for _ in range(k):
        mx = work.max(dim=-1, keepdim=True).values
        first = (work == mx).to(torch.int64).argmax(dim=-1)
        idxs.append(first)
        work.scatter_(-1, first[:, None], -2.0)
    idx = torch.stack(idxs, dim=-1)
    w = probs.gather(-1, idx)
    if norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    return probs, idx, w * scale, lse


def quant_rows(x):
    """Per-row symmetric int8: scale = max|x|/127 (>=1e-8); q = clamp(rint(x/scale), -127, 127)."""
    xf = x.float()
    s = (xf.abs().amax(dim=-1) / 127.0).clamp_min(1e-8)
    q = torch.clamp(torch.round(xf / s[:, None]), -127, 127).to(torch.int8)
    return q, s


def adamw_(p, m, v, g, lr, beta1, beta2, eps, wd, step, coef=1.0):
    """In-place AdamW on flat fp32 tensors; eps outside the sqrt, decoupled decay (adamw.wgsl)."""
    g = g * coef
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    mh = m / (1 - beta1 ** step)
    vh = v / (1 - beta2 ** step)
    p.sub_(lr * (mh / (vh.sqrt() + eps) + wd * p))
    return p
