"""Mixture-of-experts layer math: softmax router with greedy top-k, SwiGLU experts applied only to
routed rows, weighted combine, and the load-balancing / z auxiliary losses

    aux = aux_coef * E * sum_e f_e * mean_n p[n,e]  +  z_coef * mean_n lse_n^2 ,
    f_e = (#tokens routed to e) / (n * top_k)           (a constant w.r.t. the gradient)

(reference: crates/model/src/moe.rs:57-286, crates/kernels/wgsl/{router_gate_train,expert_counts,
router_bwd,moe_linear_gated,scale_add}.wgsl).

CPU tensors run a differentiable PyTorch restatement (the oracle).  CUDA tensors run the
row-compacted path: warp-per-token router kernel, deterministic expert-sorted row positions padded
to 128 rows per expert, a row gather, grouped tcgen05 GEMMs over all experts in one launch each,
and a gather-based weighted combine; with an expert-parallel group the gather/combine pull rows
from peer GPUs over NVLink (``parallel.ep``)."""
from __future__ import annotations

import torch

from . import functional as F
from . import reference as ref


def _aux_losses(probs, idx, lse, E, k, aux_coef, z_coef):
    n = probs.shape[0]
    counts = torch.bincount(idx.reshape(-1), minlength=E).to(probs.dtype)
    fe = (counts / float(n * k)).detach()
    aux = aux_coef * E * (fe * probs.mean(dim=0)).sum()
    if z_coef:
        aux = aux + z_coef * (lse ** 2).mean()
    return aux, counts


def moe_forward_reference(x, router, w_gate_up, w_down, top_k, norm_topk_prob, routed_scaling,
                          aux_coef, z_coef):
    n, d = x.shape
    E = router.shape[0]
    logits = ref.linear(x, router)
    if logits.dtype in (torch.bfloat16, torch.float16):
        logits = logits.float()
    probs, idx, w, lse = ref.router_topk(logits, top_k, norm_topk_prob, routed_scaling)
    y = torch.zeros_like(x)
    for e in range(w_gate_up.shape[0]):
        sel = (idx == e)
        rows = sel.any(dim=-1).nonzero(as_tuple=True)[0]
        if rows.numel() == 0:
            continue
        h = ref.swiglu(ref.linear(x[rows], w_gate_up[e]))
        o = ref.linear(h, w_down[e])
        gate = (w * sel).sum(dim=-1)[rows].to(o.dtype)
        y = y.index_add(0, rows, o * gate[:, None])
    aux, counts = _aux_losses(probs, idx, lse, E, top_k, aux_coef, z_coef)
    return y, aux, counts


def moe_forward(x, router, w_gate_up, w_down, top_k, norm_topk_prob=True, routed_scaling=1.0,
                aux_coef=0.0, z_coef=0.0, ep=None):
    """x [n, d] -> (y [n, d], aux scalar, per-expert token counts)."""
    if not x.is_cuda:
        if ep is not None and ep.world > 1:
            return ep.forward_reference(x, router, w_gate_up, w_down, top_k, norm_topk_prob,
                                        routed_scaling, aux_coef, z_coef)
        return moe_forward_reference(x, router, w_gate_up, w_down, top_k, norm_topk_prob,
                                     routed_scaling, aux_coef, z_coef)
    from .moe_cuda import moe_forward_cuda
    return moe_forward_cuda(x, router, w_gate_up, w_down, top_k, norm_topk_prob, routed_scaling,
                            aux_coef, z_coef, ep)
