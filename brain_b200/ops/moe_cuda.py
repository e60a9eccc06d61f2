"""Row-compacted MoE layer on the sm_100a kernels (see ``ops.moe`` for the math).

Forward:  router GEMM (fp32 logits) -> router kernel (probs, top-k, counts) -> plan/positions
(expert-sorted rows padded to 128) -> gather -> grouped GEMM (gate|up) -> SwiGLU -> grouped GEMM
(down) -> weighted combine.  Backward mirrors it with the grouped dX GEMMs (weights read MN-major)
and the k-grouped dW GEMMs accumulating straight into the fp32 main-grad of the stacked expert
weights.  With an expert-parallel group, ``gather``/``combine`` read rows from every rank's
symmetric buffers (the all-to-all dispatch/combine is the kernels' own peer loads) and each rank
runs the grouped GEMMs of its local experts over the tokens of all ranks."""
from __future__ import annotations

import ctypes

import torch

from . import functional as F
from ._cuda import L, call, stream_ptr


def _u64(ptrs):
    return (ctypes.c_uint64 * len(ptrs))(*ptrs)


def grouped_gemm_rows(a, b_stacked, tile_group, b_group_rows, n_out, b_mn=False, out=None):
    """C[M, n_out] = A[M, K] . B_g^T per 128-row tile (g = tile_group[tile], -1 skipped).
    ``b_stacked``: [G*b_group_rows, K] (b_mn False) or [G*b_group_rows, n_out] (b_mn True)."""
    M, K = a.shape
    if out is None:
        out = torch.zeros(M, n_out, device=a.device, dtype=torch.bfloat16)
    call("gemm_bf16_grouped", a, b_stacked, out, M, n_out, K, a.stride(0), b_stacked.stride(0),
         out.stride(0), int(b_mn), 0, 1, tile_group, int(b_group_rows), int(b_stacked.shape[0]), None,
         0, L(0), 0, stream_ptr())
    return out


def grouped_gemm_dw(a, b, group_offsets, num_groups, out, accumulate=True):
    """out[g] (+)= A[rows_g, M]^T . B[rows_g, N]; out: fp32 [G, M, N]."""
    rows, M = a.shape
    N = b.shape[1]
    assert out.dtype == torch.float32 and out.shape[-2:] == (M, N)
    call("gemm_bf16_grouped", a, b, out, M, N, rows, a.stride(0), b.stride(0), N, 1,
         2 if accumulate else 1, 2, None, 0, 0, group_offsets, int(num_groups), L(M * N), 0,
         stream_ptr())
    return out


class _LinearF32(torch.autograd.Function):
    """y = x W^T with fp32 output (router logits)."""

    @staticmethod
    def forward(ctx, x, w):
        y = F.gemm(x, w, out_dtype=torch.float32)
        ctx.save_for_backward(x, w)
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        E = w.shape[0]
        d16 = dy.to(torch.bfloat16)
        wp = ctx.w_ref
        mg = getattr(wp, "main_grad", None)
        if E % 8:  # TMA rows must be 16-byte multiples: pad the expert axis with zeros
            E8 = (E + 7) // 8 * 8
            d16 = torch.nn.functional.pad(d16, (0, E8 - E))
            wpad = torch.nn.functional.pad(w, (0, 0, 0, E8 - E))
            dx = F.gemm(d16.contiguous(), wpad, b_mn=True)
            dw = F.gemm(d16, x, a_mn=True, b_mn=True, out_dtype=torch.float32)[:E]
            if mg is not None:
                mg.add_(dw)
                F._notify(wp)
                return dx, None
            return dx, dw.to(w.dtype)
        d16 = d16.contiguous()
        dx = F.gemm(d16, w, b_mn=True)
        if mg is not None:
            F.gemm(d16, x, a_mn=True, b_mn=True, out=mg, accumulate=True)
            F._notify(wp)
            return dx, None
        return dx, F.gemm(d16, x, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)


class _Router(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, norm, scale):
        n, E = logits.shape
        lg = logits.contiguous()
        probs = torch.empty_like(lg)
        lse = torch.empty(n, device=lg.device, dtype=torch.float32)
        idx = torch.empty(n, k, device=lg.device, dtype=torch.int32)
        w = torch.empty(n, k, device=lg.device, dtype=torch.float32)
        counts = torch.zeros(E, device=lg.device, dtype=torch.int32)
        call("router_topk", lg, probs, lse, idx, w, counts, n, E, k, int(norm), float(scale),
             stream_ptr())
        ctx.save_for_backward(probs, idx, lse)
        ctx.cfg = (norm, scale)
        ctx.mark_non_differentiable(idx, counts)
        return probs, idx, w, lse, counts

    @staticmethod
    def backward(ctx, d_probs, _d_idx, d_w, d_lse, _d_counts):
        probs, idx, lse = ctx.saved_tensors
        norm, scale = ctx.cfg
        li = idx.long()
        dp = torch.zeros_like(probs) if d_probs is None else d_probs.clone()
        if d_w is not None:
            ps = probs.gather(-1, li)
            if norm:
                Z = ps.sum(-1, keepdim=True)
                dsel = scale * (d_w / Z - (d_w * ps).sum(-1, keepdim=True) / (Z * Z))
            else:
                dsel = scale * d_w
            dp.scatter_add_(-1, li, dsel)
        dl = probs * (dp - (probs * dp).sum(-1, keepdim=True))
        if d_lse is not None:
            dl = dl + d_lse[:, None] * probs
        return dl, None, None, None


class _Experts(torch.autograd.Function):
    """y = sum_s w[t,s] * Expert_{idx[t,s]}(x[t]) over the local experts (single rank)."""

    @staticmethod
    def forward(ctx, x, w, w_gate_up, w_down, idx, counts):
        n, d = x.shape
        k = idx.shape[1]
        E, ff2, _ = w_gate_up.shape
        ff = ff2 // 2
        dev = x.device
        max_rows = (n * k + E * 127 + 127) // 128 * 128
        max_tiles = max_rows // 128
        offsets = torch.empty(E + 1, device=dev, dtype=torch.int32)
        tile_group = torch.empty(max_tiles, device=dev, dtype=torch.int32)
        call("moe_plan", counts, E, offsets, tile_group, max_tiles, stream_ptr())
        pos_of_pair = torch.full((n * k,), -1, device=dev, dtype=torch.int32)
        pair_of_pos = torch.full((max_rows,), -1, device=dev, dtype=torch.int32)
        call("moe_positions", idx, L(n * k), 0, E, offsets, pos_of_pair, pair_of_pos, stream_ptr())
        xc = x.contiguous()
        xp = torch.empty(max_rows, d, device=dev, dtype=x.dtype)
        call("moe_gather", _u64([xc.data_ptr()]), 1, n, pair_of_pos, None, k, xp, offsets, E, d,
             max_rows, stream_ptr())
        gu = grouped_gemm_rows(xp, w_gate_up.view(E * ff2, d), tile_group, ff2, ff2)
        h = torch.empty(max_rows, ff, device=dev, dtype=x.dtype)
        call("swiglu_fwd", gu, h, L(max_rows), ff, stream_ptr())
        yp = grouped_gemm_rows(h, w_down.view(E * d, ff), tile_group, d, d)
        y = torch.empty(n, d, device=dev, dtype=x.dtype)
        wc = w.contiguous()
        call("moe_combine", _u64([yp.data_ptr()]), _u64([pos_of_pair.data_ptr()]), 1, idx, L(0), wc,
             k, E, y, n, d, stream_ptr())
        ctx.save_for_backward(xp, gu, h, yp, wc, idx, offsets, tile_group, pos_of_pair, pair_of_pos)
        ctx.w_refs = (w_gate_up, w_down)
        ctx.dims = (n, d, k, E, ff, max_rows)
        return y

    @staticmethod
    def backward(ctx, dy):
        xp, gu, h, yp, wc, idx, offsets, tile_group, pos_of_pair, pair_of_pos = ctx.saved_tensors
        w_gate_up, w_down = ctx.w_refs
        n, d, k, E, ff, max_rows = ctx.dims
        dev = dy.device
        dy = dy.contiguous()
        s = stream_ptr()
        d_w = torch.empty(n, k, device=dev, dtype=torch.float32)
        call("moe_rowdot", dy, _u64([yp.data_ptr()]), _u64([pos_of_pair.data_ptr()]), 1, idx, L(0),
             k, E, d_w, L(n * k), d, s)
        dyp = torch.empty(max_rows, d, device=dev, dtype=dy.dtype)
        call("moe_gather", _u64([dy.data_ptr()]), 1, n, pair_of_pos, wc, k, dyp, offsets, E, d,
             max_rows, s)
        dh = grouped_gemm_rows(dyp, w_down.view(E * d, ff), tile_group, d, ff, b_mn=True)
        dgu = torch.empty_like(gu)
        call("swiglu_bwd", dh, gu, dgu, L(max_rows), ff, s)
        dxp = grouped_gemm_rows(dgu, w_gate_up.view(E * 2 * ff, d), tile_group, 2 * ff, d, b_mn=True)
        dx = torch.empty(n, d, device=dev, dtype=dy.dtype)
        call("moe_combine", _u64([dxp.data_ptr()]), _u64([pos_of_pair.data_ptr()]), 1, idx, L(0),
             None, k, E, dx, n, d, s)
        grads = []
        for wp, a_rows, b_rows in ((w_down, dyp, h), (w_gate_up, dgu, xp)):
            mg = getattr(wp, "main_grad", None)
            if mg is not None:
                grouped_gemm_dw(a_rows, b_rows, offsets, E, mg, accumulate=True)
                F._notify(wp)
                grads.append(None)
            else:
                g = torch.zeros(wp.shape, device=dev, dtype=torch.float32)
                grouped_gemm_dw(a_rows, b_rows, offsets, E, g, accumulate=True)
                grads.append(g.to(wp.dtype))
        return dx, d_w, grads[1], grads[0], None, None


def moe_forward_cuda(x, router, w_gate_up, w_down, top_k, norm_topk_prob, routed_scaling, aux_coef,
                     z_coef, ep=None):
    n, d = x.shape
    E = router.shape[0]
    logits = _LinearF32.apply(x, router)
    probs, idx, w, lse, counts = _Router.apply(logits, top_k, bool(norm_topk_prob),
                                               float(routed_scaling))
    fe = counts.to(torch.float32) / float(n * top_k)
    aux = aux_coef * E * (fe * probs.mean(dim=0)).sum()
    if z_coef:
        aux = aux + z_coef * (lse ** 2).mean()
    if ep is not None and ep.world > 1:
        y = ep.experts(x, w, w_gate_up, w_down, idx, counts)
    else:
        y = _Experts.apply(x, w, w_gate_up, w_down, idx, counts)
    return y, aux, counts
