"""Kernel micro-benchmarks with roofline fractions against the measured peaks.

    python -m brain_b200.perf.kernel_bench gemm  [--m 16384 --n 4096 --k 1024 --layout tn|nn|tt --bn 0]
    python -m brain_b200.perf.kernel_bench flash [--b 4 --t 4096 --hq 16 --hk 8 --hd 128 --bwd]
    python -m brain_b200.perf.kernel_bench i8    [--m 256 --n 4096 --k 4096]
    python -m brain_b200.perf.kernel_bench copy  (HBM copy bandwidth probe)

Timing: CUDA events on the launching stream, warm-up first, inputs rotated through a pool larger
than the 126 MB L2 so every timed launch starts cold.  ``--iters 1 --warmup 0`` gives a run that is
small enough to put under ``ncu``.  The roofline denominators come from ``MEASURED_PEAKS.json``
(driver-measured cuBLAS bf16 throughput and copy bandwidth) when present, else the documented
fallback (1.59 PFLOP/s, 6.65 TB/s)."""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return p["bf16_tflops"] * 1e12, p["hbm_gbs"] * 1e9, "measured"
    except Exception:
        return 1.59e15, 6.65e12, "fallback"


def timeit(fns, iters, warmup):
    """``fns``: list of closures over distinct input sets (rotated so inputs exceed L2)."""
    for i in range(warmup):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(iters):
        fns[i % len(fns)]()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters * 1e-3


def elementwise_suite(a, dev, bw):
    """Bandwidth-bound kernels at the training shapes (rows = b*t): algorithmic bytes / device time
    as a fraction of the measured copy bandwidth.  Inputs total > 126 MB per call, so L2 does not
    hold them between iterations."""
    from brain_b200.ops import functional as F
    from brain_b200.ops import reference as ref
    from brain_b200.ops._cuda import L, call, stream_ptr
    rows, d, ff, hq, hk, hd = a.b * a.t, a.k, 3 * a.k, a.hq, a.hk, a.hd
    bf = torch.bfloat16
    res = {}

    def rec(name, fn, nbytes):
        t = timeit([fn], a.iters, a.warmup)
        res[name] = {"us": round(t * 1e6, 1), "gbs": round(nbytes / t / 1e9), "frac_of_copy": round(nbytes / t / bw, 3)}
    x = torch.randn(rows, d, device=dev, dtype=bf)
    r = torch.randn(rows, d, device=dev, dtype=bf)
    w = torch.ones(d, device=dev, dtype=bf)
    y, h, dx = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    rstd = torch.empty(rows, device=dev, dtype=torch.float32)
    rec("rmsnorm_fwd(+residual)", lambda: call("rmsnorm_fwd", x, r, w, y, h, rstd, rows, d, 1e-6, stream_ptr()), 4 * rows * d * 2)
    rec("rmsnorm_bwd_dx(+dres)", lambda: call("rmsnorm_bwd_dx", y, x, w, rstd, r, dx, rows, d, stream_ptr()), 4 * rows * d * 2)
    gu = torch.randn(rows, 2 * ff, device=dev, dtype=bf)
    hh = torch.empty(rows, ff, device=dev, dtype=bf)
    dgu = torch.empty_like(gu)
    rec("swiglu_fwd", lambda: call("swiglu_fwd", gu, hh, L(rows), ff, stream_ptr()), 3 * rows * ff * 2)
    rec("swiglu_bwd", lambda: call("swiglu_bwd", hh, gu, dgu, L(rows), ff, stream_ptr()), 5 * rows * ff * 2)
    width = (hq + 2 * hk) * hd
    qkw = (hq + hk) * hd
    qkv = torch.randn(rows, width, device=dev, dtype=bf)
    qk = torch.empty(rows, qkw, device=dev, dtype=bf)
    dqkv = torch.empty_like(qkv)
    rs2 = torch.empty(rows * (hq + hk), device=dev, dtype=torch.float32)
    gq = torch.ones(hd, device=dev, dtype=bf)
    cos, sin = ref.rope_tables(a.t, hd, 1e6, device=dev)
    pos = torch.arange(a.t, device=dev, dtype=torch.int32).repeat(a.b)
    tq, tk = torch.zeros(hd, device=dev), torch.zeros(hd, device=dev)
    rec("qknorm_rope_fwd", lambda: call("qknorm_rope_fwd", qkv, width, gq, gq, cos, sin, pos, qk, qkw, rs2, rows, hq, hk, hd,
                                        1e-6, stream_ptr()), 2 * rows * qkw * 2)
    rec("qknorm_rope_bwd", lambda: call("qknorm_rope_bwd", qk, qkw, qkv, width, gq, gq, rs2, cos, sin, pos, dqkv, width, tq, tk,
                                        rows, hq, hk, hd, stream_ptr()), 3 * rows * qkw * 2)
    n = rows * d * 8
    m_, v_, ms, g = (torch.zeros(n, device=dev) for _ in range(4))
    w16 = torch.zeros(n, device=dev, dtype=bf)
    coef = torch.ones(1, device=dev)
    rec("adamw", lambda: call("adamw", ms, m_, v_, g, w16, L(n), 1e-4, 0.9, 0.999, 1e-8, 0.1, 3, coef, stream_ptr()), n * 30)
    del m_, v_, ms, g, w16
    # router softmax + top-8 over 128 experts (fp32 logits in, probabilities + ids + weights out)
    E, kk = 128, 8
    ntok = rows * 8
    lg = torch.randn(ntok, E, device=dev)
    probs, lse = torch.empty_like(lg), torch.empty(ntok, device=dev)
    idx = torch.empty(ntok, kk, device=dev, dtype=torch.int32)
    tw = torch.empty(ntok, kk, device=dev)
    cnt = torch.zeros(E, device=dev, dtype=torch.int32)
    rec("router_topk(128 experts, top-8)", lambda: call("router_topk", lg, probs, lse, idx, tw, cnt, ntok, E, kk, 1, 1.0,
                                                        stream_ptr()), ntok * (2 * E * 4 + kk * 8 + 4))
    # masked cross-entropy over a vocabulary chunk: reads the bf16 logits, writes their gradient in place
    V, crows = 151936, 2048
    logits = torch.randn(crows, V, device=dev).bfloat16()
    tgt = torch.randint(0, V, (crows,), device=dev, dtype=torch.int32)
    lrows = torch.empty(crows, device=dev)
    rec("cross_entropy(+grad in place)", lambda: call("cross_entropy", logits, L(logits.stride(0)), tgt, lrows, None, crows, V,
                                                     1, None, 1.0 / crows, stream_ptr()), 2 * crows * V * 2)
    return res


def cpu_gemm_suite(threads: int):
    """The native fp32 GEMM of csrc/cpu against PyTorch's (oneDNN) on GPT-2 small's layer shapes, the
    three products of a linear layer each; GFLOP/s, best of 6 trials of 5 calls (no GPU needed)."""
    import time
    from brain_b200.ops import cpu_native
    torch.set_num_threads(threads)
    cpu_native.threads = threads

    def best(fn, n=5, trials=6):
        fn()
        fn()
        b = 1e9
        for _ in range(trials):
            t = time.perf_counter()
            for _ in range(n):
                fn()
            b = min(b, (time.perf_counter() - t) / n)
        return b

    rows = []
    for M, N, K in ((512, 768, 768), (512, 2304, 768), (512, 3072, 768), (512, 768, 3072), (512, 50257, 768)):
        x, w, g = torch.randn(M, K), torch.randn(N, K), torch.randn(M, N)
        fl = 2.0 * M * N * K
        row = {"m": M, "n": N, "k": K}
        for name, native, lib in (("fwd", lambda: cpu_native.gemm(x, w, tb=True), lambda: x @ w.t()),
                                  ("dx", lambda: cpu_native.gemm(g, w), lambda: g @ w),
                                  ("dw", lambda: cpu_native.gemm(g, x, ta=True), lambda: g.t() @ x)):
            row[name + "_native_gflops"] = round(fl / best(native) / 1e9)
            row[name + "_pytorch_gflops"] = round(fl / best(lib) / 1e9)
        rows.append(row)
    return {"what": "cpu-gemm", "threads": threads, "shapes": rows}


def cpu_attn_suite(threads: int):
    """Native CPU attention (csrc/cpu/attention.cpp) against the materialised-scores PyTorch path,
    causal, forward alone and forward + backward; milliseconds, best of 6 trials of 5 calls."""
    import math
    import time
    from brain_b200.ops import cpu_native, reference as ref
    torch.set_num_threads(threads)
    cpu_native.threads = threads

    def best(fn, n=5, trials=6):
        fn()
        b = 1e9
        for _ in range(trials):
            t = time.perf_counter()
            for _ in range(n):
                fn()
            b = min(b, (time.perf_counter() - t) / n)
        return round(b * 1e3, 2)

    rows = []
    for B, T, hq, hk, hd in ((4, 128, 12, 12, 64), (2, 1024, 12, 12, 64), (1, 2048, 16, 8, 128)):
        q = torch.randn(B * T, hq * hd, requires_grad=True)
        k = torch.randn(B * T, hk * hd, requires_grad=True)
        v = torch.randn(B * T, hk * hd, requires_grad=True)
        g = torch.randn(B * T, hq * hd)
        sc = 1 / math.sqrt(hd)

        def native(train):
            with torch.set_grad_enabled(train):
                o = cpu_native.attention(q, k, v, B, T, T, hq, hk, hd, True)
            if train:
                torch.autograd.grad(o, (q, k, v), g)

        def lib(train):
            with torch.set_grad_enabled(train):
                o = ref.attention(q.reshape(B, T, hq, hd), k.reshape(B, T, hk, hd), v.reshape(B, T, hk, hd), True,
                                  sc).reshape(B * T, hq * hd)
            if train:
                torch.autograd.grad(o, (q, k, v), g)

        rows.append({"batch": B, "seq": T, "heads": f"{hq}q/{hk}kv", "head_dim": hd,
                     "routed_to_native": cpu_native.attention_supported(q, hd, T),
                     "native_fwd_ms": best(lambda: native(False)), "native_fwd_bwd_ms": best(lambda: native(True)),
                     "pytorch_fwd_ms": best(lambda: lib(False)), "pytorch_fwd_bwd_ms": best(lambda: lib(True))})
    return {"what": "cpu-attn", "threads": threads, "shapes": rows}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "flash", "i8", "copy", "elementwise", "decode", "grouped", "cpu-gemm", "cpu-attn"])
    ap.add_argument("--threads", type=int, default=4, help="cpu-gemm: threads of both the native GEMM and PyTorch")
    ap.add_argument("--experts", type=int, default=16, help="grouped: experts (rows are split evenly)")
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--layout", default="tn", help="tn: x.W^T (fwd), nn: dy.W (dX), tt: dy^T.x (dW)")
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--b", type=int, default=4)
    ap.add_argument("--t", type=int, default=4096)
    ap.add_argument("--hq", type=int, default=16)
    ap.add_argument("--hk", type=int, default=8)
    ap.add_argument("--hd", type=int, default=128)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--seqlen", type=int, default=1200, help="decode: keys per sequence")
    ap.add_argument("--kv-int8", action="store_true", help="decode: int8 KV pools with per-row scales")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--library", action="store_true", help="also time the cuBLAS / SDPA baseline")
    a = ap.parse_args(argv)
    if a.what == "cpu-gemm":
        print(json.dumps(cpu_gemm_suite(a.threads)))
        return 0
    if a.what == "cpu-attn":
        print(json.dumps(cpu_attn_suite(a.threads)))
        return 0
    from brain_b200.ops import _cuda, functional as F
    from brain_b200.ops.attention import flash_attention

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    pf, bw, src = peaks()
    out = {"what": a.what, "peaks": src}
    if a.what == "copy":
        n = 1 << 30
        x = torch.empty(n, device=dev, dtype=torch.bfloat16)
        y = torch.empty_like(x)
        t = timeit([lambda: y.copy_(x)], a.iters, a.warmup)
        out.update(seconds=t, gbs=2 * n * 2 / t / 1e9, frac_of_peak=2 * n * 2 / t / bw)
    elif a.what == "elementwise":
        out["kernels"] = elementwise_suite(a, dev, bw)
    elif a.what in ("gemm", "i8"):
        M, N, K = a.m, a.n, a.k
        es = 1 if a.what == "i8" else 2
        pool = max(1, min(8, int(200e6 // ((M * K + N * K) * es + M * N * 2)) + 1))
        sets = []
        for _ in range(pool):
            if a.what == "i8":
                A = torch.randint(-127, 128, (M, K), device=dev, dtype=torch.int8)
                B = torch.randint(-127, 128, (N, K), device=dev, dtype=torch.int8)
                sa = torch.rand(M, device=dev) + 0.5
                sb = torch.rand(N, device=dev) + 0.5
                C = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
                sets.append((A, B, sa, sb, C))
            else:
                A = torch.randn(M, K, device=dev).bfloat16()
                B = torch.randn(N, K, device=dev).bfloat16()
                C = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
                if a.layout == "nn":      # dX = dy[M,K] . W[K,N]: B stored [K, N]
                    B = B.t().contiguous()
                elif a.layout == "tt":    # dW += dy^T . x: both stored [K, rows], fp32 accumulate
                    A, B = A.t().contiguous(), B.t().contiguous()
                    C = torch.zeros(M, N, device=dev, dtype=torch.float32)
                sets.append((A, B, C))
        if a.what == "i8":
            fns = [(lambda s=s: F.gemm_i8(s[0], s[1], s[2], s[3], out=s[4], bn=a.bn)) for s in sets]
        else:
            amn, bmn = a.layout == "tt", a.layout in ("nn", "tt")
            fns = [(lambda s=s: F.gemm(s[0], s[1], a_mn=amn, b_mn=bmn, out=s[2], bn=a.bn,
                                       accumulate=a.layout == "tt")) for s in sets]
        t = timeit(fns, a.iters, a.warmup)
        fl = 2.0 * M * N * K
        peak = pf * (2 if a.what == "i8" else 1)
        out.update(M=M, N=N, K=K, layout=a.layout, seconds=t, tflops=fl / t / 1e12,
                   frac_of_peak=fl / t / peak)
        if a.library and a.what == "gemm" and a.layout == "tn":
            A, B, C = sets[0]
            tl = timeit([lambda: torch.matmul(A, B.t(), out=C)], a.iters, a.warmup)
            out["library_tflops"] = fl / tl / 1e12
    elif a.what == "grouped":
        # row-grouped expert GEMM: expert-sorted rows, one launch for all experts (gate/up shape of an MoE layer)
        from brain_b200.ops.moe_cuda import grouped_gemm_rows
        G, M, N, K = a.experts, a.m, a.n, a.k
        assert M % (128 * G) == 0
        x = torch.randn(M, K, device=dev).bfloat16()
        w = torch.randn(G * N, K, device=dev).bfloat16()
        tile_group = torch.arange(M // 128, device=dev, dtype=torch.int32) // (M // 128 // G)
        out_ = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        t = timeit([lambda: grouped_gemm_rows(x, w, tile_group, N, N, out=out_)], a.iters, a.warmup)
        fl = 2.0 * M * N * K
        out.update(M=M, N=N, K=K, experts=G, seconds=t, tflops=fl / t / 1e12, frac_of_peak=fl / t / pf)
    elif a.what == "decode":
        # split-KV paged decode attention: every K and V row of every sequence is read once
        from brain_b200.ops._cuda import call, stream_ptr
        B_, hq, hk, hd, S, bs = a.b, a.hq, a.hk, a.hd, a.seqlen, 16
        per = -(-S // bs)
        nb = B_ * per
        es = 1 if a.kv_int8 else 2
        if a.kv_int8:
            kc = torch.randint(-127, 128, (nb, hk, bs, hd), device=dev, dtype=torch.int8)
            vc = torch.randint(-127, 128, (nb, hk, bs, hd), device=dev, dtype=torch.int8)
            ks = torch.rand(nb, hk, bs, device=dev) * 0.02
            vs = torch.rand(nb, hk, bs, device=dev) * 0.02
        else:
            kc = torch.randn(nb, hk, bs, hd, device=dev).bfloat16()
            vc = torch.randn(nb, hk, bs, hd, device=dev).bfloat16()
        bts = torch.randperm(nb, device=dev).to(torch.int32).reshape(B_, per)
        seqlens = torch.full((B_,), S, device=dev, dtype=torch.int32)
        q = torch.randn(B_, hq * hd, device=dev).bfloat16()
        o = torch.empty_like(q)
        splits = max(1, min(16, (4 * 148 + B_ * hk - 1) // (B_ * hk)))
        po = torch.empty(B_ * hq * splits * hd, device=dev)
        pm = torch.empty(B_ * hq * splits * 2, device=dev)

        def run():
            if a.kv_int8:
                call("paged_decode_i8", q, q.stride(0), kc, vc, ks, vs, bts, per, seqlens, o, o.stride(0), po, pm,
                     B_, hq, hk, hd, bs, splits, float(hd ** -0.5), stream_ptr())
            else:
                call("paged_decode", q, q.stride(0), kc, vc, bts, per, seqlens, o, o.stride(0), po, pm,
                     B_, hq, hk, hd, bs, splits, float(hd ** -0.5), stream_ptr())
        t = timeit([run], a.iters, a.warmup)
        nbytes = 2.0 * B_ * S * hk * hd * es + (8.0 * B_ * S * hk if a.kv_int8 else 0.0)
        out.update(B=B_, S=S, hq=hq, hk=hk, hd=hd, kv="int8" if a.kv_int8 else "bf16", splits=splits, seconds=t,
                   gbs=nbytes / t / 1e9, frac_of_peak=nbytes / t / bw)
    else:
        B_, T, hq, hk, hd = a.b, a.t, a.hq, a.hk, a.hd
        sets = []
        for _ in range(3):
            q = torch.randn(B_ * T, hq * hd, device=dev).bfloat16().requires_grad_(a.bwd)
            k = torch.randn(B_ * T, hk * hd, device=dev).bfloat16().requires_grad_(a.bwd)
            v = torch.randn(B_ * T, hk * hd, device=dev).bfloat16().requires_grad_(a.bwd)
            sets.append((q, k, v))
        fl = 4.0 * B_ * hq * T * T * hd / 2
        if not a.bwd:
            fns = [(lambda s=s: flash_attention(s[0], s[1], s[2], B_, T, hq, hk, hd, True)) for s in sets]
        else:
            outs = [flash_attention(s[0], s[1], s[2], B_, T, hq, hk, hd, True) for s in sets]
            do = torch.randn_like(outs[0])
            fns = [(lambda s=s, o=o: torch.autograd.grad(o, s, do, retain_graph=True))
                   for s, o in zip(sets, outs)]
            fl *= 2.5
        t = timeit(fns, a.iters, a.warmup)
        out.update(B=B_, T=T, hq=hq, hk=hk, hd=hd, bwd=a.bwd, seconds=t, tflops=fl / t / 1e12,
                   frac_of_peak=fl / t / pf)
    _cuda.check_error()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
