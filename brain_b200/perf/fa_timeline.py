"""clock64 timeline of the flash-attention backward kernels: CTA (0,0,0) of the dQ and of the dK/dV
kernel records, per block / iteration, when its MMA-issuing thread was released by the softmax
warps and when each softmax warpgroup got its scores, finished phase 1, got dP and finished phase 2.

    BB_TIMELINE=1 python -m brain_b200._build --force      # profiling build: stamps compiled in
    python -m brain_b200.perf.fa_timeline [--batch 4 --seq 4096 --hq 16 --hk 8 --hd 128]
    (or: brain perf tool fa-timeline ...)

Production builds carry no clock reads: without ``BB_TIMELINE=1`` at build time the entry point
``bb_flash_bwd_timeline`` does not exist and this tool says so."""
from __future__ import annotations

import argparse
import ctypes
import sys

import numpy as np
import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--hq", type=int, default=16)
    ap.add_argument("--hk", type=int, default=8)
    ap.add_argument("--hd", type=int, default=128)
    a = ap.parse_args(argv)
    from brain_b200.ops import _cuda
    from brain_b200.ops.attention import flash_attention
    lib = _cuda.lib()
    if not hasattr(lib, "bb_flash_bwd_timeline"):
        print("this build has no timeline stamps: rebuild with BB_TIMELINE=1", file=sys.stderr)
        return 2
    B, T, hq, hk, hd = a.batch, a.seq, a.hq, a.hk, a.hd
    q, k, v = (torch.randn(B * T, h * hd, device="cuda").bfloat16().requires_grad_() for h in (hq, hk, hk))
    o = flash_attention(q, k, v, B, T, hq, hk, hd, True)
    do = torch.randn_like(o)
    for _ in range(2):
        torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
    tl = torch.zeros(6 * 4096, device="cuda", dtype=torch.int64)
    lib.bb_flash_bwd_timeline(ctypes.c_void_p(tl.data_ptr()))
    torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
    torch.cuda.synchronize()
    lib.bb_flash_bwd_timeline(ctypes.c_void_p(0))
    _cuda.check_error()
    t = tl.cpu().numpy()
    for name, base in (("dQ kernel", 0), ("dK/dV kernel", 3 * 4096)):
        m = t[base:base + 4096].reshape(-1, 4)
        m = m[m[:, 0] > 0]
        if len(m) < 6:
            print(name, ": no stamps")
            continue
        print(f"{name}: {len(m)} iterations stamped, {(m[-1, 0] - m[0, 0]) / (len(m) - 1):.0f} clk per iteration")
        mm = m[2:-2]
        if base == 0:
            print(f"  MMA thread: issue of dQ, next dP, next S (with waits for K/V tiles) {np.mean(mm[:, 1] - mm[:, 0]):.0f} clk")
        else:
            print(f"  MMA thread: dV + next S^T issue {np.mean(mm[:, 1] - mm[:, 0]):.0f}, wait for dS {np.mean(mm[:, 2] - mm[:, 1]):.0f}, "
                  f"dK + next dP^T issue {np.mean(mm[:, 3] - mm[:, 2]):.0f} clk")
        for g in (0, 1):
            w = t[base + 4096 * (1 + g): base + 4096 * (2 + g)].reshape(-1, 4)
            w = w[w[:, 0] > 0]
            d = w[2:-2]
            print(f"  warpgroup {g}: wait for S {np.mean(d[:, 1] - d[:, 0]):.0f}, phase 1 {np.mean(d[:, 2] - d[:, 1]):.0f}, "
                  f"wait for dP {np.mean(d[:, 3] - d[:, 2]):.0f}, phase 2 + loop {np.mean(w[3:-1, 0] - d[:, 3]):.0f} clk")
    return 0


if __name__ == "__main__":
    sys.exit(main())
