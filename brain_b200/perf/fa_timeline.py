"""clock64 timeline of the flash-attention backward kernels (one CTA of each kernel records when its
MMA issuer and its two softmax warpgroups wait and work).

    python -m brain_b200.perf.fa_timeline [--batch 4 --seq 4096 --hq 16 --hk 8 --hd 128]

Prints, per 64-wide unit: the MMA issuer's issue time and its wait for dS, and each warpgroup's
compute time and wait for S/dP — which tells whether the tensor pipe or the softmax is the limiter."""
from __future__ import annotations

import argparse
import ctypes

import torch

from ..ops import _cuda
from ..ops.attention import flash_attention


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--hq", type=int, default=16)
    ap.add_argument("--hk", type=int, default=8)
    ap.add_argument("--hd", type=int, default=128)
    a = ap.parse_args(argv)
    B, T, hq, hk, hd = a.batch, a.seq, a.hq, a.hk, a.hd
    mk = lambda h: torch.randn(B * T, h * hd, device="cuda").bfloat16().requires_grad_()
    q, k, v = mk(hq), mk(hk), mk(hk)
    o = flash_attention(q, k, v, B, T, hq, hk, hd, True)
    do = torch.randn_like(o)
    for _ in range(2):
        torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
    tl = torch.zeros(6 * 4096, device="cuda", dtype=torch.int64)
    _cuda.lib().bb_flash_bwd_timeline(ctypes.c_void_p(tl.data_ptr()))
    torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
    torch.cuda.synchronize()
    _cuda.lib().bb_flash_bwd_timeline(ctypes.c_void_p(0))
    _cuda.check_error()
    t = tl.cpu().numpy()
    for name, base in (("dQ kernel", 0), ("dK/dV kernel", 3 * 4096)):
        mma = t[base:base + 4096].reshape(-1, 2)
        mma = mma[mma[:, 0] > 0]
        n = len(mma)
        print(f"{name}: {n} units stamped")
        if n < 8:
            continue
        issue = mma[:, 1] - mma[:, 0]
        gap = mma[1:, 0] - mma[:-1, 1]
        print(f"  MMA issuer : {(mma[-1, 1] - mma[0, 0]) / (n - 1):.0f} clk per unit "
              f"(issuing {issue[2:-2].mean():.0f}, waiting for dS {gap[2:-2].mean():.0f})")
        for g in (0, 1):
            w = t[base + 4096 * (1 + g): base + 4096 * (2 + g)].reshape(-1, 2)
            w = w[w[:, 0] > 0]
            comp, wait = w[:, 1] - w[:, 0], w[1:, 0] - w[:-1, 1]
            print(f"  warpgroup {g}: compute {comp[2:-2].mean():.0f} clk per unit, waiting for S/dP {wait[2:-2].mean():.0f}")


if __name__ == "__main__":
    main()
