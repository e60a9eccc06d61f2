"""Clocks per ``tcgen05.mma`` (M = 128, K = 16, bf16) by N and operand source, measured on the device
(``csrc/kernels/mma_probe.cu``: one thread per CTA issues a chain of MMAs over shared memory and times
it with ``clock64``).  The table decides tile shapes; on B200 every N <= 128 costs about as much as
N = 128.

    python -m brain_b200.perf.mma_probe [--grid 148]          (or: brain perf tool mma-probe)"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--grid", type=int, default=148)
    ap.add_argument("--per", type=int, default=256)
    a = ap.parse_args(argv)
    from brain_b200.ops import _cuda
    from brain_b200.ops._cuda import call, stream_ptr
    out = torch.zeros(a.grid, device="cuda", dtype=torch.int64)
    rows = []
    for ts in (0, 1):
        for mn in (0, 1):
            for n in ((32, 64, 128) if mn else (32, 64, 128, 256)):
                call("mma_probe", n, ts, mn, a.grid, 20, a.per, out, stream_ptr())
                torch.cuda.synchronize()
                clk = float(out.min().item()) / a.per
                rows.append({"n": n, "a": "tmem" if ts else "smem", "b": "mn-major" if mn else "k-major",
                             "clk_per_mma": round(clk, 1), "ideal_clk": n // 2,
                             "efficiency": round((n / 2) / clk, 3)})
    _cuda.check_error()
    print(json.dumps({"grid": a.grid, "mma_per_chain": a.per, "rows": rows}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
