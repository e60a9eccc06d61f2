"""Latency of the peer-memory two-shot all-reduce against NCCL on the same ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m brain_b200.perf.comm_bench [--rows 256 2048 8192 --dim 4096]

The fused number is device time of a CUDA graph of 64 back-to-back calls (no host launch cost in
it), max over ranks; the NCCL number is an eager loop (its launch cost included).  Rank 0 prints one
JSON line per size."""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    import torch
    import torch.distributed as dist
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="+", default=[256, 2048, 8192])
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--arena-mb", type=int, default=512)
    a = ap.parse_args(argv)
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import _cuda
    from ..parallel.tp import TensorParallel
    tp = TensorParallel(impl="fused", device=dev, arena_mb=a.arena_mb, wait_seconds=5.0)
    torch.manual_seed(rank)
    for rows in a.rows:
        x = torch.randn(rows, a.dim, device=dev).bfloat16()
        want = x.float().clone()
        dist.all_reduce(want)
        y = tp.all_reduce(x)
        torch.cuda.synchronize()
        err = ((y.float() - want).norm() / want.norm()).item()
        for _ in range(4):
            tp.all_reduce(x)
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            for _ in range(64):
                y = tp.all_reduce(x)
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(5):
            g.replay()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / (5 * 64) * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        z = x.clone()
        for _ in range(5):
            dist.all_reduce(z)
        torch.cuda.synchronize()
        s.record()
        for _ in range(50):
            dist.all_reduce(z)
        e.record()
        torch.cuda.synchronize()
        n = torch.tensor([s.elapsed_time(e) / 50 * 1e3], device=dev)
        dist.all_reduce(n, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(json.dumps({"op": "all_reduce", "world": dist.get_world_size(), "rows": rows, "dim": a.dim,
                              "mbytes": rows * a.dim * 2 / 1e6, "two_shot_us": round(t.item(), 1),
                              "nccl_eager_us": round(n.item(), 1), "rel_err": err}), flush=True)
    _cuda.check_error()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
