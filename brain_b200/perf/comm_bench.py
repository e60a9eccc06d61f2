"""Latency of the peer-memory two-shot all-reduce against NCCL on the same ranks, and device time of
the fused tensor-parallel GEMMs (all-gather -> GEMM, GEMM -> reduce-scatter) against their unfused
NCCL form and against the roofline max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s).

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
    ap.add_argument("--gemm-rows", type=int, nargs="*", default=[8192, 16384],
                    help="token rows (all ranks together) of the fused GEMM + collective rows")
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
    # ---- fused GEMM + collective (sequence-parallel Megatron shapes of a d = 4096 layer)
    from ..utils import roof
    r = roof.measure()
    peak = r.bf16_tflops * 1e12
    link = r.nvlink_gbs * 1e9           # measured peer copy, per direction per GPU
    world = dist.get_world_size()
    ref_tp = TensorParallel(impl="nccl", device=dev)

    def timed(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    for rows in a.gemm_rows:
        K = a.dim
        n_col = 3 * a.dim // world          # column-parallel: this rank's slice of a 3d-wide projection
        xs = torch.randn(rows // world, K, device=dev).bfloat16()
        w1 = (torch.randn(n_col, K, device=dev) * 0.02).bfloat16()
        f_us = timed(lambda: tp.ag_gemm(xs, w1))
        n_us = timed(lambda: ref_tp.ag_gemm(xs, w1))
        flops = 2.0 * rows * n_col * K
        nv = (world - 1) * (rows // world) * K * 2            # bytes this rank pulls
        roof_us = max(flops / peak, nv / link) * 1e6
        if rank == 0:
            print(json.dumps({"op": "all_gather->gemm", "world": world, "M": rows, "N_local": n_col, "K": K,
                              "fused_us": round(f_us, 1), "nccl_us": round(n_us, 1), "roof_us": round(roof_us, 1),
                              "fused_frac_of_roof": round(roof_us / f_us, 3)}), flush=True)
        k_row = a.dim // world              # row-parallel: this rank's slice of the reduction dim
        x2 = torch.randn(rows, k_row, device=dev).bfloat16()
        w2 = (torch.randn(a.dim, k_row, device=dev) * 0.02).bfloat16()
        f_us = timed(lambda: tp.gemm_rs(x2, w2))
        n_us = timed(lambda: ref_tp.gemm_rs(x2, w2))
        flops = 2.0 * rows * a.dim * k_row
        nv = (world - 1) * (rows // world) * a.dim * 2        # bytes this rank sends
        roof_us = max(flops / peak, nv / link) * 1e6
        if rank == 0:
            print(json.dumps({"op": "gemm->reduce_scatter", "world": world, "M": rows, "N": a.dim, "K_local": k_row,
                              "fused_us": round(f_us, 1), "nccl_us": round(n_us, 1), "roof_us": round(roof_us, 1),
                              "fused_frac_of_roof": round(roof_us / f_us, 3)}), flush=True)
    _cuda.check_error()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
