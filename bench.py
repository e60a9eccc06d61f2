#!/usr/bin/env python
"""Headline benchmark: Qwen3-0.6B bf16 pre-training tokens/s, ZeRO-style data parallel, seq 4096,
global batch 64 sequences of uniform-random token ids (synthetic data, random-init weights).

    python bench.py --gpus N --steps K --warmup W           (N>1: launched by torch.distributed.run)

Prints ONE JSON line on rank 0.  ``value`` is device-timed (CUDA events, max over ranks) with the
step's inputs already resident; ``e2e`` times the public ``Trainer.train_step`` call including the
pinned-host -> device copy of every step's tokens/targets and the device -> host read of the loss.
``--impl reference`` would run the unmodified reference; it cannot be built here (Rust workspace,
no cargo/rustc in the image, GPU path is a graphics API), so that arm prints an ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "nccl", "torchlib"])
    ap.add_argument("--model", default="0.6b")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--global-batch", type=int, default=64)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override depth (invalidates the number)")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of this rank's GPU during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def main():
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is a Rust/wgpu workspace: no cargo/rustc in the image, pip "
                          "finds no Python project at its root, and its GPU path is a graphics API "
                          "(unavailable on this box)"}))
        return 0

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # re-launch under torch.distributed.run so `python bench.py --gpus N` also works by hand
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                   f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port",
                   os.environ.get("MASTER_PORT", "29511"), os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from brain_b200.data.rng import Rng
    from brain_b200.engine import Trainer
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.ops import _cuda
    from brain_b200.parallel.zero import ZeroDP

    cfg = QwenConfig.preset(args.model, block_size=args.seq)
    if args.layers:
        cfg.n_layers = args.layers
    torch.manual_seed(0)
    model = Qwen3(cfg).init_weights(seed=0)
    if args.impl == "torchlib":
        # stock PyTorch on the same architecture (cuBLAS / SDPA / fused AdamW / DDP): the library
        # anchor on this box, NOT the reference project and none of this repository's kernels
        from brain_b200.perf.torchlib_ref import TorchlibTrainer
        trainer = TorchlibTrainer(cfg, dev, world, betas=(0.9, 0.95), weight_decay=0.1, grad_clip=1.0)
    else:
        dp = ZeroDP(impl="fused" if args.impl == "native" else "nccl") if world > 1 else None
        trainer = Trainer(model, device=dev, betas=(0.9, 0.95), weight_decay=0.1, grad_clip=1.0, dp=dp)

    assert args.global_batch % world == 0
    per_rank = args.global_batch // world
    micro = min(args.micro_batch, per_rank)
    T = args.seq
    n_steps = args.warmup + args.steps
    # synthetic uniform token ids (SplitMix64, seed 0), a distinct slice per rank and step, pinned
    rng = Rng(0 + 7919 * rank)
    host_tok, host_tgt = [], []
    for _ in range(2 * n_steps):
        ids = torch.from_numpy(rng.tokens(per_rank * (T + 1), cfg.vocab)).view(per_rank, T + 1)
        host_tok.append(ids[:, :T].contiguous().pin_memory())
        host_tgt.append(ids[:, 1:].contiguous().pin_memory())
    global_count = args.global_batch * T
    lr = 3e-4

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed: inputs resident on the GPU --------------------------------------------
    dev_tok = [t.to(dev) for t in host_tok[:n_steps]]
    dev_tgt = [t.to(dev) for t in host_tgt[:n_steps]]
    for i in range(args.warmup):
        trainer.train_step(dev_tok[i], dev_tgt[i], lr, micro, global_count)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _cuda.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    loss = None
    for i in range(args.warmup, n_steps):
        loss = trainer.train_step(dev_tok[i], dev_tgt[i], lr, micro, global_count)
    ev1.record()
    barrier()
    launches = _cuda.launch_count - launches0
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    t_ms = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(t_ms.item()) / args.steps
    tok_per_s = global_count / (ms_per_step / 1e3)
    loss_t = loss.detach().clone().reshape(1)
    if world > 1:
        dist.all_reduce(loss_t)        # each rank holds its rows' share of the global mean
    final_loss = float(loss_t.item())
    _cuda.check_error()
    del dev_tok, dev_tgt

    # ---- end to end: pinned host inputs every step + loss read back --------------------------
    e2e = None
    if not args.no_e2e:
        for i in range(1):
            trainer.train_step(host_tok[n_steps + i], host_tgt[n_steps + i], lr, micro, global_count)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            l = trainer.train_step(host_tok[n_steps + 1 + i], host_tgt[n_steps + 1 + i], lr, micro,
                                   global_count)
            _ = float(l.item())   # D2H read of the step's loss
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], device=dev)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e_s = float(dt.item()) / args.steps
        e2e = {"value": global_count / e2e_s, "unit": "tokens/s",
               "h2d_bytes_per_step": int(2 * per_rank * T * 4), "d2h_bytes_per_step": 4,
               "ms_per_step": e2e_s * 1e3}

    if rank == 0:
        out = {
            "metric": "train tok/s (Qwen3-0.6B bf16 ZeRO-DP, seq 4096, global batch 64)",
            "value": tok_per_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": args.impl,
            "config": {"model": f"qwen3-{args.model}", "global_batch": args.global_batch,
                       "seq_len": T, "parallelism": f"dp{world}", "micro_batch": micro,
                       "layers": cfg.n_layers,
                       "optimizer": ("torch.optim.AdamW(fused), fp32 params under bf16 autocast, DDP, clip 1.0"
                                     if args.impl == "torchlib" else "AdamW sharded (ZeRO-1), clip 1.0"),
                       "l2": "per-step working set (weights+grads+activations, >10 GB) exceeds the 126 MB L2"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": final_loss,
            "mfu_vs_measured_sustained": None,
        }
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
            fl = model.flops_per_token(T, True) * tok_per_s / world
            out["mfu_vs_measured_sustained"] = fl / (peaks["bf16_tflops_sustained"] * 1e12)
        except Exception:
            pass
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
