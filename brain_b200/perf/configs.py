"""The benchmark configurations beside the flagship one that ``bench.py`` runs.

    python -m brain_b200.perf.configs cpu-dp      # GPT-2 small, fp32, CPU backend, 2 data-parallel
                                                  # thread workers, 20 steps + the d64 gradcheck gate

Each prints one JSON line.  Synthetic data (uniform-random token ids) and random-init weights."""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def cpu_dp(args) -> dict:
    """GPT-2 small (12 layers, d 768, 12 heads, ff 3072, vocab 50257, ctx 1024) fp32 on the CPU
    backend with 2 data-parallel thread workers, per-worker batch 4 x 128, AdamW lr 3e-4 betas
    0.9/0.95 wd 0.1, 20 steps; then the finite-difference gradcheck on a 2-layer d64 variant.  The
    timed oracle is the same model through plain PyTorch autograd ops on one worker."""
    from .. import gradcheck
    from ..data.rng import Rng
    from ..models.config import GptConfig
    from ..models.gpt2 import Gpt2
    from ..parallel.dp import DataParallel
    torch.manual_seed(0)
    cfg = GptConfig(vocab=50257, block_size=1024, n_layers=args.layers, d_model=768, n_heads=12, d_ff=3072)
    workers, B, T = 2, 4, 128

    def make():
        return Gpt2(cfg).init_weights(0)
    t0 = time.perf_counter()
    dp = DataParallel(make, workers, betas=(0.9, 0.95))
    build_s = time.perf_counter() - t0
    rng = Rng(0)
    losses, times = [], []
    for step in range(args.steps):
        mbs = []
        for _ in range(workers):
            toks = torch.from_numpy(rng.tokens(B * (T + 1), cfg.vocab).astype("int64")).view(B, T + 1)
            mbs.append((toks[:, :-1].to(torch.int32).contiguous(), toks[:, 1:].contiguous()))
        t1 = time.perf_counter()
        losses.append(dp.train_step(mbs, 3e-4, wd=0.1, clip=1.0))
        times.append(time.perf_counter() - t1)
    steady = times[2:] if len(times) > 4 else times
    ms = 1e3 * sum(steady) / len(steady)
    report = gradcheck.check_gpt(n_dirs=4, d_model=64)
    fails = report.failures()
    worst = report.worst()
    return {"config": "cpu-dp", "metric": "train tok/s (GPT-2 small fp32, CPU backend, 2 DP thread workers)",
            "value": workers * B * T / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms, "steps": args.steps,
            "loss_first": losses[0], "loss_last": losses[-1], "loss_decreased": losses[-1] < losses[0],
            "build_s": build_s, "threads": torch.get_num_threads(),
            "gradcheck": {"model": "gpt 2-layer d64", "tensors": len(report.entries), "failures": len(fails),
                          "worst_rel": worst.rel if worst else None, "worst_name": worst.name if worst else None},
            "dtype": "fp32", "data": "synthetic"}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("which", choices=["cpu-dp"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--layers", type=int, default=12)
    a = ap.parse_args(argv)
    out = {"cpu-dp": cpu_dp}[a.which](a)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
