"""A/B of the scheduler's mixed steps on one GPU: the same closed-loop serving workload through one
engine with prompt chunks and the decode batch as separate forwards, then as one forward per step.

    python -m brain_b200.perf.mixed_ab [--model 8b --requests 64 --concurrency 32 --out-tokens 48]

Prints one JSON line per arm (a short warm-up arm that builds the decode graphs, then
separate / mixed / separate again): wall time, output tokens per second, p50 time to first token and
per-token latency, and the engine's own time split."""
from __future__ import annotations

import argparse
import json
import sys
import time


def main(argv=None) -> int:
    import torch
    from ..models.config import QwenConfig
    from ..serve.engine import QwenEngine
    from .configs import _random_qwen
    from .driver import drive
    from .metrics import Summary
    from .targets import SchedulerTarget
    from .workload import Arrival, standard
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="8b")
    ap.add_argument("--weights", default="int8", choices=["int8", "bf16"])
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--concurrency", type=int, default=32)
    ap.add_argument("--out-tokens", type=int, default=48)
    a = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    cfg = QwenConfig.preset(a.model, 4096)
    conc = a.concurrency
    per_seq = -(-(2048 + a.out_tokens + 16) // 16)
    model = _random_qwen(cfg, dev)
    eng = QwenEngine(model, block_size=16, num_blocks=per_seq * conc + conc, max_seq_len=per_seq * 16,
                     max_prefill=2048, weights=a.weights, cuda_graphs=True)
    del model
    torch.cuda.empty_cache()
    for arm, mixed in (("warm", False), ("separate", False), ("mixed", True), ("separate2", False)):
        n = 8 if arm == "warm" else a.requests
        wl = standard("serving_mix", Arrival.closed_loop(min(conc, n)), n, seed=1 if arm == "warm" else 0,
                      vocab=cfg.vocab)
        wl.classes[0].output.n = 8 if arm == "warm" else a.out_tokens
        target = SchedulerTarget(None, max_batch=conc, ctx=per_seq * 16, engine=eng, name=f"qwen3-{a.model}",
                                 mixed=mixed, prefix_cache=False)
        for k in eng.acct:
            eng.acct[k] = type(eng.acct[k])(0)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        run = drive(target, wl)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        s = Summary.build(run.records, dt, wl.classes[0].slo)
        j = s.to_json()
        print(json.dumps({"arm": arm, "mixed": mixed, "wall_s": round(dt, 4), "out_tok_s": round(s.output_per_s, 1),
                          "completed": s.completed, "ttft_ms_p50": j["ttfa_ms"].get("p50"),
                          "tpot_ms_p50": j["tpoa_ms"].get("p50"),
                          "engine_time": {k: (round(v, 3) if isinstance(v, float) else v)
                                          for k, v in eng.acct.items()}}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
