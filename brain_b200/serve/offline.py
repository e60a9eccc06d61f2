"""Offline batch serving: build an engine + scheduler sized for a set of prompts, run to idle, and
report aggregate throughput (reference: ``brain qwen3 serve``, crates/cli/src/qwen_cli.rs:158-267 —
pool sizing ``blocks_per_seq * n + n``, EOS ``<|im_end|>``, the ``served N prompts …`` line)."""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

from .engine import QwenEngine
from .sampling import SampleParams
from .scheduler import Scheduler


def serve_prompts(model, prompts: Sequence[Sequence[int]], max_new: int = 64, block_size: int = 16,
                  weights: str = "bf16", eos: Optional[int] = None, params: Optional[SampleParams] = None,
                  seed: int = 0, max_batch: Optional[int] = None, tp=None, kv_dtype: str = "bf16",
                  kv_clip=None) -> Dict:
    n = len(prompts)
    max_prompt = max(len(p) for p in prompts)
    max_len = max_prompt + max_new + 8
    blocks_per_seq = -(-max_len // block_size)
    eng = QwenEngine(model, block_size=block_size, num_blocks=blocks_per_seq * n + n,
                     max_seq_len=blocks_per_seq * block_size, max_prefill=max(max_prompt, 1),
                     weights=weights, tp=tp, kv_dtype=kv_dtype, kv_clip=kv_clip)
    sched = Scheduler(eng, max_batch=max_batch or n, eos=eos, mixed=True)
    ids = [sched.submit(list(p), max_new, params, seed=seed + i) for i, p in enumerate(prompts)]
    t0 = time.perf_counter()
    sched.run_until_idle()
    if eng.cuda:
        import torch
        torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    outs: List[List[int]] = [sched.tokens_of(r) for r in ids]
    total = sum(len(o) for o in outs)
    return {"outputs": outs, "tokens": total, "secs": secs, "tok_s": total / max(secs, 1e-9),
            "engine": eng, "stats": sched.stats()}
