#!/usr/bin/env python3
"""The serving engine without a server: paged KV cache + continuous-batching scheduler driven from
Python.  A synthetic Qwen3 (random weights) keeps it self-contained; pass --weights/--tokenizer for a
real checkpoint.

    python examples/serving/offline_batch.py --requests 12 --max-batch 4
Shows: requests queue while the batch is full, prompts longer than the prefill chunk are processed
in pieces, a shared prefix is served from the prefix cache, one request is cancelled mid-flight."""
import argparse
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from brain_b200.perf.targets import synth_qwen  # noqa: E402
from brain_b200.serve.engine import QwenEngine  # noqa: E402
from brain_b200.serve.scheduler import Scheduler  # noqa: E402


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shape", default="2x64x4x512", help="layers x d_model x heads x vocab of the synthetic model")
    ap.add_argument("--requests", type=int, default=12)
    ap.add_argument("--max-batch", type=int, default=4)
    ap.add_argument("--max-new", type=int, default=12)
    ap.add_argument("--weights", default="bf16", choices=["bf16", "int8"])
    a = ap.parse_args()
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    model = synth_qwen(a.shape, dev)
    vocab = model.cfg.vocab
    eng = QwenEngine(model, block_size=16, num_blocks=256, max_seq_len=512, max_prefill=64, weights=a.weights)
    sched = Scheduler(eng, max_batch=a.max_batch, window=4, mixed=True)
    rng = np.random.default_rng(0)
    shared = rng.integers(0, vocab, 48).tolist()          # a common system prompt: prefix-cache hits
    ids = []
    for i in range(a.requests):
        tail = rng.integers(0, vocab, int(rng.integers(8, 120))).tolist()
        ids.append(sched.submit(shared + tail, a.max_new))
    cancelled = None
    steps = 0
    while not sched.is_idle():
        rep = sched.step()
        steps += 1
        if steps == 3 and cancelled is None:
            cancelled = ids[-1]
            kept = sched.cancel(cancelled)
            print(f"step {steps}: cancelled request {cancelled} after {len(kept)} tokens")
        if rep.admitted or rep.finished:
            print(f"step {steps}: admitted {rep.admitted}, prefill tokens {rep.prefill_tokens}, decoded rows "
                  f"{rep.decoded} x window {rep.window}{' (one forward)' if rep.mixed else ''}, finished {rep.finished}")
    st = sched.stats()
    print(f"{steps} steps; generated {st['generated']} tokens; prefix cache served "
          f"{st['kv_prefix_hit_tokens']} of {st['kv_prefix_lookup_tokens']} prompt tokens; "
          f"free blocks {st['free_blocks']}/{st['num_blocks']}")
    for r in ids[:3]:
        print(f"request {r}: {sched.tokens_of(r)}")
    assert all(len(sched.tokens_of(r)) == a.max_new for r in ids if r != cancelled)


if __name__ == "__main__":
    main()
