"""Single-GPU time of one decode step and one prefill step of the serving engine at the PER-RANK
shapes of a tensor-parallel deployment (no all-reduce): what a rank spends between collectives.

    python -m brain_b200.perf.serve_micro [--model 8b --tp 8 --batch 256 --weights int8]

Prints one JSON line: decode step through the CUDA graph and eagerly, prefill of 1x256, 1x1024,
1x2048 and 4x1024 tokens, each with the native layer sequence and through the Python wrappers."""
from __future__ import annotations

import argparse
import json
import sys
import time


def main(argv=None) -> int:
    import numpy as np
    import torch
    from ..models.config import QwenConfig
    from ..ops import _cuda
    from ..serve.engine import QwenEngine
    from .configs import _random_qwen
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="8b")
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--weights", default="int8")
    ap.add_argument("--kv", default="bf16")
    a = ap.parse_args(argv)
    dev = torch.device("cuda:0")
    full = QwenConfig.preset(a.model, 4096)
    cfg = QwenConfig(vocab=full.vocab, block_size=4096, n_layers=full.n_layers, d_model=full.d_model,
                     n_heads=full.n_heads // a.tp, n_kv_heads=max(full.n_kv_heads // a.tp, 1), head_dim=full.head_dim,
                     d_ff=full.d_ff // a.tp, tie_embeddings=False, max_position_embeddings=4096)
    m = _random_qwen(cfg, dev)
    B, ctx = a.batch, 2320
    per_seq = ctx // 16
    rng = np.random.default_rng(0)
    bts = np.arange(B * per_seq, dtype=np.int32).reshape(B, per_seq)
    pos = rng.integers(600, 1800, B).astype(np.int32)
    tok = rng.integers(0, 1000, B).astype(np.int32)
    out = {"model": a.model, "tp": a.tp, "batch": B, "weights": a.weights, "kv": a.kv}

    def timed(fn, warm, it):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(it):
            fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / it * 1e3

    for native in (True, False):
        eng = QwenEngine(m, block_size=16, num_blocks=per_seq * B + B, max_seq_len=ctx, max_prefill=2048,
                         weights=a.weights, kv_dtype=a.kv, native=native)
        key = "native" if native else "python"
        res = {}
        for name, graphs in (("decode_graph_ms", True), ("decode_eager_ms", False)):
            eng.cuda_graphs = graphs
            res[name] = round(timed(lambda: eng.decode(tok, pos, bts, 1, True), 3, 10), 2)
        for nseq, n in ((1, 256), (1, 1024), (1, 2048), (4, 1024)):
            items = [(rng.integers(0, 1000, n).astype(np.int32), 0, bts[i], True, True) for i in range(nseq)]
            res[f"prefill_{nseq}x{n}_ms"] = round(timed(lambda: eng.prefill_batch(items), 2, 5), 2)
        out[key] = res
        del eng
        torch.cuda.empty_cache()
    _cuda.check_error()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
