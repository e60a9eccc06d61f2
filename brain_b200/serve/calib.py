"""KV-cache calibration statistics (reference: ``brain qwen3 calib``, crates/cli/src/qwen_cli.rs:
1004-1100 and crates/model/src/kvcalib.rs — per-layer, per-KV-head clip values for a quantised KV
cache taken at a percentile of |K| and |V| over calibration text).

Each sequence is prefilled through the serving engine; the post-RoPE K and V rows are then read
back from the paged pool, so the statistics describe exactly what a quantised cache would store."""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

from .engine import QwenEngine


@torch.no_grad()
def collect_kv_stats(model, seqs: Sequence[Sequence[int]], percentile: float = 0.999,
                     block_size: int = 16, max_samples: int = 1 << 20) -> Dict:
    longest = max(len(s) for s in seqs)
    nblk = -(-longest // block_size)
    eng = QwenEngine(model, block_size=block_size, num_blocks=nblk + 1, max_seq_len=nblk * block_size,
                     max_prefill=min(longest, 2048))
    from ..utils.actstats import Collector
    L, hk = len(eng.layers), eng.hk
    cap = max(2, (min(max_samples, 1 << 20) // 2) * 2)
    stats = Collector(cap)                      # bounded memory however long the calibration set is
    table = np.arange(nblk, dtype=np.int32)
    total = 0
    for s in seqs:
        toks = np.asarray(s, dtype=np.int64)
        n = len(toks)
        if n == 0:
            continue
        for st in range(0, n, eng.max_prefill_tokens):
            en = min(n, st + eng.max_prefill_tokens)
            eng.prefill_chunk(toks[st:en], st, table, last=False)
        used = -(-n // block_size)
        for li in range(L):
            # pool layout [blocks][hk][bs][hd] -> per head [tokens, hd]
            k = eng.kc[li][:used].permute(1, 0, 2, 3).reshape(hk, used * block_size, -1)[:, :n]
            v = eng.vc[li][:used].permute(1, 0, 2, 3).reshape(hk, used * block_size, -1)[:, :n]
            for h in range(hk):
                stats.observe(f"k.{li}.{h}", k[h])
                stats.observe(f"v.{li}.{h}", v[h])
        total += n

    def reduce(name):
        return stats.streams[name].absmax, stats.quantile(name, percentile)

    out = {"tokens": total, "percentile": percentile, "layers": [], "k_clip": [], "v_clip": []}
    for li in range(L):
        ks = [reduce(f"k.{li}.{h}") for h in range(hk)]
        vs = [reduce(f"v.{li}.{h}") for h in range(hk)]
        out["layers"].append({"layer": li, "k_absmax": [a for a, _ in ks], "v_absmax": [a for a, _ in vs]})
        out["k_clip"].append([q for _, q in ks])
        out["v_clip"].append([q for _, q in vs])
    return out


def load_kv_clip(weights_path: str):
    """The ``kv_calib.json`` written beside a checkpoint by ``brain qwen3 calib`` ->
    ``{"k_clip": [[…per kv head] per layer], "v_clip": …}`` for ``QwenEngine(kv_clip=…)``; None when
    the file is absent."""
    import json
    import os
    path = os.path.join(os.path.dirname(weights_path) or ".", "kv_calib.json")
    if not os.path.exists(path):
        return None
    d = json.loads(open(path).read())
    return {"k_clip": d["k"], "v_clip": d["v"]}
