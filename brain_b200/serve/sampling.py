"""Host-side sampling over the top-K candidates the device returns (descending by logit):
temperature -> top-k -> top-p nucleus -> inverse CDF with the request's SplitMix64 stream.
Reference: crates/model/src/serve.rs:119-177."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence, Tuple

from ..data.rng import Rng


@dataclass
class SampleParams:
    temp: float = 0.0
    top_k: int = 0
    top_p: float = 1.0

    @staticmethod
    def greedy() -> "SampleParams":
        return SampleParams(0.0, 0, 1.0)

    def is_greedy(self) -> bool:
        return self.temp <= 0.0


def sample_from_topk(candidates: Sequence[Tuple[int, float]], params: SampleParams, rng: Rng) -> int:
    if not candidates:
        raise ValueError("sample_from_topk: no candidates")
    if params.is_greedy():
        return candidates[0][0]
    temp = max(params.temp, 1e-6)
    n = min(params.top_k, len(candidates)) if params.top_k > 0 else len(candidates)
    vals = [v / temp for _, v in candidates[:n]]
    mx = max(vals)
    probs = [math.exp(v - mx) for v in vals]
    total = sum(probs)
    cut = n
    if 0.0 < params.top_p < 1.0 and total > 0.0:
        kept = 0.0
        for rank, p in enumerate(probs):
            kept += p
            if kept / total >= params.top_p:
                cut = rank + 1
                break
    kept_sum = sum(probs[:cut])
    r = rng.next_f32() * kept_sum
    acc = 0.0
    for i, p in enumerate(probs[:cut]):
        acc += p
        if acc >= r:
            return candidates[i][0]
    return candidates[cut - 1][0]
