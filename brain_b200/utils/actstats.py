"""Activation-magnitude statistics over named streams with bounded memory (reference:
crates/model/src/actstats.rs:29-122 — a strided subsample of ``|x|`` per stream; ``quantile`` for
sweeping clip ceilings; ``report`` sorted by outlier ratio, the most quantisation-hostile first)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch


@dataclass
class StreamReport:
    name: str
    absmax: float
    p99: float
    p9999: float
    outlier_ratio: float      # absmax / p99: how much a max-based scale wastes on outliers
    seen: int


class _Stream:
    __slots__ = ("sample", "seen", "absmax", "stride", "fill")

    def __init__(self, cap: int):
        self.sample = torch.empty(cap, dtype=torch.float32)
        self.fill = 0
        self.seen = 0
        self.absmax = 0.0
        self.stride = 1


class Collector:
    """``observe(name, x)`` records ``|x|``; each stream keeps at most ``cap`` values.  When the
    buffer fills, every other kept value is dropped and the sampling stride doubles, so the kept set
    stays a uniform strided subsample of everything seen (deterministic: no random numbers)."""

    def __init__(self, cap: int = 1 << 16):
        assert cap >= 2 and cap % 2 == 0
        self.cap = cap
        self.streams: Dict[str, _Stream] = {}

    def observe(self, name: str, x: torch.Tensor) -> None:
        a = x.detach().reshape(-1).abs().float().cpu()
        if a.numel() == 0:
            return
        st = self.streams.get(name)
        if st is None:
            st = self.streams[name] = _Stream(self.cap)
        st.absmax = max(st.absmax, float(a.max()))
        # positions (in the stream's global order) that the current stride keeps
        first = (-st.seen) % st.stride
        keep = a[first::st.stride]
        st.seen += a.numel()
        while keep.numel():
            room = self.cap - st.fill
            take = keep[:room]
            st.sample[st.fill:st.fill + take.numel()] = take
            st.fill += take.numel()
            keep = keep[take.numel():]
            if st.fill == self.cap:
                # halve the kept set, double the stride; what is left of `keep` follows the new stride
                st.sample[: self.cap // 2] = st.sample[0:self.cap:2].clone()
                st.fill = self.cap // 2
                st.stride *= 2
                keep = keep[0::2]      # the next position, cap * stride, is a multiple of the new stride

    def quantile(self, name: str, q: float) -> Optional[float]:
        st = self.streams.get(name)
        if st is None or st.fill == 0:
            return None
        return float(torch.quantile(st.sample[:st.fill], min(max(q, 0.0), 1.0)))

    def report(self) -> List[StreamReport]:
        out = []
        for name, st in self.streams.items():
            p99 = self.quantile(name, 0.99) or 0.0
            out.append(StreamReport(name, st.absmax, p99, self.quantile(name, 0.9999) or 0.0,
                                    st.absmax / p99 if p99 > 0 else float("inf"), st.seen))
        return sorted(out, key=lambda r: -r.outlier_ratio)
