"""Analytic cost registry: FLOPs / integer ops / bytes for every native kernel and whole-model
forward/backward reports (reference: crates/gpu-core/src/cost.rs:117 ``kernel_cost`` and :217
``coverage`` — an honest share of launches the registry can cost; the per-model ``cost_fwd`` /
``cost_bwd`` reports printed by ``brain flops``, crates/cli/src/flops_cli.rs:52-80)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple


@dataclass
class OpCost:
    flops: float = 0.0
    int_ops: float = 0.0
    bytes: float = 0.0

    def __iadd__(self, o: "OpCost"):
        self.flops += o.flops
        self.int_ops += o.int_ops
        self.bytes += o.bytes
        return self

    def scaled(self, k: float) -> "OpCost":
        return OpCost(self.flops * k, self.int_ops * k, self.bytes * k)


def gemm(M, N, K, es_in=2, es_out=2, int8=False) -> OpCost:
    ops = 2.0 * M * N * K
    by = es_in * (M * K + N * K) + es_out * M * N
    return OpCost(0.0, ops, by) if int8 else OpCost(ops, 0.0, by)


def attention_fwd(B, T, S, hq, hk, hd, causal=True, es=2) -> OpCost:
    pairs = B * hq * (T * S / 2.0 + T / 2.0 if causal and T == S else T * S)
    return OpCost(4.0 * pairs * hd + 6.0 * pairs, 0.0, es * (2 * B * T * hq * hd + 2 * B * S * hk * hd))


def attention_bwd(B, T, S, hq, hk, hd, causal=True, es=2) -> OpCost:
    """Five model GEMMs per tile pair (the recomputed scores in the second kernel are overhead,
    not model FLOPs)."""
    pairs = B * hq * (T * S / 2.0 + T / 2.0 if causal and T == S else T * S)
    return OpCost(10.0 * pairs * hd + 10.0 * pairs, 0.0,
                  es * (4 * B * T * hq * hd + 4 * B * S * hk * hd))


def rowwise(rows, d, reads=1, writes=1, es=2, flops_per_elem=4.0) -> OpCost:
    return OpCost(flops_per_elem * rows * d, 0.0, es * rows * d * (reads + writes))


def kernel_cost(name: str, **p) -> Optional[OpCost]:
    """Cost of one launch of native kernel ``name``; None when the registry cannot cost it."""
    if name in ("gemm_bf16", "gemm_bf16_tp"):
        return gemm(p["M"], p["N"], p["K"], 2, p.get("es_out", 2))
    if name == "gemm_i8":
        return gemm(p["M"], p["N"], p["K"], 1, 2, int8=True)
    if name == "gemm_bf16_grouped":
        return gemm(p["M"], p["N"], p["K"], 2, p.get("es_out", 2))
    if name == "flash_fwd":
        return attention_fwd(p["B"], p["T"], p["S"], p["hq"], p["hk"], p["hd"], p.get("causal", True))
    if name == "flash_bwd":
        return attention_bwd(p["B"], p["T"], p["S"], p["hq"], p["hk"], p["hd"], p.get("causal", True))
    if name in ("rmsnorm_fwd", "layernorm_fwd"):
        return rowwise(p["rows"], p["d"], 1, 1)
    if name in ("rmsnorm_bwd_dx", "layernorm_bwd_dx"):
        return rowwise(p["rows"], p["d"], 2, 1, flops_per_elem=8.0)
    if name in ("swiglu_fwd",):
        return rowwise(p["rows"], p["d"], 2, 1, flops_per_elem=8.0)
    if name in ("swiglu_bwd",):
        return rowwise(p["rows"], p["d"], 3, 2, flops_per_elem=16.0)
    if name == "cross_entropy":
        return rowwise(p["rows"], p["d"], 1, p.get("writes", 1), flops_per_elem=6.0)
    if name == "adamw":
        n = p["n"]
        return OpCost(14.0 * n, 0.0, n * (4 + 4 + 4 + 2) + n * (4 + 4 + 2))
    if "bytes" in p:
        return OpCost(p.get("flops", 0.0), 0.0, p["bytes"])
    return None


_CLASSES = ("matmul", "attention", "norm", "elementwise", "loss", "embed", "optimizer")


@dataclass
class CostReport:
    steps: int = 0
    by_class: Dict[str, OpCost] = field(default_factory=dict)
    uncosted: int = 0

    def add(self, cls: str, c: Optional[OpCost], n: int = 1):
        self.steps += n
        if c is None:
            self.uncosted += n
            return
        self.by_class.setdefault(cls, OpCost()).__iadd__(c.scaled(n))

    @property
    def total(self) -> OpCost:
        t = OpCost()
        for c in self.by_class.values():
            t += c
        return t

    def merge(self, o: "CostReport"):
        self.steps += o.steps
        self.uncosted += o.uncosted
        for k, c in o.by_class.items():
            self.by_class.setdefault(k, OpCost()).__iadd__(c)

    def coverage(self) -> float:
        return 1.0 if self.steps == 0 else 1.0 - self.uncosted / self.steps

    def __str__(self):
        t = self.total
        lines = [f"{'class':<12} {'GFLOP':>12} {'Gint-op':>12} {'MB moved':>12} {'FLOP/B':>8}"]
        for k in _CLASSES:
            c = self.by_class.get(k)
            if c is None:
                continue
            ai = (c.flops + c.int_ops) / c.bytes if c.bytes else 0.0
            lines.append(f"{k:<12} {c.flops / 1e9:>12.3f} {c.int_ops / 1e9:>12.3f} {c.bytes / 1e6:>12.2f} {ai:>8.1f}")
        ai = (t.flops + t.int_ops) / t.bytes if t.bytes else 0.0
        lines.append(f"{'total':<12} {t.flops / 1e9:>12.3f} {t.int_ops / 1e9:>12.3f} {t.bytes / 1e6:>12.2f} {ai:>8.1f}")
        lines.append(f"steps {self.steps}  coverage {100 * self.coverage():.0f}%")
        return "\n".join(lines)


def even_shards(n_layers: int, n: int):
    """(start, end, embed, head) per stage, layers split evenly (flops_cli.rs:38-48)."""
    return [(s * n_layers // n, (s + 1) * n_layers // n, s == 0, s == n - 1) for s in range(n)]


def qwen_cost(cfg, b: int, t: int, train: bool = False, i8: bool = False,
              shard: Optional[Tuple[int, int, bool, bool]] = None) -> Tuple[CostReport, Optional[CostReport]]:
    """(forward, backward) cost of a Qwen-family stage holding layers ``[start, end)``."""
    start, end, embed, head = shard or (0, cfg.n_layers, True, True)
    rows, d = b * t, cfg.d_model
    fwd, bwd = CostReport(), CostReport()
    es_w = 1 if i8 else 2
    if embed:
        fwd.add("embed", OpCost(0, 0, 2 * rows * d * 2))
        bwd.add("embed", OpCost(rows * d, 0, rows * d * (2 + 4)))
    for _ in range(start, end):
        fwd.add("norm", rowwise(rows, d), 2)
        for (n, k) in ((cfg.q_dim + 2 * cfg.kv_dim, d), (d, cfg.q_dim), (2 * cfg.d_ff, d), (d, cfg.d_ff)):
            fwd.add("matmul", gemm(rows, n, k, es_w, 2, int8=i8))
            bwd.add("matmul", gemm(rows, k, n), 1)            # dX
            bwd.add("matmul", gemm(n, k, rows, 2, 4), 1)      # dW (fp32 accumulate)
        fwd.add("elementwise", rowwise(rows, cfg.q_dim + cfg.kv_dim, 1, 1, flops_per_elem=10.0))   # qk-norm + rope
        fwd.add("attention", attention_fwd(b, t, t, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim))
        fwd.add("elementwise", rowwise(rows, cfg.d_ff, 2, 1, flops_per_elem=8.0))                  # swiglu
        bwd.add("norm", rowwise(rows, d, 2, 1, flops_per_elem=8.0), 2)
        bwd.add("attention", attention_bwd(b, t, t, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim))
        bwd.add("elementwise", rowwise(rows, cfg.q_dim + cfg.kv_dim, 2, 1, flops_per_elem=20.0))
        bwd.add("elementwise", rowwise(rows, cfg.d_ff, 3, 2, flops_per_elem=16.0))
    if head:
        fwd.add("norm", rowwise(rows, d))
        fwd.add("matmul", gemm(rows, cfg.vocab, d, es_w, 2, int8=i8))
        if train:
            fwd.add("loss", rowwise(rows, cfg.vocab, 1, 1, flops_per_elem=6.0))
            bwd.add("matmul", gemm(rows, d, cfg.vocab))
            bwd.add("matmul", gemm(cfg.vocab, d, rows, 2, 4))
            bwd.add("norm", rowwise(rows, d, 2, 1, flops_per_elem=8.0))
    return fwd, (bwd if train else None)


def gpt_cost(cfg, b: int, t: int, train: bool = False,
             shard: Optional[Tuple[int, int, bool, bool]] = None) -> Tuple[CostReport, Optional[CostReport]]:
    start, end, embed, head = shard or (0, cfg.n_layers, True, True)
    rows, d, ff = b * t, cfg.d_model, cfg.d_ff
    hd = d // cfg.n_heads
    fwd, bwd = CostReport(), CostReport()
    if embed:
        fwd.add("embed", OpCost(rows * d, 0, 3 * rows * d * 2))
        bwd.add("embed", OpCost(2 * rows * d, 0, rows * d * (2 + 8)))
    for _ in range(start, end):
        fwd.add("norm", rowwise(rows, d, flops_per_elem=8.0), 2)
        for (n, k) in ((3 * d, d), (d, d), (ff, d), (d, ff)):
            fwd.add("matmul", gemm(rows, n, k))
            bwd.add("matmul", gemm(rows, k, n))
            bwd.add("matmul", gemm(n, k, rows, 2, 4))
        fwd.add("attention", attention_fwd(b, t, t, cfg.n_heads, cfg.n_heads, hd))
        fwd.add("elementwise", rowwise(rows, ff, 1, 1, flops_per_elem=12.0))
        bwd.add("norm", rowwise(rows, d, 2, 1, flops_per_elem=12.0), 2)
        bwd.add("attention", attention_bwd(b, t, t, cfg.n_heads, cfg.n_heads, hd))
        bwd.add("elementwise", rowwise(rows, ff, 2, 1, flops_per_elem=20.0))
    if head:
        fwd.add("norm", rowwise(rows, d, flops_per_elem=8.0))
        fwd.add("matmul", gemm(rows, cfg.vocab, d))
        if train:
            fwd.add("loss", rowwise(rows, cfg.vocab, 1, 1, flops_per_elem=6.0))
            bwd.add("matmul", gemm(rows, d, cfg.vocab))
            bwd.add("matmul", gemm(cfg.vocab, d, rows, 2, 4))
            bwd.add("norm", rowwise(rows, d, 2, 1, flops_per_elem=12.0))
    return fwd, (bwd if train else None)
