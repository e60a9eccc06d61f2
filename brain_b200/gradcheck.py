"""Finite-difference gradient gate (reference: crates/gradcheck/src/lib.rs:55-81, 115-171, 189,
217-262, 290-516; CLI gate crates/cli/src/main.rs:769-779).

``directional_check``: one analytic backward, then per parameter tensor and per Rademacher
direction ``v`` (``rng.next_f32() < 0.5 -> -1``): analytic ``<g, v>`` against the central
difference ``(L(w + eps v) - L(w - eps v)) / (2 eps)``; the direction with the smallest relative
error is kept.  A tensor passes when ``|a - n| <= atol + rtol * max(|a|, |n|)``.
The CLI gate uses eps 5e-3, 4 directions, atol 4e-3, rtol 8e-2 on a tiny GPT."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from .data.rng import Rng


@dataclass
class Entry:
    name: str
    analytic: float
    numeric: float
    rel: float


@dataclass
class Report:
    entries: List[Entry] = field(default_factory=list)

    def failures(self, atol: float = 4e-3, rtol: float = 8e-2) -> List[Entry]:
        return [e for e in self.entries
                if abs(e.analytic - e.numeric) > atol + rtol * max(abs(e.analytic), abs(e.numeric))]

    def worst(self) -> Optional[Entry]:
        return max(self.entries, key=lambda e: e.rel) if self.entries else None

    def dead_gradients(self, thresh: float = 1e-3) -> List[Entry]:
        """Analytic gradient exactly zero while the loss visibly moves (a missing backward)."""
        return [e for e in self.entries if e.analytic == 0.0 and abs(e.numeric) > thresh]

    def summary(self) -> str:
        lines = [f"{'tensor':40s} {'analytic':>13s} {'numeric':>13s} {'rel':>9s}"]
        for e in self.entries:
            lines.append(f"{e.name:40s} {e.analytic:13.6e} {e.numeric:13.6e} {e.rel:9.2e}")
        return "\n".join(lines)


def _rademacher(rng: Rng, n: int) -> torch.Tensor:
    u = rng.u64s(n)
    f = ((u >> np.uint64(11)).astype(np.float64) / float(1 << 53)).astype(np.float32)
    return torch.from_numpy(np.where(f < 0.5, -1.0, 1.0))


def directional_check(loss_fn: Callable[[], torch.Tensor], params: Dict[str, torch.Tensor],
                      eps: float = 5e-3, n_dirs: int = 4, seed: int = 0) -> Report:
    """``loss_fn()`` recomputes the scalar loss from the current values of ``params`` (leaf
    tensors with requires_grad)."""
    for p in params.values():
        p.grad = None
    loss = loss_fn()
    loss.backward()
    grads = {n: (p.grad.detach().clone() if p.grad is not None else torch.zeros_like(p))
             for n, p in params.items()}
    rng = Rng(seed)
    rep = Report()
    with torch.no_grad():
        for name, p in params.items():
            best = None
            for _ in range(n_dirs):
                v = _rademacher(rng, p.numel()).to(p.dtype).reshape(p.shape)
                analytic = float((grads[name].double() * v.double()).sum())
                orig = p.detach().clone()
                p.copy_(orig + eps * v)
                lp = float(loss_fn())
                p.copy_(orig - eps * v)
                lm = float(loss_fn())
                p.copy_(orig)
                numeric = (lp - lm) / (2.0 * eps)
                rel = abs(analytic - numeric) / max(abs(analytic), abs(numeric), 1e-3)
                if best is None or rel < best.rel:
                    best = Entry(name, analytic, numeric, rel)
            rep.entries.append(best)
    return rep


def elementwise_check(loss_fn, params: Dict[str, torch.Tensor], eps: float = 5e-3,
                      max_elems: int = 16, seed: int = 0) -> Report:
    """Per-element central differences on a sample of elements; for tensors whose directional sum
    is degenerate (crates/gradcheck/src/lib.rs:135-171)."""
    for p in params.values():
        p.grad = None
    loss_fn().backward()
    rng = Rng(seed)
    rep = Report()
    with torch.no_grad():
        for name, p in params.items():
            g = p.grad.reshape(-1) if p.grad is not None else torch.zeros(p.numel())
            flat = p.reshape(-1)
            n = p.numel()
            idxs = range(n) if n <= max_elems else [rng.gen_range_inclusive(0, n - 1)
                                                   for _ in range(max_elems)]
            for i in idxs:
                o = float(flat[i])
                flat[i] = o + eps
                lp = float(loss_fn())
                flat[i] = o - eps
                lm = float(loss_fn())
                flat[i] = o
                numeric = (lp - lm) / (2 * eps)
                a = float(g[i])
                rep.entries.append(Entry(f"{name}[{i}]", a, numeric,
                                         abs(a - numeric) / max(abs(a), abs(numeric), 1e-3)))
    return rep


def zero_grad_params(model, loss_fn) -> List[str]:
    """Names of parameters whose analytic gradient is identically zero."""
    for p in model.parameters():
        p.grad = None
    loss_fn().backward()
    return [n for n, p in model.named_parameters()
            if p.requires_grad and (p.grad is None or float(p.grad.abs().max()) == 0.0)]


# ------------------------------------------------------------------------------------ model gates
def _fixed_batch(vocab: int, B: int, T: int):
    """x_i = (5i+1) % V, y_i = (5i+2) % V (crates/gradcheck/src/lib.rs:290-300)."""
    i = torch.arange(B * T)
    return ((5 * i + 1) % vocab).view(B, T), ((5 * i + 2) % vocab).view(B, T)


def _model_check(model, vocab, B, T, n_dirs, eps, seed, dtype=torch.float32, only=None):
    model = model.to(dtype)
    x, y = _fixed_batch(vocab, B, T)
    params = {n: p for n, p in model.named_parameters() if p.requires_grad}
    if only is not None:
        params = {n: p for n, p in params.items() if only(n)}
    return directional_check(lambda: model.loss(x, y), params, eps, n_dirs, seed)


def check_gpt(n_dirs: int = 4, eps: float = 5e-3, seed: int = 0, d_model: int = 16,
              dtype=torch.float32) -> Report:
    from .models.config import GptConfig
    from .models.gpt2 import Gpt2
    cfg = GptConfig(vocab=23, block_size=12, n_layers=2, d_model=d_model,
                    n_heads=2, d_ff=2 * d_model)
    return _model_check(Gpt2(cfg).init_weights(1), cfg.vocab, 2, 6, n_dirs, eps, seed, dtype)


def check_qwen(n_dirs: int = 4, eps: float = 5e-3, seed: int = 0, dtype=torch.float32) -> Report:
    from .models.config import QwenConfig
    from .models.qwen3 import Qwen3
    cfg = QwenConfig.tiny()
    return _model_check(Qwen3(cfg).init_weights(1), cfg.vocab, 2, 6, n_dirs, eps, seed, dtype)


def check_qwen2(n_dirs: int = 4, eps: float = 5e-3, seed: int = 0, dtype=torch.float32) -> Report:
    """Qwen2 flavour: no QK-norm, biased q/k/v, untied head."""
    from .models.config import QwenConfig
    from .models.qwen3 import Qwen3
    cfg = QwenConfig.tiny()
    cfg.qk_norm, cfg.attn_bias, cfg.tie_embeddings = False, True, False
    m = Qwen3(cfg).init_weights(1)
    with torch.no_grad():
        for b in m.blocks:
            b.bqkv.normal_(0, 0.02)
    return _model_check(m, cfg.vocab, 2, 6, n_dirs, eps, seed, dtype)


def check_qwen3_weighted(n_dirs: int = 4, eps: float = 5e-3, seed: int = 0, dtype=torch.float32) -> Report:
    """Per-position weighted loss sum_i w_i CE_i / count with weights of both signs and a zero
    (crates/gradcheck ``check_qwen3_weighted``)."""
    from .models.config import QwenConfig
    from .models.qwen3 import Qwen3
    cfg = QwenConfig.tiny()
    model = Qwen3(cfg).init_weights(1).to(dtype)
    x, y = _fixed_batch(cfg.vocab, 2, 6)
    w = torch.tensor([1.0, -0.5, 2.0, 0.0, 0.25, 1.5] * 2, dtype=dtype).view(2, 6)
    params = {n: p for n, p in model.named_parameters() if p.requires_grad}
    return directional_check(lambda: model.loss(x, y, None, w), params, eps, n_dirs, seed)


def check_qwen_lora(n_dirs: int = 4, eps: float = 5e-3, seed: int = 0, dtype=torch.float32) -> Report:
    from .models.config import LoraCfg, QwenConfig
    from .models.lora import attach_lora
    from .models.qwen3 import Qwen3
    cfg = QwenConfig.tiny()
    cfg.lora = LoraCfg(rank=2, alpha=4.0, targets=["wq", "wv", "wo", "down"])
    m = Qwen3(cfg).init_weights(1)
    attach_lora(m, cfg.lora, seed=2)
    with torch.no_grad():   # B starts at zero; nudge it so dL/dA is not identically zero
        for n, p in m.named_parameters():
            if n.endswith("lora_b"):
                p.normal_(0, 0.02)
    return _model_check(m, cfg.vocab, 2, 6, n_dirs, eps, seed, dtype)


def check_moe(n_dirs: int = 4, eps: float = 1e-5, seed: int = 0, dtype=torch.float64,
              family: str = "toymoe") -> Report:
    """Top-k routing is piecewise: a 5e-3 step flips expert selections on a tiny model and the
    central difference then straddles a discontinuity, so this gate differentiates in fp64 with a
    small step (the selection is stable inside it)."""
    from .models.config import MoeConfig
    from .models.moe import MoeModel
    if family == "toymoe":
        cfg = MoeConfig.toy(vocab=23, block=12)
        cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.d_ff = 16, 2, 2, 8, 24
    else:
        cfg = MoeConfig(vocab=23, block_size=12, n_layers=2, d_model=16, n_heads=4, n_kv_heads=2,
                        head_dim=8, n_experts=4, top_k=2, d_ff=24, aux_coef=0.01, z_coef=1e-4,
                        tie_embeddings=True)
    return _model_check(MoeModel(cfg).init_weights(1), cfg.vocab, 2, 6, n_dirs, eps, seed, dtype)


def check_qwen_moe(n_dirs: int = 4, eps: float = 1e-5, seed: int = 0, dtype=torch.float64) -> Report:
    return check_moe(n_dirs, eps, seed, dtype, family="qwen3_moe")


GATES = {
    "gpt": check_gpt, "qwen": check_qwen, "qwen2": check_qwen2, "qwen_lora": check_qwen_lora,
    "qwen3_weighted": check_qwen3_weighted, "moe": check_moe, "qwen_moe": check_qwen_moe,
}


def run_gate(names=("gpt",), n_dirs: int = 4, atol: float = 4e-3, rtol: float = 8e-2, out=print) -> int:
    """Run the named gates; returns the number of failing tensors (process exit code of the CLI)."""
    bad = 0
    for n in names:
        rep = GATES[n](n_dirs)
        fails = rep.failures(atol, rtol)
        w = rep.worst()
        out(f"gradcheck {n}: {len(rep.entries)} tensors, {len(fails)} failures, "
            f"worst rel {w.rel:.3e} ({w.name})")
        for e in fails:
            out(f"  FAIL {e.name}: analytic {e.analytic:.6e} numeric {e.numeric:.6e}")
        bad += len(fails)
    return bad
