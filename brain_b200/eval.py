"""Evaluation helpers (reference: crates/model/src/eval.rs and the ``brain gpt eval`` verb,
crates/cli/src/gpt_cli.rs:34-58): validation perplexity over random windows, and exact-match
accuracy on held-out ``prompt=answer`` lines for the synthetic task datasets."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .checkpoint import st
from .data import binio
from .data.rng import Rng
from .data.tokenizer import CharTokenizer
from .train import evaluate, generate


def val_perplexity(weights: str, data_dir: str, batches: int = 20, seed: int = 99, device="cpu",
                   batch: int = 8) -> float:
    model, _, _ = st.load_model(weights, device=device)
    model.eval()
    return math.exp(evaluate(model, data_dir, batches=batches, batch=batch, seed=seed))


@torch.no_grad()
def exact_match(weights: str, data_dir: str, samples: int = 200, seed: int = 99, device="cpu",
                marker: str = "=") -> Tuple[float, int]:
    """Greedy-complete up to ``samples`` validation lines after ``marker``; (accuracy, n)."""
    model, cfg, _ = st.load_model(weights, device=device)
    model.eval()
    meta = binio.read_meta(data_dir)
    itos = meta.get("itos") or (cfg or {}).get("itos")
    if not itos or marker not in itos or "\n" not in itos:
        return 0.0, 0
    tok = CharTokenizer(itos)
    text = tok.decode(binio.read_tokens(data_dir, "val").tolist())
    lines = [l for l in text.split("\n") if marker in l and len(l) + 1 < model.cfg.block_size]
    if not lines:
        return 0.0, 0
    rng = Rng(seed)
    picks = [rng.choice(lines) for _ in range(min(samples, len(lines)))]
    nl = tok.stoi["\n"]
    good = 0
    for line in picks:
        prompt, answer = line.split(marker, 1)
        ids = tok.encode("\n" + prompt + marker)
        out = generate(model, ids, len(answer) + 2, temp=0.0, eos=nl)
        good += int(tok.decode(out) == answer)
    return good / len(picks), len(picks)
