"""``brain toymoe <train|infer|eval>`` (reference: crates/cli/src/resolve.rs:70-77 dispatch to
crates/toymoe/src/train.rs ``run_train``/``run_eval``/``run_generate``: a synthetic
next-token task — token t+1 = (a·t + b) mod V per sequence family — so the sparse model can be
trained and scored without a dataset on disk).  ``--ep N`` is additive."""
from __future__ import annotations

import sys
import time
from typing import List

from .args import Args, canon_verb


def run_toymoe(argv: List[str], device: str = "auto") -> int:
    verb = canon_verb(argv[0]) if argv else None
    if verb == "train":
        return _train(argv[1:], device) or 0
    if verb == "eval":
        return _eval(argv[1:], device) or 0
    if verb == "infer":
        return _infer(argv[1:], device) or 0
    print(f"usage: brain toymoe <train|eval|infer> ...  (got {verb!r})", file=sys.stderr)
    return 2


def synthetic_batch(rng, batch: int, block: int, vocab: int):
    """Sequences x[t+1] = (m·x[t] + c) mod vocab with (m, c) drawn per sequence from a small family,
    which gives the router distinct token populations to specialise on."""
    import numpy as np
    import torch
    fam = [(1, 1), (1, 3), (3, 1), (5, 2), (1, vocab - 1), (7, 5), (3, 4), (9, 7)]
    x = np.empty((batch, block + 1), dtype=np.int64)
    for b in range(batch):
        m, c = fam[rng.gen_range_inclusive(0, len(fam) - 1)]
        v = rng.gen_range_inclusive(0, vocab - 1)
        for t in range(block + 1):
            x[b, t] = v
            v = (m * v + c) % vocab
    t = torch.from_numpy(x)
    return t[:, :-1].to(torch.int32).contiguous(), t[:, 1:].contiguous()


def _train(args, device):
    import torch
    from ..checkpoint import st
    from ..data.rng import Rng
    from ..engine import Trainer
    from ..models.config import MoeConfig
    from ..models.moe import MoeModel
    from ..optim.lr import cosine_lr
    from ..train import pick_device
    a = Args(args)
    steps = a.int_or("--steps", 300)
    batch = a.int_or("--batch-size", 16)
    block = a.int_or("--block-size", 32)
    lr = a.float_or("--lr", 3e-3)
    out = a.str_or("--out", "out/toymoe.safetensors")
    seed = a.int_or("--seed", 1337)
    experts = a.int_or("--experts", 4)
    top_k = a.int_or("--top-k", 2)
    a.finish()
    cfg = MoeConfig.toy(block=block)
    cfg.n_experts, cfg.top_k = experts, top_k
    model = MoeModel(cfg)
    model.init_weights(seed)
    dev = pick_device(device)
    tr = Trainer(model, device=dev, betas=(0.9, 0.95), weight_decay=0.1, grad_clip=1.0)
    rng = Rng(seed)
    first = last = None
    t0 = time.time()
    for step in range(steps):
        x, y = synthetic_batch(rng, batch, block, cfg.vocab)
        loss = float(tr.train_step(x, y, cosine_lr(step, lr, lr * 0.1, min(20, steps), steps)))
        first = loss if first is None else first
        last = loss
        if (step + 1) % max(steps // 10, 1) == 0:
            print(f"step {step + 1:>6}  loss {loss:.4f}")
    import os
    os.makedirs(os.path.dirname(out) or ".", exist_ok=True)
    st.save_model(out, model)
    print(f"trained: loss {first:.4f} -> {last:.4f} in {time.time() - t0:.1f}s; saved {out}")


def _eval(args, device):
    import torch
    from ..checkpoint import st
    from ..data.rng import Rng
    from ..train import pick_device
    a = Args(args)
    weights = a.str_or("--weights", "")
    samples = a.int_or("--samples", 64)
    a.finish()
    if not weights:
        print("usage: brain toymoe eval --weights F [--samples N]", file=sys.stderr)
        return 2
    model, _, _ = st.load_model(weights, device=pick_device(device))
    model.eval()
    dev = next(model.parameters()).device
    rng = Rng(4242)
    x, y = synthetic_batch(rng, samples, model.cfg.block_size, model.cfg.vocab)
    with torch.no_grad():
        logits = model(x.to(dev))
        acc = float((logits.argmax(-1).cpu() == y)[:, 1:].float().mean())
        loss = float(model.loss(x.to(dev), y.to(dev)))
    print(f"eval: loss {loss:.4f}  next-token accuracy {100 * acc:.1f}%  ({samples} sequences)")


def _infer(args, device):
    from ..checkpoint import st
    from ..train import generate, pick_device
    a = Args(args)
    weights = a.str_or("--weights", "")
    prompt = a.str_or("--prompt", "1,2,3,4")
    max_new = a.int_or("--max-new", 16)
    temp = a.float_or("--temperature", 0.0)
    top_k = a.int_or("--top-k", 0)
    a.finish()
    if not weights:
        print("usage: brain toymoe infer --weights F [--prompt 1,2,3,4 --max-new N --temperature X --top-k K]",
              file=sys.stderr)
        return 2
    model, _, _ = st.load_model(weights, device=pick_device(device))
    model.eval()
    ids = [int(t) for t in prompt.split(",") if t.strip()]
    out = generate(model, ids, max_new, temp, top_k)
    print(",".join(str(t) for t in ids + out))
