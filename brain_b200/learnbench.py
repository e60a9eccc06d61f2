"""A small "does it learn?" battery (reference: crates/bench — mqar / parity / mod_add / dyck task
families trained to a pass bar through a ``DecoderLm`` seam).  Three synthetic sequence tasks are
generated on the fly; a tiny decoder is trained on each for a fixed number of steps and scored by
exact-match accuracy of the answer tokens on held-out samples:

    copy      a b c d | a b c d          (attention must route every position)
    mod_add   a + b = (a + b) mod p      (a lookup the MLP has to memorise and generalise)
    parity    b1 p1 b2 p2 …              (a running state carried along the sequence: p_i = p_{i-1} xor b_i,
                                          every p_i scored)

``brain bench learn [task…] [--arch qwen|gpt --steps N --seed S]``; exit code 0 when every task
reaches its bar."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Tuple

import torch

from .data.rng import Rng


@dataclass
class Task:
    name: str
    vocab: int
    seq: int
    answer: List[int]      # positions of the answer tokens in the sequence
    bar: float             # exact-match accuracy required (all answer tokens of a sample right)
    make: Callable[[Rng], List[int]]


def _copy_task(n: int = 6, sym: int = 12) -> Task:
    sep = sym

    def make(r: Rng) -> List[int]:
        xs = [r.next_u64() % sym for _ in range(n)]
        return xs + [sep] + xs
    return Task("copy", sym + 1, 2 * n + 1, list(range(n + 1, 2 * n + 1)), 0.95, make)


def _mod_add_task(p: int = 11) -> Task:
    plus, eq = p, p + 1

    def make(r: Rng) -> List[int]:
        a, b = r.next_u64() % p, r.next_u64() % p
        return [a, plus, b, eq, (a + b) % p]
    return Task("mod_add", p + 2, 5, [4], 0.95, make)


def _parity_task(n: int = 8) -> Task:
    # bits are tokens 0/1, running parities tokens 2/3
    def make(r: Rng) -> List[int]:
        out, p = [], 0
        for _ in range(n):
            b = r.next_u64() % 2
            p ^= b
            out += [b, 2 + p]
        return out
    return Task("parity", 4, 2 * n, list(range(1, 2 * n, 2)), 0.9, make)


TASKS: Dict[str, Callable[[], Task]] = {"copy": _copy_task, "mod_add": _mod_add_task, "parity": _parity_task}


def _model(arch: str, vocab: int, seq: int, seed: int):
    if arch == "gpt":
        from .models.config import GptConfig
        from .models.gpt2 import Gpt2
        return Gpt2(GptConfig(vocab=vocab, block_size=seq, n_layers=2, d_model=64, n_heads=4, d_ff=128)).init_weights(seed)
    from .models.config import QwenConfig
    from .models.qwen3 import Qwen3
    return Qwen3(QwenConfig(vocab=vocab, block_size=seq, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16,
                            d_ff=128)).init_weights(seed)


def _batch(task: Task, rng: Rng, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
    rows = [task.make(rng) for _ in range(n)]
    full = torch.tensor(rows, dtype=torch.int64)
    x = full[:, :-1].to(torch.int32)
    y = torch.full_like(full[:, 1:], -1)
    idx = torch.tensor([a - 1 for a in task.answer])     # target position t predicts token t + 1
    y[:, idx] = full[:, 1:][:, idx]                      # only the answer positions are scored
    return x, y


def run_task(task: Task, arch: str = "qwen", steps: int = 400, batch: int = 64, lr: float = 3e-3, seed: int = 0,
             device: str = "cpu", log: Callable[[str], None] = lambda s: None) -> Dict:
    from .engine import Trainer
    from .optim.lr import cosine_lr
    model = _model(arch, task.vocab, task.seq, seed + 1)
    tr = Trainer(model, device=device, weight_decay=0.0, grad_clip=1.0)
    rng = Rng(seed ^ 0x5EED)
    t0 = time.time()
    loss = float("nan")
    for step in range(steps):
        x, y = _batch(task, rng, batch)
        loss = float(tr.train_step(x, y, cosine_lr(step, lr, lr * 0.1, 20, steps)))
        if (step + 1) % 100 == 0:
            log(f"  {task.name}: step {step + 1} loss {loss:.4f}")
    # held-out exact match of the answer tokens (fresh samples from a different stream)
    ev = Rng(seed ^ 0xE7A1)
    x, y = _batch(task, ev, 256)
    dev = next(model.parameters()).device
    with torch.no_grad():
        pred = model(x.to(dev)).argmax(-1).cpu()
    ans = torch.tensor([a - 1 for a in task.answer])
    acc = float((pred[:, ans] == y[:, ans]).all(dim=1).float().mean())
    return {"task": task.name, "arch": arch, "steps": steps, "final_loss": loss, "accuracy": acc, "bar": task.bar,
            "passed": acc >= task.bar, "seconds": time.time() - t0}


def run_battery(names: List[str], arch: str = "qwen", steps: int = 400, seed: int = 0, device: str = "cpu",
                log: Callable[[str], None] = print) -> List[Dict]:
    out = []
    for n in names or list(TASKS):
        if n not in TASKS:
            raise ValueError(f"unknown task {n!r}; have: {' '.join(TASKS)}")
        r = run_task(TASKS[n](), arch, steps, seed=seed, device=device, log=log)
        log(f"{r['task']:<8} {arch:<5} accuracy {r['accuracy']:.3f} (bar {r['bar']:.2f})  loss {r['final_loss']:.4f}  "
            f"{r['seconds']:.1f}s  {'PASS' if r['passed'] else 'FAIL'}")
        out.append(r)
    return out
