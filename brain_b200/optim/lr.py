"""Learning-rate schedule: linear warm-up then cosine decay to ``min_lr`` over ``decay_iters``
(reference: crates/model/src/train.rs:83-93)."""
import math


def cosine_lr(it: int, lr: float, min_lr: float, warmup: int, decay_iters: int) -> float:
    if it < warmup:
        return lr * (it + 1) / max(warmup, 1)
    if it >= decay_iters:
        return min_lr
    ratio = (it - warmup) / max(decay_iters - warmup, 1)
    coeff = 0.5 * (1.0 + math.cos(math.pi * ratio))
    return min_lr + coeff * (lr - min_lr)
