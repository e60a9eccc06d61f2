"""``brain federated {split,verify,merge,assemble,train-expert}`` (reference:
crates/cli/src/federated_cli.rs)."""
from __future__ import annotations

import os
import sys
from typing import List

from ..cli.args import Args
from . import shard


def run_federated(argv: List[str], device: str = "auto") -> int:
    sub = argv[0] if argv else None
    a = Args(argv[1:])
    try:
        if sub == "split":
            src, out = a.positional(), a.positional()
            if not src or not out:
                print("usage: brain federated split <base.safetensors> <out_dir>", file=sys.stderr)
                return 2
            m = shard.split(src, out)
            print(f"split {src} -> {out} ({len(m.experts)} experts: {m.experts})")
        elif sub == "verify":
            d = a.positional()
            if not d:
                print("usage: brain federated verify <dir>", file=sys.stderr)
                return 2
            m = shard.verify(d)
            print(f"OK: {d} ({len(m.files)} files, base {m.base_config_sha256[:16]})")
        elif sub == "merge":
            out, d = a.take_str("--out"), a.positional()
            if not d or not out:
                print("usage: brain federated merge <dir> --out <full.safetensors>", file=sys.stderr)
                return 2
            shard.merge_to_full(d, out)
            print(f"merged {d} -> {out}")
        elif sub == "assemble":
            out = a.take_str("--out")
            pos = []
            while True:
                p = a.positional()
                if p is None:
                    break
                pos.append(p)
            if not pos or not out:
                print("usage: brain federated assemble <base_dir> [overlay_dir ...] --out <full.safetensors>", file=sys.stderr)
                return 2
            shard.assemble(pos[0], pos[1:], out)
            print(f"assembled {pos[0]} (+{len(pos) - 1} overlays) -> {out}")
        elif sub == "train-expert":
            return _train_expert(a, device)
        else:
            print(f"usage: brain federated <split|verify|merge|assemble|train-expert> ...  (got {sub!r})", file=sys.stderr)
            return 2
    except (IOError, ValueError, KeyError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


def _train_expert(a: Args, device: str) -> int:
    """Train ONLY expert E's tensors of a toy-MoE base (router and shared weights frozen) and write
    that expert's overlay shard."""
    import torch
    from ..checkpoint import st
    from ..cli.toymoe_cli import synthetic_batch
    from ..data.rng import Rng
    from ..engine import Trainer
    from ..train import pick_device
    base, out = a.str_or("--base", ""), a.str_or("--out", "")
    expert = a.int_or("--expert", 0)
    steps, b, t = a.int_or("--steps", 200), a.int_or("--batch", 16), a.int_or("--block", 64)
    lr, seed = a.float_or("--lr", 6e-4), a.int_or("--seed", 1337)
    a.finish()
    if not base or not out:
        print("usage: brain federated train-expert --base <base.safetensors> --expert E --out <dir> "
              "[--steps N --batch B --block T --lr X --seed S]", file=sys.stderr)
        return 2
    model, _, _ = st.load_model(base)
    t = min(t, model.cfg.block_size)
    if not hasattr(model.blocks[0], "moe"):
        print("error: the base checkpoint is not a mixture-of-experts model", file=sys.stderr)
        return 1
    if not 0 <= expert < model.cfg.n_experts:
        print(f"error: --expert {expert} out of range (the base has {model.cfg.n_experts})", file=sys.stderr)
        return 1
    # experts are stored stacked ([E, …] per layer): only the stacked expert tensors are trainable,
    # and every other expert's gradient rows are zeroed before each optimiser step, so with no
    # weight decay their weights (and Adam moments) never move
    stacked = []
    for blk in model.blocks:
        stacked += [blk.moe.w_gate_up, blk.moe.w_down]
    own = {id(p) for p in stacked}
    for p in model.parameters():
        p.requires_grad_(id(p) in own)
    tr = Trainer(model, device=pick_device(device), betas=(0.9, 0.95), weight_decay=0.0, grad_clip=1.0)
    rng = Rng(seed ^ (expert * 0x9E3779B1))
    first = last = None
    for _ in range(steps):
        x, y = synthetic_batch(rng, b, t, model.cfg.vocab)
        tr.zero_grads()
        n_tgt = int((y >= 0).sum())
        last = float(tr.forward_backward(x, y, b, 1.0 / max(n_tgt, 1)))
        for blk in model.blocks:
            for p in (blk.moe.w_gate_up, blk.moe.w_down):
                g = p.main_grad
                g[:expert].zero_()
                g[expert + 1:].zero_()
        tr.optimizer_step(lr)
        first = last if first is None else first
    os.makedirs(out, exist_ok=True)
    tmp = os.path.join(out, ".worker_full.safetensors")
    st.save_model(tmp, model)
    shard.split_filtered(tmp, out, [expert])
    os.remove(tmp)
    print(f"expert {expert} overlay shard -> {out}  (loss {first:.4f} -> {last:.4f})")
    return 0
