"""``brain gpt2 <train|infer|eval>`` (reference: crates/cli/src/gpt_cli.rs:24-142)."""
from __future__ import annotations

import os
import sys
from typing import List

from .args import Args, canon_verb


def run_gpt(argv: List[str], device: str = "auto") -> int:
    verb = canon_verb(argv[0]) if argv else None
    if verb == "train":
        return _train(argv[1:], device)
    if verb == "infer":
        return _infer(argv[1:], device)
    if verb == "eval":
        return _eval(argv[1:], device)
    print(f"usage: brain gpt <train|infer|eval> ...  (got {verb!r})", file=sys.stderr)
    return 2


def _train(args: List[str], device: str) -> int:
    from ..models.config import GptConfig
    from ..models.gpt2 import Gpt2
    from ..train import FitOpts, fit
    a = Args(args)
    d = a.positional()
    if d is None:
        print("usage: brain gpt train <data_dir> [flags]", file=sys.stderr)
        return 2
    o = FitOpts(device=device)
    out = a.take_str("--out")
    o.steps = a.int_or("--steps", o.steps)
    o.batch_size = a.int_or("--batch", o.batch_size)
    o.block_size = a.int_or("--block", o.block_size)
    o.lr = a.float_or("--lr", o.lr)
    o.warmup = a.int_or("--warmup", o.warmup)
    o.eval_interval = a.int_or("--eval-interval", o.eval_interval)
    o.grad_accum = a.int_or("--grad-accum", o.grad_accum)
    layers = a.int_or("--layers", 4)
    d_model = a.int_or("--d-model", 128)
    heads = a.int_or("--heads", 4)
    o.seed = a.int_or("--seed", o.seed)
    m = a.char_opt("--mask")
    if m is not None:
        o.mask_before, o.mask_per_line = m, True
    o.align_to_lines = a.take_flag("--align")
    a.finish()
    o.decay_iters = o.steps
    print(f"training gpt on {d}: steps={o.steps} batch={o.batch_size} block={o.block_size} "
          f"layers={layers} d_model={d_model} heads={heads}")

    def build(vocab, block):
        return Gpt2(GptConfig(vocab=vocab, block_size=block, n_layers=layers, d_model=d_model,
                              n_heads=heads, d_ff=4 * d_model))
    try:
        l0, l1 = fit(d, build, o, out)
    except Exception as e:  # noqa: BLE001 - the CLI reports and exits non-zero
        print(f"error: {e}", file=sys.stderr)
        return 1
    print(f"done: train loss {l0:.4f} -> {l1:.4f}")
    return 0


def _eval(args: List[str], device: str) -> int:
    from .. import eval as ev
    from ..train import pick_device
    a = Args(args)
    weights = a.str_or("--weights", "")
    data_dir = a.str_or("--data", "")
    batches = a.int_or("--batches", 20)
    samples = a.int_or("--samples", 200)
    seed = a.int_or("--seed", 99)
    a.finish()
    if not weights or not data_dir:
        print("usage: brain gpt eval --weights F --data <dir> [--batches N --samples M]", file=sys.stderr)
        return 2
    dev = pick_device(device)
    try:
        print(f"val_perplexity {ev.val_perplexity(weights, data_dir, batches, seed, dev):.4f}")
    except Exception as e:  # noqa: BLE001
        print(f"perplexity error: {e}", file=sys.stderr)
    if os.path.exists(os.path.join(data_dir, "meta.json")):
        try:
            acc, n = ev.exact_match(weights, data_dir, samples, seed, dev)
            if n > 0:
                print(f"exact_match {acc:.4f} ({round(acc * n)}/{n} held-out)")
        except Exception as e:  # noqa: BLE001
            print(f"exact-match error: {e}", file=sys.stderr)
    return 0


def _infer(args: List[str], device: str) -> int:
    from ..checkpoint import st
    from ..data import binio
    from ..data.tokenizer import CharTokenizer
    from ..train import generate, pick_device
    a = Args(args)
    weights = a.str_or("--weights", "")
    data_dir = a.str_or("--data", "")
    prompt = a.str_or("--prompt", "")
    max_new = a.int_or("--max-new", 200)
    temp = a.float_or("--temp", 0.8)
    top_k = a.int_or("--top-k", 40)
    seed = a.int_or("--seed", 1234)
    a.finish()
    if not weights:
        print("usage: brain gpt infer --weights F [--data <dir>] [--prompt ... --max-new N --temp X --top-k K]",
              file=sys.stderr)
        return 2
    model, cfg, _ = st.load_model(weights, device=pick_device(device))
    itos = (cfg or {}).get("itos")
    if not itos:
        if not data_dir:
            print("this checkpoint has no embedded vocab (a BPE model, or trained without one); "
                  "pass --data <dir> with its meta.json", file=sys.stderr)
            return 1
        itos = binio.read_meta(data_dir).get("itos")
        if not itos:
            print(f"gen needs a char vocab: none embedded and no meta.json at {data_dir}/meta.json",
                  file=sys.stderr)
            return 1
    tok = CharTokenizer(itos)
    text = prompt or "\n"
    model.eval()
    out = generate(model, tok.encode(text), max_new, temp, top_k, seed)
    print(text + tok.decode(out))
    return 0
