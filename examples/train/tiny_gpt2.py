#!/usr/bin/env python3
"""Train a tiny character-level GPT-2 through the public trainer, save it, load it back, sample.

    python examples/train/tiny_gpt2.py --steps 60            # CPU in under a minute; a GPU when present
The same flow as `brain prepare` + `brain gpt2 train` + `brain gpt2 infer`, as library calls."""
import argparse
import os
import sys
import tempfile

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from brain_b200 import train as T  # noqa: E402
from brain_b200.checkpoint import st  # noqa: E402
from brain_b200.data import binio  # noqa: E402
from brain_b200.data.datasets import write_char_dataset  # noqa: E402
from brain_b200.models.config import GptConfig  # noqa: E402
from brain_b200.models.gpt2 import Gpt2  # noqa: E402

TEXT = ("the quick brown fox jumps over the lazy dog. " * 40 +
        "pack my box with five dozen liquor jugs. " * 40)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--device", default="auto")
    a = ap.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        data = os.path.join(tmp, "data")
        write_char_dataset(TEXT, data)
        ckpt = os.path.join(tmp, "tiny.safetensors")
        opts = T.FitOpts(steps=a.steps, batch_size=16, block_size=32, lr=3e-3, min_lr=3e-4, warmup=5,
                         decay_iters=a.steps, eval_interval=max(a.steps // 3, 1), eval_batches=4, device=a.device)
        build = lambda vocab, block: Gpt2(GptConfig(vocab=vocab, block_size=block, n_layers=2, d_model=64,
                                                    n_heads=4, d_ff=256))
        first, last = T.fit(data, build, opts, out=ckpt)
        print(f"loss {first:.3f} -> {last:.3f}")
        assert last < first
        model, cfg, card = st.load_model(ckpt, device=str(T.pick_device(a.device)))
        itos = binio.read_meta(data)["itos"]
        stoi = {ch: i for i, ch in enumerate(itos)}
        prompt = [stoi[ch] for ch in "the quick "]
        with torch.no_grad():
            out = T.generate(model.eval(), prompt, 40, temp=0.0)
        print("sample:", "the quick " + "".join(itos[t] for t in out))
        print(f"checkpoint: {os.path.getsize(ckpt)} bytes, card id {card.id if card else None}, "
              f"config {cfg['n_layers']} layers x d{cfg['d_model']}")


if __name__ == "__main__":
    main()
