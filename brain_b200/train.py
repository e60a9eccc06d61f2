"""Generic training driver and text generation (reference: crates/model/src/train.rs:31-93 FitOpts
and cosine schedule, :216-314 ``fit`` — resume-if-exists with the checkpoint's config winning,
gradient accumulation, periodic eval lines, wall-clock atomic checkpoints — and :320-391
``generate`` — window to the last ``block`` tokens, temperature, top-k threshold keeping ties,
softmax, inverse CDF)."""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch

from .checkpoint import st
from .data import binio
from .data.loader import BatchConfig, TokenDataset
from .data.rng import Rng
from .engine import Trainer
from .optim.lr import cosine_lr


@dataclass
class FitOpts:
    steps: int = 2000
    batch_size: int = 32
    block_size: int = 64
    lr: float = 3e-4
    min_lr: float = 3e-5
    warmup: int = 100
    decay_iters: int = 2000
    weight_decay: float = 0.1
    grad_clip: float = 1.0
    grad_accum: int = 1
    eval_interval: int = 250
    eval_batches: int = 20
    seed: int = 1337
    checkpoint_secs: int = 600
    mask_before: Optional[object] = None      # token id, or a character looked up in the vocabulary
    mask_per_line: bool = False
    align_to_lines: bool = False
    betas: Tuple[float, float] = (0.9, 0.999)
    device: str = "auto"
    weighted: bool = False                    # per-position loss weights from train.weight.bin


def load_dataset(dirpath: str, opts: FitOpts):
    """(train, val, vocab, itos, BatchConfig) from a ``data.binio`` directory."""
    meta = binio.read_meta(dirpath)
    train = binio.read_tokens(dirpath, "train")
    val = binio.read_tokens(dirpath, "val")
    itos = meta.get("itos")
    vocab = int(meta.get("vocab_size") or (int(max(train.max(), val.max())) + 1))
    newline = itos.index("\n") if itos and "\n" in itos else None
    tr = TokenDataset(train, binio.read_mask(dirpath, "train"), binio.read_weights(dirpath, "train"))
    va = TokenDataset(val)
    if opts.align_to_lines and newline is not None:
        tr.align_to_lines(newline, opts.block_size)
        va.align_to_lines(newline, opts.block_size)
    mask_tok = opts.mask_before
    if isinstance(mask_tok, str):
        if not itos or mask_tok not in itos:
            raise ValueError(f"--mask {mask_tok!r}: character not in the dataset vocabulary")
        mask_tok = itos.index(mask_tok)
    bc = BatchConfig(opts.batch_size, opts.block_size, mask_tok, opts.mask_per_line, newline)
    return tr, va, vocab, itos, bc


def pick_device(name: str = "auto") -> torch.device:
    """The device single-device work runs on for a ``--device`` selection (see utils.devices for
    the grammar); an indexed CPU selection also pins the affinity and sizes the thread pool."""
    from .utils.devices import apply_selection, parse_selection
    if name in ("cuda",) or name.startswith("cuda:"):
        return torch.device(name if ":" in name else "cuda:0")
    return apply_selection(parse_selection(name)).first()


def fit(data_dir: str, build_model: Callable[[int, int], torch.nn.Module], opts: FitOpts,
        out: Optional[str] = None, log: Callable[[str], None] = print, dp=None, model=None,
        save: Optional[Callable[[str, torch.nn.Module], None]] = None):
    """Train ``build_model(vocab, block)`` on the dataset directory; returns (initial, final) loss.
    ``model`` supplies a prebuilt model (adapter finetunes: frozen base + trainable adapters) and
    ``save`` replaces the whole-model checkpoint writer; both bypass resume-from-``out``."""
    tr_ds, va_ds, vocab, itos, bc = load_dataset(data_dir, opts)
    save = save or st.save_model
    if out:
        os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
    resume = model is None and bool(out) and os.path.exists(out)
    if model is not None:
        pass
    elif resume:
        log(f"resuming from existing checkpoint {out}")
        model, cfg_json, _ = st.load_model(out)
        if int(cfg_json.get("block_size", opts.block_size)) != opts.block_size:
            raise ValueError(f"checkpoint block_size {cfg_json.get('block_size')} != --block "
                             f"{opts.block_size} — resume with the same --block")
        if int(cfg_json.get("vocab_size", vocab)) != vocab:
            raise ValueError("checkpoint vocab != dataset vocab — wrong dataset for this checkpoint")
    else:
        model = build_model(vocab, opts.block_size)
        model.init_weights(opts.seed)
    if itos is not None and hasattr(model.cfg, "itos"):
        model.cfg.itos = list(itos)
    dev = pick_device(opts.device)
    trainer = Trainer(model, device=dev, betas=opts.betas, weight_decay=opts.weight_decay,
                      grad_clip=opts.grad_clip if opts.grad_clip > 0 else None, dp=dp)
    rng = Rng(opts.seed ^ 0xA5A55A5A)
    pin = dev.type == "cuda"

    def sample_loss(ds: TokenDataset, r: Rng, batches: int) -> float:
        tot = 0.0
        with torch.no_grad():
            for _ in range(max(batches, 1)):
                x, y = ds.get_batch(bc, r, pin=pin)
                tot += float(model.loss(x.to(dev), y.to(dev)))
        return tot / max(batches, 1)

    def clone_rng(r: Rng) -> Rng:
        c = Rng(0)
        c.state = r.state
        return c

    initial = sample_loss(tr_ds, clone_rng(rng), 5)
    last_train = initial
    last_save = time.time()
    accum = max(opts.grad_accum, 1)
    from .utils import shutdown, trace
    for step in range(opts.steps):
        if shutdown.requested():
            log(f"step {step:>6}  shutdown requested: saving and stopping")
            break
        trace.event("train", 4, "step", step=step)
        lr = cosine_lr(step, opts.lr, opts.min_lr, opts.warmup, opts.decay_iters)
        trainer.zero_grads()
        step_loss = 0.0
        batches = [tr_ds.get_batch(bc, rng, weighted=opts.weighted, pin=pin) for _ in range(accum)]
        count = sum(int((b[1] >= 0).sum()) for b in batches)
        world = dp.world if dp is not None else 1
        for b in batches:
            x, y = b[0], b[1]
            loss = trainer.forward_backward(x, y, x.shape[0], 1.0 / max(count * world, 1),
                                            b[2] if opts.weighted else None)
            step_loss += float(loss) * world
        trainer.optimizer_step(lr)
        last_train = step_loss
        if opts.eval_interval > 0 and (step + 1) % opts.eval_interval == 0:
            ev = sample_loss(va_ds, clone_rng(rng), opts.eval_batches)
            log(f"step {step + 1:>6}  lr {lr:.2e}  train {last_train:.4f}  eval {ev:.4f}")
        if out and opts.checkpoint_secs > 0 and time.time() - last_save >= opts.checkpoint_secs:
            t0 = time.time()
            save(out, model)
            log(f"step {step + 1:>6}  saved checkpoint -> {out} ({time.time() - t0:.1f} s)")
            last_save = time.time()
    if out:
        t0 = time.time()
        save(out, model)
        log(f"saved checkpoint -> {out} ({time.time() - t0:.1f} s)")
    return initial, last_train


@torch.no_grad()
def generate(model, tokens: List[int], max_new: int, temp: float = 0.8, top_k: int = 40,
             seed: int = 1234, block: Optional[int] = None, eos: Optional[int] = None) -> List[int]:
    """Autoregressive sampling without a KV cache (small models / CPU): the context is the last
    ``block`` tokens; ``temp <= 0`` is greedy; the top-k threshold keeps ties."""
    dev = next(model.parameters()).device
    block = block or model.cfg.block_size
    rng = Rng(seed)
    out = list(tokens)
    for _ in range(max_new):
        ctx = torch.tensor([out[-block:]], device=dev, dtype=torch.int32)
        logits = model(ctx)[0, -1].float()
        if temp <= 0:
            nxt = int(logits.argmax())
        else:
            logits = logits / temp
            if 0 < top_k < logits.numel():
                thr = torch.topk(logits, top_k).values[-1]
                logits = torch.where(logits < thr, torch.full_like(logits, float("-inf")), logits)
            probs = torch.softmax(logits, dim=-1).cpu()
            r = rng.next_f32()
            cdf = torch.cumsum(probs, 0)
            nxt = int(torch.searchsorted(cdf, torch.tensor(r)).clamp_max(probs.numel() - 1))
        if eos is not None and nxt == eos:
            break
        out.append(nxt)
    return out[len(tokens):]


@torch.no_grad()
def evaluate(model, data_dir: str, batches: int = 20, batch: int = 8, block: Optional[int] = None,
             seed: int = 0) -> float:
    """Mean validation loss over ``batches`` random windows."""
    dev = next(model.parameters()).device
    block = block or model.cfg.block_size
    opts = FitOpts(batch_size=batch, block_size=block)
    _, va, _, _, bc = load_dataset(data_dir, opts)
    rng = Rng(seed)
    tot = 0.0
    for _ in range(batches):
        x, y = va.get_batch(bc, rng)
        tot += float(model.loss(x.to(dev), y.to(dev)))
    return tot / batches
