"""Synthetic dataset generators and ``prepare`` (``brain data gen <name>``): calculator
(``EXPR=RESULT`` lines), reverser (``s=reversed(s)``), wordcalc (spelled-out arithmetic),
timeseries (noisy seasonal signal, quantised), shakespeare_char / gpt (from ``input.txt``).
Lines are at most 64 characters including the newline; a fixed seed gives a fixed corpus.  Written
in the dataset format of ``data.binio`` with a 90/10 train/val split.
Reference: crates/data/src/{gen_calculator,gen_reverser,gen_wordcalc,gen_timeseries,prepare}.rs."""
from __future__ import annotations

import math
from pathlib import Path
from typing import List

import numpy as np

from . import binio
from .rng import Rng

MAX_CHARS_PER_LINE = 64
OPS = "+-*/"
NAMES = ["calculator", "reverser", "wordcalc", "timeseries", "shakespeare_char", "gpt"]


def _fmt(num: float) -> str:
    if abs(num - round(num)) < 1e-9:
        return str(int(round(num)))
    return f"{num:.10f}".rstrip("0").rstrip(".")


def _number(lo: float, hi: float, rng: Rng) -> float:
    r = rng.next_f64()
    if r < 0.4:
        return float(rng.gen_range_inclusive(int(max(1.0, lo)), int(hi)))
    places = 1 if r < 0.6 else 2 if r < 0.8 else 3 if r < 0.9 else 4
    return round(rng.uniform(lo, hi), places)


def _calc_line(rng: Rng) -> str:
    for _ in range(50):
        n_ops = 1 if rng.next_f64() < 0.7 else 2
        nums = [_number(1, 100, rng) for _ in range(n_ops + 1)]
        ops = [rng.choice(OPS) for _ in range(n_ops)]
        expr = _fmt(nums[0])
        for o, n in zip(ops, nums[1:]):
            expr += o + _fmt(n)
        try:
            val = eval(expr, {"__builtins__": {}})  # digits and + - * / only
        except ZeroDivisionError:
            continue
        line = f"{expr}={_fmt(round(val, 4))}\n"
        if len(line) <= MAX_CHARS_PER_LINE:
            return line
    return "1+1=2\n"


def gen_calculator(n: int, rng: Rng) -> str:
    return "".join(_calc_line(rng) for _ in range(n))


_ALNUM = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789"


def _rev_line(rng: Rng) -> str:
    for _ in range(20):
        kind = rng.next_f64()
        n = rng.gen_range_inclusive(1, 24)
        if kind < 0.4:
            s = "".join(rng.choice(_ALNUM[:26]) for _ in range(n))
        elif kind < 0.7:
            s = "".join(rng.choice(_ALNUM) for _ in range(n))
        else:
            s = " ".join("".join(rng.choice(_ALNUM[:26]) for _ in range(rng.gen_range_inclusive(1, 6)))
                         for _ in range(rng.gen_range_inclusive(1, 4)))
        s = " ".join(s.split())
        if not s:
            continue
        line = f"{s}={s[::-1]}\n"
        if len(line) <= MAX_CHARS_PER_LINE:
            return line
    return "abc=cba\n"


def gen_reverser(n: int, rng: Rng) -> str:
    return "".join(_rev_line(rng) for _ in range(n))


_ONES = ["zero", "one", "two", "three", "four", "five", "six", "seven", "eight", "nine", "ten", "eleven",
         "twelve", "thirteen", "fourteen", "fifteen", "sixteen", "seventeen", "eighteen", "nineteen"]
_TENS = ["", "", "twenty", "thirty", "forty", "fifty", "sixty", "seventy", "eighty", "ninety"]


def number_words(n: int) -> str:
    if n < 0:
        return "minus " + number_words(-n)
    if n < 20:
        return _ONES[n]
    if n < 100:
        return _TENS[n // 10] + ("" if n % 10 == 0 else " " + _ONES[n % 10])
    if n < 1000:
        return _ONES[n // 100] + " hundred" + ("" if n % 100 == 0 else " " + number_words(n % 100))
    return number_words(n // 1000) + " thousand" + ("" if n % 1000 == 0 else " " + number_words(n % 1000))


def _wordcalc_line(rng: Rng) -> str:
    for _ in range(20):
        a, b = rng.gen_range_inclusive(0, 99), rng.gen_range_inclusive(0, 99)
        op = rng.choice(["plus", "minus", "times"])
        val = a + b if op == "plus" else a - b if op == "minus" else a * b
        line = f"{number_words(a)} {op} {number_words(b)}={number_words(val)}\n"
        if len(line) <= MAX_CHARS_PER_LINE:
            return line
    return "one plus one=two\n"


def gen_wordcalc(n: int, rng: Rng) -> str:
    return "".join(_wordcalc_line(rng) for _ in range(n))


def gen_timeseries(n_steps: int, seed: int) -> np.ndarray:
    """Trend + two seasonalities + gaussian noise (float32)."""
    rng = Rng(seed)
    t = np.arange(n_steps, dtype=np.float64)
    noise = np.array([rng.next_gaussian() for _ in range(n_steps)])
    y = 0.002 * t + np.sin(2 * math.pi * t / 24.0) + 0.5 * np.sin(2 * math.pi * t / 168.0) + 0.1 * noise
    return y.astype(np.float32)


def write_char_dataset(text: str, dirpath) -> None:
    chars = sorted(set(text))
    stoi = {ch: i for i, ch in enumerate(chars)}
    ids = np.fromiter((stoi[ch] for ch in text), dtype=np.uint32, count=len(text))
    cut = int(len(ids) * 0.9)
    binio.write_dataset(dirpath, ids[:cut], ids[cut:], len(chars), itos=chars)


def write_bpe_dataset(text: str, dirpath, tokenizer=None) -> None:
    from .tokenizer import BpeTokenizer
    tok = tokenizer or BpeTokenizer.byte_level()
    ids = np.asarray(tok.encode(text), dtype=np.uint32)
    cut = int(len(ids) * 0.9)
    binio.write_dataset(dirpath, ids[:cut], ids[cut:], tok.vocab_size)


def prepare(name: str, dirpath, n_examples: int = 10000, seed: int = 0) -> None:
    d = Path(dirpath)
    d.mkdir(parents=True, exist_ok=True)
    if name == "calculator":
        write_char_dataset(gen_calculator(n_examples, Rng(seed)), d)
    elif name == "reverser":
        write_char_dataset(gen_reverser(n_examples, Rng(seed)), d)
    elif name == "wordcalc":
        write_char_dataset(gen_wordcalc(n_examples, Rng(seed)), d)
    elif name == "timeseries":
        y = gen_timeseries(max(n_examples, 1), seed)
        lo, hi = float(y.min()), float(y.max())
        q = np.clip(((y - lo) / max(hi - lo, 1e-9) * 255).round(), 0, 255).astype(np.uint32)
        cut = int(len(q) * 0.9)
        binio.write_dataset(d, q[:cut], q[cut:], 256)
        y.tofile(d / "series.f32")
    elif name in ("shakespeare_char", "gpt"):
        p = d / "input.txt"
        if not p.exists():
            raise FileNotFoundError(f"{p}: missing source text (place the corpus there first; nothing is downloaded)")
        text = p.read_text(encoding="utf-8")
        (write_char_dataset if name == "shakespeare_char" else write_bpe_dataset)(text, d)
    else:
        raise ValueError(f"unknown dataset {name!r}; have {NAMES}")
