"""Dataset files, byte-compatible with the reference (crates/data/src/binio.rs:1-17):
``train.bin``/``val.bin`` little-endian u16 tokens (or ``*.u32.bin``), ``meta.json``
``{vocab_size, itos, token_width}``, optional ``train.mask.bin`` (u8) and ``train.weight.bin`` (f32)."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np


def write_tokens(path, tokens, width: int = 16) -> None:
    arr = np.asarray(tokens)
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    if width == 16:
        if arr.size and int(arr.max()) > 0xFFFF:
            raise ValueError("token id does not fit u16; use the .u32.bin form")
        arr.astype("<u2").tofile(path)
    else:
        arr.astype("<u4").tofile(path)


def read_tokens(dir_or_file, split: str = "train") -> np.ndarray:
    p = Path(dir_or_file)
    if p.is_dir():
        p32 = p / f"{split}.u32.bin"
        if p32.exists():
            return np.fromfile(p32, dtype="<u4").astype(np.uint32)
        return np.fromfile(p / f"{split}.bin", dtype="<u2").astype(np.uint32)
    if p.name.endswith(".u32.bin"):
        return np.fromfile(p, dtype="<u4").astype(np.uint32)
    return np.fromfile(p, dtype="<u2").astype(np.uint32)


def write_meta(dirpath, vocab_size: int, itos=None, token_width: int = 16) -> None:
    meta = {"vocab_size": int(vocab_size), "token_width": int(token_width)}
    if itos is not None:
        meta["itos"] = list(itos)
    Path(dirpath).mkdir(parents=True, exist_ok=True)
    (Path(dirpath) / "meta.json").write_text(json.dumps(meta))


def read_meta(dirpath) -> dict:
    p = Path(dirpath) / "meta.json"
    return json.loads(p.read_text()) if p.exists() else {}


def read_mask(dirpath, split: str = "train"):
    p = Path(dirpath) / f"{split}.mask.bin"
    return np.fromfile(p, dtype=np.uint8) if p.exists() else None


def read_weights(dirpath, split: str = "train"):
    p = Path(dirpath) / f"{split}.weight.bin"
    return np.fromfile(p, dtype="<f4") if p.exists() else None


def write_dataset(dirpath, train, val, vocab_size, itos=None, mask=None, weights=None) -> None:
    width = 16 if vocab_size <= 0x10000 else 32
    d = Path(dirpath)
    name = (lambda s: f"{s}.bin") if width == 16 else (lambda s: f"{s}.u32.bin")
    write_tokens(d / name("train"), train, width)
    write_tokens(d / name("val"), val, width)
    write_meta(d, vocab_size, itos, width)
    if mask is not None:
        np.asarray(mask, dtype=np.uint8).tofile(d / "train.mask.bin")
    if weights is not None:
        np.asarray(weights, dtype="<f4").tofile(d / "train.weight.bin")
