"""Token-window batch sampler (reference: crates/data/src/loader.rs:125-290), native hot path.

``TokenDataset.get_batch`` draws ``batch`` random window starts with the SplitMix64 stream (or
line-aligned starts), shifts targets by one and writes ``IGNORE`` (-1) on masked positions:
prompt masking up to a marker token (global or per line) and the optional per-token supervision
mask.  Output arrays are pinned host tensors so the trainer's H2D copy is asynchronous."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .. import _host
from .rng import Rng

IGNORE = -1


@dataclass
class BatchConfig:
    batch_size: int
    block_size: int
    mask_before_token: Optional[int] = None
    mask_per_line: bool = False
    newline_token: Optional[int] = None


class TokenDataset:
    def __init__(self, data, mask=None, weights=None):
        self.data = np.ascontiguousarray(np.asarray(data, dtype=np.uint32))
        m = None if mask is None else np.ascontiguousarray(np.asarray(mask, dtype=np.uint8))
        w = None if weights is None else np.ascontiguousarray(np.asarray(weights, dtype=np.float32))
        if m is not None and m.size != self.data.size:
            raise ValueError("mask length must match data length")
        if w is not None and w.size != self.data.size:
            raise ValueError("weights length must match data length")
        self._h = _host.lib().bbh_dataset_new(self.data.ctypes.data, self.data.size,
                                              m.ctypes.data if m is not None else None,
                                              w.ctypes.data if w is not None else None)
        self.has_weights = w is not None

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _host.lib().bbh_dataset_free(h)
            except Exception:
                pass
            self._h = None

    def __len__(self):
        return int(self.data.size)

    def align_to_lines(self, newline_token: int, block_size: int) -> int:
        """Restrict window starts to line starts whose line fits the block; returns how many."""
        return int(_host.lib().bbh_dataset_align(self._h, newline_token, block_size))

    def get_batch(self, cfg: BatchConfig, rng: Rng, weighted: bool = False, pin: bool = False):
        b, t = cfg.batch_size, cfg.block_size
        if len(self) < t + 1:
            raise ValueError(f"dataset has {len(self)} tokens but block_size {t} needs at least "
                             f"{t + 1} - use a longer dataset or a smaller --block-size")
        x = torch.empty(b, t, dtype=torch.int32, pin_memory=pin)
        y = torch.empty(b, t, dtype=torch.int32, pin_memory=pin)
        w = torch.empty(b, t, dtype=torch.float32, pin_memory=pin) if weighted else None
        st = ctypes.c_uint64(rng.state)
        rc = _host.lib().bbh_dataset_get_batch(
            self._h, ctypes.byref(st), b, t,
            -1 if cfg.mask_before_token is None else int(cfg.mask_before_token),
            int(cfg.mask_per_line), -1 if cfg.newline_token is None else int(cfg.newline_token),
            x.data_ptr(), y.data_ptr(), w.data_ptr() if w is not None else None, None)
        if rc != 0:
            raise RuntimeError("native batch sampler failed")
        rng.state = st.value
        return (x, y, w) if weighted else (x, y)
