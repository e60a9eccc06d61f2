"""Checkpoint container: standard safetensors with ``__metadata__["brain.config"]`` (config JSON)
and ``["brain.card"]`` (model card JSON).  Parameters are written 1-D, dtype F32 (optionally
BF16/F16), shape ``[numel]``, under the reference's names and order; written atomically through
``<path>.tmp`` + rename.  The loader accepts F32/F16/BF16 and any shape.
Reference: crates/checkpoint/src/st.rs:112-114,161-186,216,263-308; crates/checkpoint/src/lib.rs:180-215.
The byte path (mmap, dtype decode, append, fsync/rename) is native: csrc/runtime/safetensors.cpp."""
from __future__ import annotations

import ctypes
import json
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .. import _host
from .card import CARD_KEY, CONFIG_KEY, ModelCard

c = ctypes
_host.register({
    "bbh_st_map": (c.c_void_p, [c.c_char_p]),
    "bbh_st_unmap": (None, [c.c_void_p]),
    "bbh_st_header_len": (c.c_uint64, [c.c_void_p]),
    "bbh_st_header_ptr": (c.c_void_p, [c.c_void_p]),
    "bbh_st_data_bytes": (c.c_uint64, [c.c_void_p]),
    "bbh_st_decode_f32": (c.c_int, [c.c_void_p, c.c_uint64, c.c_int64, c.c_int, c.c_void_p]),
    "bbh_st_read_raw": (c.c_int, [c.c_void_p, c.c_uint64, c.c_uint64, c.c_void_p]),
    "bbh_stw_open": (c.c_void_p, [c.c_char_p, c.c_char_p, c.c_uint64]),
    "bbh_stw_append_f32": (c.c_int, [c.c_void_p, c.c_void_p, c.c_int64, c.c_int]),
    "bbh_stw_append_raw": (c.c_int, [c.c_void_p, c.c_void_p, c.c_uint64]),
    "bbh_stw_close": (c.c_int, [c.c_void_p, c.c_char_p, c.c_int]),
})

_DT = {"F32": 0, "F16": 1, "BF16": 2}
_ES = {"F32": 4, "F16": 2, "BF16": 2, "I8": 1, "U8": 1, "I32": 4, "U32": 4, "I64": 8, "F64": 8, "F8_E4M3": 1}
_TORCH = {"I8": torch.int8, "U8": torch.uint8, "I32": torch.int32, "I64": torch.int64,
          "F64": torch.float64, "U32": torch.int32}


class WeightReader:
    """Streaming reader over one safetensors file: tensors are decoded to fp32 one at a time
    straight from the mapping, so checkpoints larger than RAM can be walked."""

    def __init__(self, path: str):
        self.path = str(path)
        self._h = _host.lib().bbh_st_map(self.path.encode())
        if not self._h:
            raise FileNotFoundError(f"cannot map safetensors file {path}")
        n = _host.lib().bbh_st_header_len(self._h)
        raw = ctypes.string_at(_host.lib().bbh_st_header_ptr(self._h), n)
        hdr = json.loads(raw.decode("utf-8"))
        self.metadata: Dict[str, str] = hdr.pop("__metadata__", {}) or {}
        self.entries: Dict[str, dict] = hdr
        data_bytes = _host.lib().bbh_st_data_bytes(self._h)
        for name, e in hdr.items():
            b, en = e["data_offsets"]
            if not (0 <= b <= en <= data_bytes):
                raise ValueError(f"{path}: tensor {name!r} has offsets outside the file")

    def close(self):
        if getattr(self, "_h", None):
            _host.lib().bbh_st_unmap(self._h)
            self._h = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def names(self) -> List[str]:
        return sorted(self.entries, key=lambda k: self.entries[k]["data_offsets"][0])

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> str:
        return self.entries[name]["dtype"]

    def read(self, name: str) -> torch.Tensor:
        """fp32 tensor (F32/F16/BF16 sources) or the raw integer tensor, in the stored shape."""
        e = self.entries[name]
        dt, shape = e["dtype"], e["shape"]
        b, en = e["data_offsets"]
        numel = 1
        for s in shape:
            numel *= s
        if dt not in _ES:
            raise ValueError(f"{name}: unsupported dtype {dt}")
        if (en - b) != numel * _ES[dt]:
            raise ValueError(f"{name}: byte length does not match shape/dtype")
        if dt in _DT:
            out = torch.empty(numel, dtype=torch.float32)
            rc = _host.lib().bbh_st_decode_f32(self._h, b, numel, _DT[dt], out.data_ptr())
            if rc != 0:
                raise IOError(f"decode of {name} failed ({rc})")
            return out.view(shape)
        if dt in _TORCH:
            out = torch.empty(numel, dtype=_TORCH[dt])
            rc = _host.lib().bbh_st_read_raw(self._h, b, en - b, out.data_ptr())
            if rc != 0:
                raise IOError(f"read of {name} failed ({rc})")
            if dt == "U32":
                # torch has no arithmetic on uint32: widen, so values >= 2^31 stay positive
                out = (out.to(torch.int64) & 0xFFFFFFFF)
            return out.view(shape)
        if dt == "F8_E4M3":
            # raw (unscaled) fp8 values as fp32; block scales are applied by the importer
            out = torch.empty(numel, dtype=torch.uint8)
            rc = _host.lib().bbh_st_read_raw(self._h, b, en - b, out.data_ptr())
            if rc != 0:
                raise IOError(f"read of {name} failed ({rc})")
            return out.view(torch.float8_e4m3fn).float().view(shape)
        raise ValueError(f"{name}: unsupported dtype {dt}")

    def config(self) -> Optional[dict]:
        raw = self.metadata.get(CONFIG_KEY)
        return json.loads(raw) if raw else None

    def card(self) -> Optional[ModelCard]:
        return ModelCard.from_metadata(self.metadata)


class StWriter:
    """Incremental writer: declare every tensor up front (name, numel or shape), then ``write`` them
    in the same order; ``close`` fsyncs and renames the temporary into place."""

    def __init__(self, path: str, specs: Iterable[Tuple[str, Tuple[int, ...]]], metadata: Dict[str, str],
                 dtype: str = "F32"):
        self.path = str(path)
        self.dtype = dtype
        self.specs = []
        self.dtypes = {}
        for spec in specs:
            n, s = spec[0], spec[1]
            self.specs.append((n, tuple(int(x) for x in (s if isinstance(s, (tuple, list)) else (s,)))))
            self.dtypes[n] = spec[2] if len(spec) > 2 else dtype      # optional per-tensor dtype
        hdr = {"__metadata__": {k: str(v) for k, v in metadata.items()}}
        off = 0
        for n, shape in self.specs:
            numel = 1
            for s in shape:
                numel *= s
            nb = numel * _ES[self.dtypes[n]]
            hdr[n] = {"dtype": self.dtypes[n], "shape": list(shape), "data_offsets": [off, off + nb]}
            off += nb
        raw = json.dumps(hdr, separators=(",", ":")).encode("utf-8")
        raw += b" " * ((8 - len(raw) % 8) % 8)
        self._h = _host.lib().bbh_stw_open(self.path.encode(), raw, len(raw))
        if not self._h:
            raise IOError(f"cannot open {path}.tmp for writing")
        self._i = 0

    def write(self, name: str, t: torch.Tensor):
        exp, shape = self.specs[self._i]
        if exp != name:
            raise ValueError(f"tensors must be written in declared order: expected {exp}, got {name}")
        dt = self.dtypes[name]
        numel = 1
        for s in shape:
            numel *= s
        if t.numel() != numel:
            raise ValueError(f"{name}: got {t.numel()} elements, declared {numel}")
        if dt in _DT:
            flat = t.detach().reshape(-1).to(device="cpu", dtype=torch.float32).contiguous()
            rc = _host.lib().bbh_stw_append_f32(self._h, flat.data_ptr(), numel, _DT[dt])
        else:
            flat = t.detach().reshape(-1).to(device="cpu", dtype=_TORCH[dt]).contiguous()
            rc = _host.lib().bbh_stw_append_raw(self._h, flat.data_ptr(), numel * _ES[dt])
        if rc != 0:
            raise IOError(f"write of {name} failed ({rc})")
        self._i += 1

    def close(self, abort: bool = False):
        if self._h:
            incomplete = self._i != len(self.specs)
            rc = _host.lib().bbh_stw_close(self._h, self.path.encode(), int(abort or incomplete))
            self._h = None
            if rc != 0 and not abort:
                raise IOError(f"finalising {self.path} failed ({rc})")
            if incomplete and not abort:
                raise IOError(f"{self.path}: only {self._i} of {len(self.specs)} tensors written")


def save(path: str, tensors: Dict[str, torch.Tensor], config: Optional[dict] = None,
         card: Optional[ModelCard] = None, dtype: str = "F32", order: Optional[List[str]] = None):
    """Write ``tensors`` (1-D ``[numel]`` each) with the config/card metadata, atomically."""
    meta: Dict[str, str] = {}
    if card is not None:
        meta.update(card.to_metadata())
    if config is not None:
        meta[CONFIG_KEY] = json.dumps(config, separators=(",", ":"))
    names = order if order is not None else list(tensors)
    w = StWriter(path, [(n, (tensors[n].numel(),)) for n in names], meta, dtype)
    try:
        for n in names:
            w.write(n, tensors[n])
    except BaseException:
        w.close(abort=True)
        raise
    w.close()


def load(path: str) -> Tuple[Dict[str, torch.Tensor], Optional[dict], Optional[ModelCard]]:
    """All tensors as fp32, plus the parsed config and card."""
    with WeightReader(path) as r:
        return {n: r.read(n) for n in r.names()}, r.config(), r.card()


def save_model(path: str, model, card: Optional[ModelCard] = None, dtype: str = "F32"):
    """Save a framework model under the reference's tensor names / order with its config JSON."""
    state = model.reference_state()
    if card is None:
        fam = getattr(model, "family", "qwen")
        card = ModelCard(id={"gpt": "brain/gpt", "qwen": "brain/qwen3"}.get(fam, f"brain/{fam}"),
                         family=fam, param_count=sum(t.numel() for t in state.values()),
                         capabilities=["generate"])
    save(path, state, model.config_json(), card, dtype)


def load_model(path: str, device="cpu", dtype=None):
    """Rebuild the model a checkpoint describes (its config wins) and load the weights."""
    from ..models import build_from_config
    tensors, config, card = load(path)
    if config is None:
        raise ValueError(f"{path}: no brain.config metadata")
    model = build_from_config(config)
    model.load_reference_state(tensors, strict=True)
    if dtype is not None or device != "cpu":
        model = model.to(device=device, dtype=dtype)
    return model, config, card
