"""GGUF container: reader, writer and the block codecs this framework can decode or encode.

GGUF (version 2/3) is little-endian: ``"GGUF"``, version u32, tensor count u64, key/value count u64,
the key/value table (typed scalars, strings, arrays), one info record per tensor (name, rank,
dimensions fastest-first, ggml type, offset into the data section) and the data section aligned to
``general.alignment`` (32 when absent).  The reader maps the file and decodes one tensor at a time
to fp32 in row-major order of the *reversed* dimension list (so a ``[out, in]`` weight comes back
as ``[out, in]``), which lets a checkpoint larger than memory be walked.

Decoded types: F32, F16, BF16, Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q4_K, Q5_K, Q6_K, I8/I16/I32.
Encoded types: F32, F16, BF16, Q8_0, Q4_0 (round-to-nearest block quantisers, identical to ggml's
reference quantisers).

Reference: crates/checkpoint/src/gguf.rs (reader + codecs), gguf_write.rs (writer),
quantize.rs:79-337 (any checkpoint -> GGUF at a tier, every skipped tensor with a stated reason)."""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

MAGIC = b"GGUF"
DEFAULT_ALIGNMENT = 32

# ggml tensor types: id -> (name, elements per block, bytes per block)
T_F32, T_F16, T_Q4_0, T_Q4_1, T_Q5_0, T_Q5_1, T_Q8_0 = 0, 1, 2, 3, 6, 7, 8
T_Q4_K, T_Q5_K, T_Q6_K = 12, 13, 14
T_I8, T_I16, T_I32, T_BF16 = 24, 25, 26, 30
TYPES: Dict[int, Tuple[str, int, int]] = {
    T_F32: ("F32", 1, 4), T_F16: ("F16", 1, 2), T_BF16: ("BF16", 1, 2),
    T_Q4_0: ("Q4_0", 32, 18), T_Q4_1: ("Q4_1", 32, 20), T_Q5_0: ("Q5_0", 32, 22), T_Q5_1: ("Q5_1", 32, 24),
    T_Q8_0: ("Q8_0", 32, 34), T_Q4_K: ("Q4_K", 256, 144), T_Q5_K: ("Q5_K", 256, 176), T_Q6_K: ("Q6_K", 256, 210),
    T_I8: ("I8", 1, 1), T_I16: ("I16", 1, 2), T_I32: ("I32", 1, 4),
}
TYPE_BY_NAME = {v[0]: k for k, v in TYPES.items()}

# key/value value types
_KV_FMT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
KV_STRING, KV_ARRAY = 8, 9


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]      # row-major (slowest first): the reverse of the order stored in the file
    ggml_type: int
    offset: int                 # relative to the start of the data section

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self) -> int:
        _, be, bb = TYPES[self.ggml_type]
        return self.numel // be * bb

    @property
    def type_name(self) -> str:
        return TYPES[self.ggml_type][0]


# ------------------------------------------------------------------------------------ codecs
def _f16(buf: np.ndarray) -> np.ndarray:
    return buf.view(np.float16).astype(np.float32)


def dequantize(raw: np.ndarray, ggml_type: int, numel: int) -> np.ndarray:
    """fp32 values of ``numel`` elements stored as ``raw`` (uint8) in the given ggml type."""
    if ggml_type not in TYPES:
        raise ValueError(f"ggml type {ggml_type} is not supported")
    name, be, bb = TYPES[ggml_type]
    if numel % be:
        raise ValueError(f"{name}: {numel} elements is not a whole number of {be}-element blocks")
    nb = numel // be
    raw = np.ascontiguousarray(raw[: nb * bb])
    if name == "F32":
        return raw.view(np.float32).copy()
    if name == "F16":
        return _f16(raw)
    if name == "BF16":
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    if name in ("I8", "I16", "I32"):
        return raw.view({"I8": np.int8, "I16": np.int16, "I32": np.int32}[name]).astype(np.float32)
    blk = raw.reshape(nb, bb)
    if name == "Q8_0":
        d = _f16(blk[:, :2].copy()).reshape(nb, 1)
        return (d * blk[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)
    if name in ("Q4_0", "Q4_1"):
        d = _f16(blk[:, :2].copy()).reshape(nb, 1)
        if name == "Q4_1":
            m = _f16(blk[:, 2:4].copy()).reshape(nb, 1)
            qs = blk[:, 4:]
        else:
            m, qs = None, blk[:, 2:]
        q = np.concatenate([qs & 0x0F, qs >> 4], axis=1).astype(np.float32)
        return ((q - 8.0) * d if m is None else q * d + m).reshape(-1)
    if name in ("Q5_0", "Q5_1"):
        d = _f16(blk[:, :2].copy()).reshape(nb, 1)
        if name == "Q5_1":
            m = _f16(blk[:, 2:4].copy()).reshape(nb, 1)
            qh, qs = blk[:, 4:8], blk[:, 8:]
        else:
            m, qh, qs = None, blk[:, 2:6], blk[:, 6:]
        bits = np.unpackbits(qh, axis=1, bitorder="little")          # [nb, 32], bit j of the u32
        q = np.concatenate([qs & 0x0F, qs >> 4], axis=1) | (bits << 4)
        q = q.astype(np.float32)
        return ((q - 16.0) * d if m is None else q * d + m).reshape(-1)
    if name == "Q6_K":
        ql, qh = blk[:, :128], blk[:, 128:192]
        sc = blk[:, 192:208].view(np.int8).astype(np.float32)        # 16 scales
        d = _f16(blk[:, 208:210].copy()).reshape(nb, 1)
        out = np.empty((nb, 256), dtype=np.float32)
        for half in range(2):
            l_, h_ = ql[:, half * 64: half * 64 + 64], qh[:, half * 32: half * 32 + 32]
            q1 = (l_[:, :32] & 0x0F) | ((h_ & 3) << 4)
            q2 = (l_[:, 32:] & 0x0F) | (((h_ >> 2) & 3) << 4)
            q3 = (l_[:, :32] >> 4) | (((h_ >> 4) & 3) << 4)
            q4 = (l_[:, 32:] >> 4) | (((h_ >> 6) & 3) << 4)
            for k, q in enumerate((q1, q2, q3, q4)):
                s = np.repeat(sc[:, half * 8 + 2 * k: half * 8 + 2 * k + 2], 16, axis=1)   # is = l / 16
                out[:, half * 128 + k * 32: half * 128 + k * 32 + 32] = (q.astype(np.float32) - 32.0) * s
        return (out * d).reshape(-1)
    if name in ("Q4_K", "Q5_K"):
        d = _f16(blk[:, 0:2].copy()).reshape(nb, 1)
        dmin = _f16(blk[:, 2:4].copy()).reshape(nb, 1)
        s12 = blk[:, 4:16]
        sc = np.empty((nb, 8), dtype=np.float32)
        mn = np.empty((nb, 8), dtype=np.float32)
        for j in range(8):
            if j < 4:
                sc[:, j] = s12[:, j] & 63
                mn[:, j] = s12[:, j + 4] & 63
            else:
                sc[:, j] = (s12[:, j + 4] & 0x0F) | ((s12[:, j - 4] >> 6) << 4)
                mn[:, j] = (s12[:, j + 4] >> 4) | ((s12[:, j] >> 6) << 4)
        if name == "Q4_K":
            qs = blk[:, 16:144]
            hi = None
        else:
            hi = np.unpackbits(blk[:, 16:48], axis=1, bitorder="little").reshape(nb, 32, 8)   # qh[l] bit u
            qs = blk[:, 48:176]
        out = np.empty((nb, 256), dtype=np.float32)
        for grp in range(4):                       # 64 elements each: low nibbles then high nibbles
            q = qs[:, grp * 32: grp * 32 + 32]
            lo, hi4 = (q & 0x0F).astype(np.float32), (q >> 4).astype(np.float32)
            if hi is not None:
                lo = lo + 16.0 * hi[:, :, 2 * grp]
                hi4 = hi4 + 16.0 * hi[:, :, 2 * grp + 1]
            out[:, grp * 64: grp * 64 + 32] = d * sc[:, 2 * grp: 2 * grp + 1] * lo - dmin * mn[:, 2 * grp: 2 * grp + 1]
            out[:, grp * 64 + 32: grp * 64 + 64] = (d * sc[:, 2 * grp + 1: 2 * grp + 2] * hi4
                                                   - dmin * mn[:, 2 * grp + 1: 2 * grp + 2])
        return out.reshape(-1)
    raise ValueError(f"no decoder for {name}")


def quantize(x: np.ndarray, ggml_type: int) -> np.ndarray:
    """Encode fp32 values (a whole number of blocks) as uint8 bytes of the given type."""
    name, be, bb = TYPES[ggml_type]
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    if x.size % be:
        raise ValueError(f"{name}: {x.size} elements is not a whole number of {be}-element blocks")
    if name == "F32":
        return x.view(np.uint8).copy()
    if name == "F16":
        return x.astype(np.float16).view(np.uint8)
    if name == "BF16":
        u = x.view(np.uint32)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)      # round to nearest even
        return r.view(np.uint8)
    nb = x.size // be
    b = x.reshape(nb, be)
    out = np.empty((nb, bb), dtype=np.uint8)
    if name == "Q8_0":
        amax = np.abs(b).max(axis=1, keepdims=True)
        d = amax / 127.0
        inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1.0), 0.0)
        out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
        out[:, 2:] = np.round(b * inv).astype(np.int8).view(np.uint8)
        return out.reshape(-1)
    if name == "Q4_0":
        idx = np.abs(b).argmax(axis=1)
        mx = b[np.arange(nb), idx].reshape(nb, 1)            # the signed value of largest magnitude
        d = mx / -8.0
        inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1.0), 0.0)
        q = np.minimum(15, (b * inv + 8.5).astype(np.int32)).astype(np.uint8)
        out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
        out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
        return out.reshape(-1)
    raise ValueError(f"no encoder for {name}")


# ------------------------------------------------------------------------------------ reader
class GgufReader:
    """Memory-mapped GGUF file: ``metadata`` (dict), ``tensors`` (name -> TensorInfo), ``read(name)``
    -> fp32 ``numpy`` array in the tensor's row-major shape."""

    def __init__(self, path: str):
        self.path = str(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._pos = 0
        if self._take(4) != MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        self.version = self._scalar("<I")
        if self.version not in (2, 3):
            raise ValueError(f"{path}: GGUF version {self.version} is not supported")
        n_tensors, n_kv = self._scalar("<Q"), self._scalar("<Q")
        self.metadata: Dict[str, object] = {}
        for _ in range(n_kv):
            key = self._string()
            self.metadata[key] = self._value(self._scalar("<I"))
        self.tensors: Dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = self._string()
            rank = self._scalar("<I")
            dims = [self._scalar("<Q") for _ in range(rank)]
            ttype = self._scalar("<I")
            off = self._scalar("<Q")
            self.tensors[name] = TensorInfo(name, tuple(reversed(dims)), ttype, off)
        align = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        self.data_start = (self._pos + align - 1) // align * align
        size = len(self._mm)
        for t in self.tensors.values():
            if t.ggml_type not in TYPES:
                continue        # listed, but read() refuses it
            if self.data_start + t.offset + t.nbytes > size:
                raise ValueError(f"{path}: tensor {t.name!r} reaches past the end of the file")

    # -- low level
    def _take(self, n: int) -> bytes:
        if self._pos + n > len(self._mm):
            raise ValueError(f"{self.path}: truncated header")
        b = self._mm[self._pos:self._pos + n]
        self._pos += n
        return b

    def _scalar(self, fmt: str):
        return struct.unpack(fmt, self._take(struct.calcsize(fmt)))[0]

    def _string(self) -> str:
        n = self._scalar("<Q")
        if n > (1 << 24):
            raise ValueError(f"{self.path}: implausible string length {n}")
        return self._take(n).decode("utf-8", errors="replace")

    def _value(self, vt: int):
        if vt in _KV_FMT:
            return self._scalar(_KV_FMT[vt])
        if vt == KV_STRING:
            return self._string()
        if vt == KV_ARRAY:
            et, n = self._scalar("<I"), self._scalar("<Q")
            if et in _KV_FMT and et != 7:
                fmt = _KV_FMT[et]
                size = struct.calcsize(fmt)
                return np.frombuffer(self._take(size * n), dtype=np.dtype(fmt[1:]).newbyteorder("<")).tolist()
            return [self._value(et) for _ in range(n)]
        raise ValueError(f"{self.path}: unknown key/value type {vt}")

    # -- tensors
    def names(self) -> List[str]:
        return list(self.tensors)

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        a = self.data_start + t.offset
        return np.frombuffer(self._mm, dtype=np.uint8, count=t.nbytes, offset=a)

    def read(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return dequantize(self.raw(name), t.ggml_type, t.numel).reshape(t.shape)

    def close(self):
        if getattr(self, "_mm", None) is not None:
            self._mm.close()
            self._f.close()
            self._mm = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


# ------------------------------------------------------------------------------------ writer
def _kv_bytes(value) -> bytes:
    def s(x: str) -> bytes:
        b = x.encode("utf-8")
        return struct.pack("<Q", len(b)) + b
    if isinstance(value, bool):
        return struct.pack("<I?", 7, value)
    if isinstance(value, int):
        return struct.pack("<Iq", 11, value) if value < 0 else struct.pack("<IQ", 10, value) if value >= 1 << 32 \
            else struct.pack("<II", 4, value)
    if isinstance(value, float):
        return struct.pack("<If", 6, value)
    if isinstance(value, str):
        return struct.pack("<I", KV_STRING) + s(value)
    if isinstance(value, (list, tuple)):
        if all(isinstance(v, str) for v in value):
            return struct.pack("<IIQ", KV_ARRAY, KV_STRING, len(value)) + b"".join(s(v) for v in value)
        if all(isinstance(v, int) and not isinstance(v, bool) for v in value):
            return struct.pack("<IIQ", KV_ARRAY, 5, len(value)) + np.asarray(value, dtype="<i4").tobytes()
        if all(isinstance(v, (int, float)) for v in value):
            return struct.pack("<IIQ", KV_ARRAY, 6, len(value)) + np.asarray(value, dtype="<f4").tobytes()
    raise TypeError(f"cannot store {type(value).__name__} in GGUF metadata")


def write_gguf(path: str, metadata: Dict[str, object], tensors: Iterable[Tuple[str, Tuple[int, ...], int, np.ndarray]],
               alignment: int = DEFAULT_ALIGNMENT) -> int:
    """Write a GGUF v3 file atomically (temporary + rename).  ``tensors``: (name, row-major shape,
    ggml type, encoded bytes as uint8).  Returns the file size."""
    import os
    tensors = list(tensors)
    meta = dict(metadata)
    meta.setdefault("general.alignment", alignment)
    head = MAGIC + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for k, v in meta.items():
        kb = k.encode("utf-8")
        head += struct.pack("<Q", len(kb)) + kb + _kv_bytes(v)
    off = 0
    offsets = []
    for name, shape, ttype, data in tensors:
        nb = name.encode("utf-8")
        head += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(shape))
        head += b"".join(struct.pack("<Q", d) for d in reversed(shape))
        head += struct.pack("<IQ", ttype, off)
        offsets.append(off)
        off = (off + len(data) + alignment - 1) // alignment * alignment
    tmp = str(path) + ".tmp"
    with open(tmp, "wb") as f:
        f.write(head)
        f.write(b"\0" * (-len(head) % alignment))
        base = f.tell()
        for (name, shape, ttype, data), o in zip(tensors, offsets):
            f.seek(base + o)
            f.write(np.ascontiguousarray(data, dtype=np.uint8).tobytes())
        end = base + off
        f.truncate(end)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
    return end
