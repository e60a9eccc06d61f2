"""Binding of the native serving forward (``csrc/serve/qwen_forward.cu``): the ctypes mirrors of its
structs, a per-engine descriptor of the weights / KV pools / tensor-parallel buffers, and scratch
sets sized per row count.  The engine calls ``pre_attn`` / ``post_attn`` around its own attention for
prefill, and ``decode`` for a whole decode step."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import torch

from ..ops import _cuda
from ..ops._cuda import NativeError, stream_ptr

P = C.c_void_p


class Lin(C.Structure):
    _fields_ = [("w", P), ("scale", P), ("bias", P), ("n", C.c_int), ("k", C.c_int)]


class Layer(C.Structure):
    _fields_ = [("ln1", P), ("ln2", P), ("q_norm", P), ("k_norm", P),
                ("qkv", Lin), ("wo", Lin), ("gate_up", Lin), ("down", Lin),
                ("kc", P), ("vc", P), ("ks", P), ("vs", P), ("kv_clip", P)]


class Cfg(C.Structure):
    _fields_ = [("d_model", C.c_int), ("hq", C.c_int), ("hk", C.c_int), ("hd", C.c_int), ("ff", C.c_int),
                ("block_size", C.c_int), ("kv_int8", C.c_int), ("n_layers", C.c_int),
                ("eps", C.c_float), ("tp_world", C.c_int), ("tp_rank", C.c_int), ("fuse_quant", C.c_int),
                ("cos_t", P), ("sin_t", P), ("layers", P),
                ("stage_ptrs", P), ("res_ptrs", P * 2), ("sig_ptrs", P), ("res", P * 2),
                ("epoch_dev", P), ("counters", P), ("wait_seconds", C.c_double), ("ar_cap", C.c_long)]


class Work(C.Structure):
    _fields_ = [(n, P) for n in ("xa", "xb", "h", "qkv", "qk", "o", "proj", "mlp", "gu", "act", "xq", "sx", "rstd",
                                 "part_o", "part_ml")] + [("rows", C.c_int), ("splits", C.c_int)]


class State(C.Structure):
    _fields_ = [("x", P), ("delta", P), ("parity", C.c_int), ("n_allreduce", C.c_int)]


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _lin(l) -> Lin:
    if l.int8:
        return Lin(_ptr(l.wq), _ptr(l.sw), None, l.wq.shape[0], l.wq.shape[1])
    return Lin(_ptr(l.w), None, _ptr(l.bias), l.w.shape[0], l.w.shape[1])


class Scratch:
    """Device buffers for up to ``rows`` rows (+ their Work struct).  ``qk``, ``qkv`` and ``o`` are
    exposed as tensors: the engine's attention reads and writes them."""

    def __init__(self, eng, rows: int, splits: int = 1):
        dev, dt = eng.device, eng.dtype
        d, hq, hk, hd, ff = eng.cfg.d_model, eng.hq, eng.hk, eng.hd, eng.ff_local
        e = lambda *s, dtype=dt: torch.empty(*s, device=dev, dtype=dtype)
        self.rows, self.splits = rows, splits
        self.xa, self.xb, self.h = e(rows, d), e(rows, d), e(rows, d)
        self.qkv, self.qk, self.o = e(rows, (hq + 2 * hk) * hd), e(rows, (hq + hk) * hd), e(rows, hq * hd)
        self.proj, self.mlp, self.gu, self.act = e(rows, d), e(rows, d), e(rows, 2 * ff), e(rows, ff)
        self.xq = e(rows, max(d, ff, hq * hd), dtype=torch.int8)
        self.sx = e(rows, dtype=torch.float32)
        self.rstd = e(rows * (hq + hk), dtype=torch.float32)
        self.part_o = e(rows * hq * splits * hd, dtype=torch.float32)
        self.part_ml = e(rows * hq * splits * 2, dtype=torch.float32)
        self.hn = e(rows, d)
        self.work = Work(*[_ptr(getattr(self, n)) for n in ("xa", "xb", "h", "qkv", "qk", "o", "proj", "mlp", "gu",
                                                           "act", "xq", "sx", "rstd", "part_o", "part_ml")],
                         rows, splits)


class NativeForward:
    """Per-engine descriptor.  ``supported(engine)`` says whether the native path covers the
    engine's configuration (everything except a bias on an int8 projection)."""

    @staticmethod
    def supported(eng) -> bool:
        if not eng.cuda:
            return False
        for l in eng.layers:
            for k in ("qkv", "wo", "gate_up", "down"):
                if l[k].int8 and l[k].bias is not None:
                    return False
        return True

    def __init__(self, eng):
        self.eng = eng
        self.lib = _cuda.lib()
        n = len(eng.layers)
        self._layers = (Layer * n)()
        for i, l in enumerate(eng.layers):
            L = self._layers[i]
            L.ln1, L.ln2 = _ptr(l["ln1"]), _ptr(l["ln2"])
            L.q_norm, L.k_norm = _ptr(l["q_norm"]), _ptr(l["k_norm"])
            L.qkv, L.wo, L.gate_up, L.down = _lin(l["qkv"]), _lin(l["wo"]), _lin(l["gate_up"]), _lin(l["down"])
            L.kc, L.vc = _ptr(eng.kc[i]), _ptr(eng.vc[i])
            if eng.kv_int8:
                L.ks, L.vs = _ptr(eng.ks[i]), _ptr(eng.vs[i])
                L.kv_clip = _ptr(eng.kv_clip[i]) if eng.kv_clip is not None else None
        c = self.cfg = Cfg()
        c.d_model, c.hq, c.hk, c.hd, c.ff = eng.cfg.d_model, eng.hq, eng.hk, eng.hd, eng.ff_local
        c.block_size, c.kv_int8, c.n_layers = eng.block_size, int(eng.kv_int8), n
        c.eps = float(eng.cfg.rms_eps)
        c.cos_t, c.sin_t = _ptr(eng.cos), _ptr(eng.sin)
        c.layers = C.cast(self._layers, P)
        c.tp_world, c.tp_rank = eng.tp_world, eng.tp_rank
        c.fuse_quant = 1     # W8A8: norm / SwiGLU kernels that write int8 rows + scales (same values)
        self.state = State()
        self._scratch: Dict[tuple, Scratch] = {}
        for name in ("bb_serve_begin", "bb_serve_pre_attn", "bb_serve_post_attn", "bb_serve_finish",
                     "bb_serve_decode"):
            getattr(self.lib, name).restype = C.c_int

    # ---- tensor-parallel buffers (the two-shot all-reduce's staging / result / flag memory)
    def _bind_tp(self, elems: int) -> None:
        tp = self.eng.tp
        if tp is None or tp.world == 1:
            return
        st = tp.ensure_ar2(elems)
        c = self.cfg
        c.stage_ptrs = C.cast(st["stage_ptrs"], P)
        c.res_ptrs[0], c.res_ptrs[1] = C.cast(st["res_ptrs"][0], P), C.cast(st["res_ptrs"][1], P)
        c.sig_ptrs = C.cast(tp.ar2_sig_ptrs, P)
        c.res[0], c.res[1] = st["res"][0].data_ptr(), st["res"][1].data_ptr()
        c.epoch_dev, c.counters = tp.ar2_state.data_ptr(), tp.ar2_state[1:].data_ptr()
        c.wait_seconds = float(tp.wait_seconds)
        c.ar_cap = int(st["cap"])
        self.state.parity = tp.ar2_calls & 1

    def _sync_tp(self, before: int) -> None:
        tp = self.eng.tp
        if tp is not None and tp.world > 1:
            tp.ar2_calls += self.state.n_allreduce - before

    def scratch(self, rows: int, splits: int = 1, key=None) -> Scratch:
        k = key if key is not None else (rows, splits)
        s = self._scratch.get(k)
        if s is None or s.rows < rows or s.splits != splits:
            s = Scratch(self.eng, rows, splits)
            self._scratch[k] = s
        return s

    def _check(self, rc: int, what: str) -> None:
        _cuda.launch_count += 1
        if rc != 0:
            raise NativeError(f"{what} failed with code {rc}")

    # ---- prefill pieces
    def begin(self, sc: Scratch, tok: torch.Tensor, n: int) -> None:
        self._bind_tp(n * self.cfg.d_model)
        self._n0 = self.state.n_allreduce
        self._check(self.lib.bb_serve_begin(C.byref(self.cfg), C.byref(sc.work), P(self.eng.tok.data_ptr()),
                                            self.eng.tok.shape[0], P(tok.data_ptr()), n, C.byref(self.state),
                                            stream_ptr()), "bb_serve_begin")

    def pre_attn(self, sc: Scratch, li: int, pos: torch.Tensor, slots: torch.Tensor, n: int) -> None:
        self._check(self.lib.bb_serve_pre_attn(C.byref(self.cfg), li, C.byref(sc.work), P(pos.data_ptr()),
                                               P(slots.data_ptr()), n, C.byref(self.state), stream_ptr()),
                    "bb_serve_pre_attn")

    def post_attn(self, sc: Scratch, li: int, n: int) -> None:
        self._check(self.lib.bb_serve_post_attn(C.byref(self.cfg), li, C.byref(sc.work), n, C.byref(self.state),
                                                stream_ptr()), "bb_serve_post_attn")

    def finish(self, sc: Scratch, n: int) -> torch.Tensor:
        self._check(self.lib.bb_serve_finish(C.byref(self.cfg), C.byref(sc.work), P(self.eng.norm.data_ptr()),
                                             P(sc.hn.data_ptr()), n, C.byref(self.state), stream_ptr()),
                    "bb_serve_finish")
        self._sync_tp(self._n0)
        return sc.hn[:n]

    # ---- a whole decode step
    def decode(self, sc: Scratch, tok, pos, slots, bts, seqlens, n: int) -> torch.Tensor:
        self._bind_tp(n * self.cfg.d_model)
        n0 = self.state.n_allreduce
        self._check(self.lib.bb_serve_decode(
            C.byref(self.cfg), C.byref(sc.work), P(self.eng.tok.data_ptr()), self.eng.tok.shape[0],
            P(tok.data_ptr()), P(pos.data_ptr()), P(slots.data_ptr()), P(bts.data_ptr()), bts.shape[1],
            P(seqlens.data_ptr()), P(self.eng.norm.data_ptr()), P(sc.hn.data_ptr()), n, C.byref(self.state),
            stream_ptr()), "bb_serve_decode")
        self._sync_tp(n0)
        return sc.hn[:n]
