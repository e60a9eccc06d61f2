"""ctypes binding to the native host runtime (``brain_b200/_lib/libbrain_host.so``): data sampler,
paged-KV allocator and scheduler, safetensors I/O, host collectives, planners, BPE tokenizer.
Built from ``csrc/**/*.cpp`` on first use when missing (g++, a few seconds)."""
from __future__ import annotations

import ctypes
from pathlib import Path

_LIB = None
_PATH = Path(__file__).resolve().parent / "_lib" / "libbrain_host.so"

c_i64, c_u64, c_i32, c_u32 = ctypes.c_int64, ctypes.c_uint64, ctypes.c_int32, ctypes.c_uint32
c_f64, c_f32, c_vp, c_cp = ctypes.c_double, ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p
P = ctypes.POINTER

_SIGS = {
    "bbh_rng_seed": (c_u64, [c_u64]),
    "bbh_rng_next_u64": (c_u64, [P(c_u64)]),
    "bbh_rng_next_f64": (c_f64, [P(c_u64)]),
    "bbh_rng_fill_u64": (None, [P(c_u64), c_vp, c_i64]),
    "bbh_rng_fill_tokens": (None, [P(c_u64), c_vp, c_i64, c_i64]),
    "bbh_dataset_new": (c_vp, [c_vp, c_i64, c_vp, c_vp]),
    "bbh_dataset_free": (None, [c_vp]),
    "bbh_dataset_len": (c_i64, [c_vp]),
    "bbh_dataset_align": (c_i64, [c_vp, c_u32, c_i64]),
    "bbh_dataset_get_batch": (ctypes.c_int, [c_vp, P(c_u64), c_i64, c_i64, c_i64, ctypes.c_int,
                                             c_i64, c_vp, c_vp, c_vp, c_vp]),
}


def register(sigs: dict) -> None:
    """Let other modules declare the signatures of the entry points they use."""
    _SIGS.update(sigs)
    if _LIB is not None:
        _apply(_LIB, sigs)


def _apply(lib, sigs):
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        from . import _build
        _build.build_host()
        _LIB = ctypes.CDLL(str(_PATH))
        _apply(_LIB, _SIGS)
    return _LIB
