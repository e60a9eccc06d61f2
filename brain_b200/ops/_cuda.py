"""ctypes binding to the in-tree sm_100a kernel library (``brain_b200/_lib/libbrain_b200.so``).

Every exported launcher takes raw device pointers plus a CUDA stream handle and returns an int
(0 = ok, >0 = cudaError_t, <0 = argument/setup error).  ``call`` raises on non-zero so a missing
or failing native path is loud: there is no silent PyTorch fallback on a GPU box.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB: ctypes.CDLL | None = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libbrain_b200.so"

#: number of native kernel launches issued through :func:`call` (bench.py reports it)
launch_count = 0

_ERR_NAMES = {
    1: "TMA producer timed out waiting for a free shared-memory slot",
    2: "MMA issuer timed out waiting for TMA data",
    3: "MMA issuer timed out waiting for a free TMEM accumulator",
    4: "epilogue timed out waiting for the accumulator",
    5: "softmax warps timed out",
    6: "peer flag never arrived",
    7: "bad argument seen on device",
}


class NativeError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not _LIB_PATH.exists():
            if os.environ.get("BRAIN_B200_NO_AUTOBUILD") == "1":
                raise NativeError(f"native library missing: {_LIB_PATH} (run __graft_entry__.build())")
            from .. import _build
            _build.build_cuda()
        _LIB = ctypes.CDLL(str(_LIB_PATH))
    return _LIB


def available() -> bool:
    """True when the kernels can run: library present (or buildable) and a CUDA device visible."""
    return torch.cuda.is_available()


def _conv(a):
    if isinstance(a, torch.Tensor):
        return ctypes.c_void_p(a.data_ptr())
    if a is None:
        return ctypes.c_void_p(0)
    if isinstance(a, bool):
        return ctypes.c_int(int(a))
    if isinstance(a, int):
        return ctypes.c_int(a)
    if isinstance(a, float):
        return ctypes.c_float(a)
    return a


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


_Tensor = torch.Tensor
#: per-launcher (function, argument count); the argument types are declared on the first call so
#: that later calls hand plain ints / floats / addresses to ctypes instead of building one ctypes
#: object per argument (that conversion was two thirds of the host cost of a launch)
_FN: dict = {}


def _argtype(a):
    if a is None or isinstance(a, _Tensor):
        return ctypes.c_void_p
    if isinstance(a, (bool, int)):
        return ctypes.c_int
    if isinstance(a, float):
        return ctypes.c_float
    if isinstance(a, ctypes.Array):
        return ctypes.c_void_p
    return type(a)      # an explicit ctypes scalar: c_long, c_uint, c_double, c_void_p


def _bind(name: str, args):
    fn = getattr(lib(), "bb_" + name)
    fn.restype = ctypes.c_int
    fn.argtypes = [_argtype(a) for a in args]
    _FN[name] = (fn, len(args))
    return _FN[name]


def call(name: str, *args) -> None:
    """Launch ``bb_<name>``; tensors become device pointers, ints c_int, floats c_float.
    Pass ``ctypes.c_long(x)`` explicitly for 64-bit parameters (and always the same kind of value
    for a given parameter: the C types are fixed by the first call)."""
    global launch_count
    ent = _FN.get(name)
    if ent is None:
        ent = _bind(name, args)
    fn, n = ent
    if n != len(args):
        raise NativeError(f"bb_{name}: {len(args)} arguments, first call had {n}")
    rc = fn(*[a.data_ptr() if isinstance(a, _Tensor) else a for a in args])
    launch_count += 1
    if rc != 0:
        raise NativeError(f"bb_{name} failed with code {rc}")


def read_error(clear: bool = True) -> int:
    """Synchronise and return the device error word (0 = no kernel reported a bounded-wait timeout)."""
    return int(lib().bb_read_error(ctypes.c_int(1 if clear else 0)))


def check_error() -> None:
    code = int(_error_source()) if _error_source is not None else read_error(True)
    if code != 0:
        raise NativeError(f"device error {code}: {_ERR_NAMES.get(code, 'unknown')}")


#: test seam: a callable returning an error code replaces the native poll/read (CPU tests)
_error_source = None


def poll_error() -> None:
    """Non-blocking check of the device error word, made once per step by the trainers and the
    serving engine.  Each call harvests the asynchronous copy the previous call enqueued and
    enqueues a new one on the current stream, so a bounded wait that ran out inside a kernel of
    step ``n`` raises :class:`NativeError` at step ``n + 1`` without a device synchronisation."""
    if _error_source is not None:
        code = int(_error_source())
    else:
        fn = lib().bb_poll_error
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p]
        code = int(fn(stream_ptr()))
    if code > 0:
        if _error_source is None:
            read_error(True)
        raise NativeError(f"device error {code}: {_ERR_NAMES.get(code, 'unknown')}")


def L(x: int) -> ctypes.c_long:
    return ctypes.c_long(int(x))
