"""The allocation-free sum-of-squares entry point, called through its exported C symbol.

Some users of the kernel library may not allocate device memory at the point where they need a
gradient norm (an allocation-free region of their program, or a host that owns every byte of
device memory and only lends out input/output buffers).  ``bb_sumsq_noalloc`` serves them: its
per-block partial sums live in a 4 KiB array that is part of the library image, so the caller
passes only the input vector and one output float.  This test checks it against the regular
``bb_sumsq`` entry point (which takes a caller-provided scratch buffer) on two calls in a row —
the second call finds the first call's partial sums still in the shared scratch — and checks that
an oversized request is refused without launching anything.

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  It passes on its own in a fresh process as well as after the rest of the suite.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ELEMS = 1 << 28
ESIZE = -3
EARG = -1


def _lib():
    from brain_b200.ops import _cuda
    lib = _cuda.lib()
    fn = lib.bb_sumsq_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    ref = lib.bb_sumsq
    ref.restype = ctypes.c_int
    ref.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                    ctypes.c_void_p]
    return fn, ref


def test_noalloc_sumsq_matches_regular_entry_point_twice():
    fn, ref = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.manual_seed(0)
    # every buffer is created up front: the calls under test allocate nothing themselves
    inputs = [torch.randn(3_000_003, device=dev), 5.0 * torch.randn(1_234_568, device=dev)]
    outs = [torch.zeros(1, device=dev) for _ in inputs]
    wants = [torch.zeros(1, device=dev) for _ in inputs]
    scratch = torch.empty(1024, device=dev)
    for x, out in zip(inputs, outs):            # two calls in a row on the shared built-in scratch
        rc = fn(x.data_ptr(), x.numel(), out.data_ptr(), 0, stream)
        assert rc == 0, rc
    for x, want in zip(inputs, wants):
        rc = ref(x.data_ptr(), x.numel(), scratch.data_ptr(), want.data_ptr(), 0, stream)
        assert rc == 0, rc
    torch.cuda.synchronize()
    for x, out, want in zip(inputs, outs, wants):
        assert abs(out.item() - want.item()) <= 1e-5 * abs(want.item())
        exact = (x.double() ** 2).sum().item()
        assert abs(out.item() - exact) <= 1e-3 * exact
    # accumulate mode adds to what is already in `out`
    before = outs[0].item()
    rc = fn(inputs[0].data_ptr(), inputs[0].numel(), outs[0].data_ptr(), 1, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert abs(outs[0].item() - 2 * before) <= 1e-5 * abs(2 * before)


def test_noalloc_sumsq_rejects_oversized_input():
    fn, _ = _lib()
    dev = torch.device("cuda:0")
    x = torch.ones(16, device=dev)
    out = torch.full((1,), -7.0, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert fn(x.data_ptr(), MAX_ELEMS + 1, out.data_ptr(), 0, stream) == ESIZE
    assert fn(x.data_ptr(), -1, out.data_ptr(), 0, stream) == ESIZE
    torch.cuda.synchronize()
    assert out.item() == -7.0   # nothing was launched


def test_noalloc_sumsq_rejects_bad_pointers():
    fn, _ = _lib()
    dev = torch.device("cuda:0")
    x = torch.ones(64, device=dev)
    out = torch.full((1,), -7.0, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert fn(x.data_ptr() + 4, 16, out.data_ptr(), 0, stream) == EARG     # input not 16-byte aligned
    assert fn(x.data_ptr(), 16, None, 0, stream) == EARG                   # no output
    assert fn(None, 16, out.data_ptr(), 0, stream) == EARG                 # no input
    torch.cuda.synchronize()
    assert out.item() == -7.0   # nothing was launched
