"""Every in-kernel wait on a peer is bounded: when the flag never arrives the kernel records
``peer flag never arrived`` in the device error word, releases what it holds (tensor memory
included) and returns, and the CUDA context stays usable.

The failure is made without a second GPU and without faulting anything: each kernel is launched as
rank 0 of a world of 2 whose "peer" buffers are ordinary local buffers that nothing ever writes, with
a wait limit of 50 ms.  A plain GEMM afterwards checks that the context and the tensor memory are
intact."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

WAIT_S = 0.05
ERR_WAIT_PEER = 6


def _u64(*ptrs):
    return (ctypes.c_uint64 * len(ptrs))(*ptrs)


def _gemm_still_works(dev):
    from brain_b200.ops import functional as F
    from brain_b200.ops import _cuda
    a = torch.randn(256, 128, device=dev, dtype=torch.bfloat16)
    w = torch.randn(192, 128, device=dev, dtype=torch.bfloat16)
    y = F.linear(a, w)
    torch.cuda.synchronize()
    ref = a.float() @ w.float().t()
    assert float((y.float() - ref).abs().max()) < 0.5
    assert _cuda.read_error(True) == 0


def test_symm_barrier_wait_runs_out():
    from brain_b200.ops import _cuda
    from brain_b200.ops._cuda import call, stream_ptr
    dev = torch.device("cuda:0")
    assert _cuda.read_error(True) == 0
    mine = torch.zeros(2, device=dev, dtype=torch.int64)
    peer = torch.zeros(2, device=dev, dtype=torch.int64)        # the absent rank's flag words
    call("symm_barrier", _u64(mine.data_ptr(), peer.data_ptr()), 0, 2, ctypes.c_uint(1),
         ctypes.c_double(WAIT_S), stream_ptr())
    torch.cuda.synchronize()
    assert _cuda.read_error(True) == ERR_WAIT_PEER
    assert int(peer[0]) == 1 and int(mine[1]) == 0              # I published; the peer never did
    _gemm_still_works(dev)


def test_two_shot_allreduce_wait_runs_out_and_leaves_the_result_untouched():
    from brain_b200.ops import _cuda
    from brain_b200.ops._cuda import L, call, stream_ptr
    dev = torch.device("cuda:0")
    n = 1 << 14
    x = torch.ones(n, device=dev, dtype=torch.bfloat16)
    stage = [torch.zeros(n, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    result = [torch.full((n,), -3.0, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    sig = [torch.zeros(2, device=dev, dtype=torch.int64) for _ in range(2)]
    state = torch.zeros(4, device=dev, dtype=torch.int32)
    call("tp_allreduce2", _u64(*[t.data_ptr() for t in stage]), _u64(*[t.data_ptr() for t in result]),
         _u64(*[t.data_ptr() for t in sig]), x, L(n), 0, 2, state, state[1:], ctypes.c_double(WAIT_S),
         stream_ptr())
    torch.cuda.synchronize()
    assert _cuda.read_error(True) == ERR_WAIT_PEER
    assert float(result[0].float().max()) == -3.0               # no partial sum was published
    _gemm_still_works(dev)


def test_allgather_gemm_wait_runs_out_and_frees_tensor_memory():
    """All-gather -> GEMM with a peer whose shard never becomes ready: the data movers and the TMA
    producer give up, the MMA and epilogue warps follow through their own bounded waits, TMEM is
    deallocated (the following GEMM allocates it again)."""
    from brain_b200.ops import _cuda
    from brain_b200.ops._cuda import call, stream_ptr
    dev = torch.device("cuda:0")
    rows, K, N = 128, 128, 128
    full = torch.zeros(2 * rows, K, device=dev, dtype=torch.bfloat16)
    shard = [torch.ones(rows, K, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    w = torch.ones(N, K, device=dev, dtype=torch.bfloat16)
    y = torch.zeros(2 * rows, N, device=dev, dtype=torch.bfloat16)
    flags = torch.zeros(16, device=dev, dtype=torch.int32)
    sig = [torch.zeros(4, device=dev, dtype=torch.int64) for _ in range(2)]
    counter = torch.zeros(4, device=dev, dtype=torch.int32)
    call("gemm_bf16_tp", 1, full, w, y, 2 * rows, N, K, K, K, N, 0, 2, rows,
         _u64(*[t.data_ptr() for t in shard]), flags, 4, _u64(*[t.data_ptr() for t in sig]),
         ctypes.c_uint(1), None, counter, ctypes.c_double(WAIT_S), stream_ptr())
    torch.cuda.synchronize()
    assert _cuda.read_error(True) != 0
    # this rank's own rows were gathered and multiplied; the absent peer's rows were not
    assert float(y[:rows].float().min()) == K and float(y[rows:].float().abs().max()) == 0.0
    _gemm_still_works(dev)
