"""The bounds-checking library (index-driven kernels compiled with -DBB_DEBUG_BOUNDS): an index that
data supplies and that lies outside its extent is RECORDED (error word = 8) and the access is
skipped, so nothing faults and the context stays usable.  The tests call that library only; if it is
not there they are skipped, never redirected to the production library."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_BOUNDS = 8
SENT = 123.0


def _lib():
    import brain_b200
    path = os.path.join(os.path.dirname(brain_b200.__file__), "_lib", "libbrain_b200_bounds.so")
    if not os.path.exists(path):
        pytest.skip("bounds-checking library not built")
    lib = ctypes.CDLL(path)
    lib.bb_read_error.restype = ctypes.c_int
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _read_and_clear(lib):
    torch.cuda.synchronize()
    return int(lib.bb_read_error(1))    # read and clear


def test_embedding_gather_records_a_token_outside_the_vocabulary_and_skips_it():
    lib = _lib()
    vocab, d, n = 50, 64, 6
    emb = torch.randn(vocab, d, device="cuda").bfloat16()
    tok = torch.tensor([3, 49, 0, 7, 50, -2], device="cuda", dtype=torch.int32)   # two bad ids
    out = torch.full((n, d), SENT, device="cuda", dtype=torch.bfloat16)
    assert _read_and_clear(lib) == 0
    rc = lib.bb_embed_fwd(_p(tok), _p(emb), None, 1, _p(out), ctypes.c_long(n), d, vocab, _stream())
    assert rc == 0
    assert _read_and_clear(lib) == ERR_BOUNDS
    assert torch.equal(out[:4], emb[tok[:4].long()])
    assert bool((out[4:] == SENT).all()), "rows of out-of-range tokens must be left untouched"
    # in range: no error, and the library is still usable after the recorded violation
    tok2 = torch.tensor([1, 2, 3, 4, 5, 6], device="cuda", dtype=torch.int32)
    rc = lib.bb_embed_fwd(_p(tok2), _p(emb), None, 1, _p(out), ctypes.c_long(n), d, vocab, _stream())
    assert rc == 0 and _read_and_clear(lib) == 0
    assert torch.equal(out, emb[tok2.long()])


def test_cross_entropy_records_a_target_past_the_vocabulary():
    lib = _lib()
    n, V = 4, 64
    logits = torch.randn(n, V, device="cuda").bfloat16()
    loss = torch.full((n,), SENT, device="cuda")
    lse = torch.empty(n, device="cuda")
    tgt = torch.tensor([5, -1, 63, 64], device="cuda", dtype=torch.int32)   # -1 = ignore (legal), 64 = caller error
    rc = lib.bb_cross_entropy(_p(logits), ctypes.c_long(V), _p(tgt), _p(loss), _p(lse), n, V, 0, None,
                              ctypes.c_float(1.0), _stream())
    assert rc == 0
    assert _read_and_clear(lib) == ERR_BOUNDS
    want = torch.nn.functional.cross_entropy(logits[[0, 2]].float(), tgt[[0, 2]].long(), reduction="none")
    assert torch.allclose(loss[[0, 2]], want, rtol=2e-3, atol=2e-3)
    assert float(loss[1]) == 0.0 and float(loss[3]) == 0.0
    tgt_ok = torch.tensor([5, -1, 63, 0], device="cuda", dtype=torch.int32)
    rc = lib.bb_cross_entropy(_p(logits), ctypes.c_long(V), _p(tgt_ok), _p(loss), _p(lse), n, V, 0, None,
                              ctypes.c_float(1.0), _stream())
    assert rc == 0 and _read_and_clear(lib) == 0


def test_moe_gather_records_a_pair_that_names_no_token():
    lib = _lib()
    n, d, k, E = 8, 64, 2, 2
    x = torch.randn(n, d, device="cuda").bfloat16()
    rows = 128
    pair_of_pos = torch.full((rows,), -1, device="cuda", dtype=torch.int32)
    pair_of_pos[0] = 3            # token 1
    pair_of_pos[1] = n * k + 4    # past the last token: would read through a null base pointer
    pair_of_pos[2] = 15           # token 7
    offsets = torch.tensor([0, 64, 128], device="cuda", dtype=torch.int32)
    xp = torch.full((rows, d), SENT, device="cuda", dtype=torch.bfloat16)
    ptrs = (ctypes.c_uint64 * 1)(x.data_ptr())
    rc = lib.bb_moe_gather(ptrs, 1, n, _p(pair_of_pos), None, k, _p(xp), _p(offsets), E, d, rows, _stream())
    assert rc == 0
    assert _read_and_clear(lib) == ERR_BOUNDS
    assert torch.equal(xp[0], x[1]) and torch.equal(xp[2], x[7])
    assert bool((xp[1] == SENT).all()), "the row of the bad pair must be left untouched"
    assert bool((xp[3:] == 0).all()), "padding rows are zero-filled"
