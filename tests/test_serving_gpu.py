"""Serving engine on the native kernels: paged decode == contiguous forward, int8 tracks bf16."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(weights="bf16"):
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.serve.engine import QwenEngine
    cfg = QwenConfig(vocab=512, block_size=512, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2,
                     head_dim=64, d_ff=512)
    m = Qwen3(cfg).init_weights(3)
    with torch.no_grad():
        for p in m.parameters():
            p.mul_(3.0)
    m = m.to("cuda", torch.bfloat16)
    return QwenEngine(m, block_size=16, num_blocks=256, max_seq_len=512, max_prefill=128, weights=weights)


def test_paged_kv_kernels_roundtrip():
    from brain_b200.ops._cuda import call, stream_ptr, check_error
    torch.manual_seed(0)
    hk, hd, bs, nb = 2, 64, 16, 8
    kc = torch.zeros(nb, hk, bs, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    n = 40
    k = torch.randn(n, hk * hd, device="cuda").bfloat16()
    v = torch.randn(n, hk * hd, device="cuda").bfloat16()
    table = torch.tensor([5, 2, 7, 0, 1, 3, 4, 6], device="cuda", dtype=torch.int32)
    pos = torch.arange(n, device="cuda")
    slots = (table[(pos // bs).long()] * bs + pos % bs).to(torch.int32)
    call("kv_append", k, k.stride(0), v, v.stride(0), slots, kc, vc, n, hk, hd, bs, stream_ptr())
    ok = torch.empty(n, hk * hd, device="cuda", dtype=torch.bfloat16)
    ov = torch.empty_like(ok)
    call("kv_gather", kc, vc, table, ok, ov, n, hk, hd, bs, stream_ptr())
    check_error()
    assert torch.equal(ok, k) and torch.equal(ov, v)


def test_paged_decode_matches_reference_attention():
    from brain_b200.ops import reference as ref
    from brain_b200.ops._cuda import call, stream_ptr, check_error
    torch.manual_seed(1)
    B, hq, hk, hd, bs = 3, 8, 2, 128, 16
    lens = [5, 130, 257]
    max_blocks = 20
    nb = 64
    kc = torch.randn(nb, hk, bs, hd, device="cuda").bfloat16()
    vc = torch.randn(nb, hk, bs, hd, device="cuda").bfloat16()
    perm = torch.randperm(nb)[:B * max_blocks].reshape(B, max_blocks).to("cuda", torch.int32)
    q = torch.randn(B, hq * hd, device="cuda").bfloat16()
    seqlens = torch.tensor(lens, device="cuda", dtype=torch.int32)
    for splits in (1, 4):
        out = torch.empty(B, hq * hd, device="cuda", dtype=torch.bfloat16)
        po = torch.empty(B * hq * splits * hd, device="cuda")
        pm = torch.empty(B * hq * splits * 2, device="cuda")
        call("paged_decode", q, q.stride(0), kc, vc, perm, max_blocks, seqlens, out, out.stride(0),
             po, pm, B, hq, hk, hd, bs, splits, float(hd ** -0.5), stream_ptr())
        check_error()
        for b in range(B):
            S = lens[b]
            t = torch.arange(S, device="cuda")
            blk = perm[b][(t // bs).long()].long()
            kk = kc[blk, :, t % bs].float().reshape(1, S, hk, hd)
            vv = vc[blk, :, t % bs].float().reshape(1, S, hk, hd)
            want = ref.attention(q[b].float().reshape(1, 1, hq, hd), kk, vv, causal=False)
            err = ((out[b].float() - want.reshape(-1)).norm() / want.norm()).item()
            assert err < 2e-2, (splits, b, err)


def test_engine_paged_decode_matches_contiguous_forward():
    from brain_b200.ops import _cuda
    from brain_b200.serve.scheduler import Scheduler
    eng = _engine()
    prompts = [list(range(3, 40)), [9, 8, 7], list(range(100, 300))]
    s = Scheduler(eng, max_batch=4, window=4)
    ids = [s.submit(p, 8) for p in prompts]
    s.run_until_idle()
    _cuda.check_error()
    for rid, p in zip(ids, prompts):
        got = s.tokens_of(rid)
        assert len(got) == 8
        # teacher-forced check: every generated token is the argmax (or within bf16 noise of it)
        toks = list(p) + got
        logits = eng.logits_all(toks)
        for i, t in enumerate(got):
            row = logits[len(p) - 1 + i]
            assert row[t] >= row.max() - 0.05 * row.abs().max(), (rid, i)


def test_engine_int8_tracks_bf16():
    eng, eng8 = _engine(), _engine("int8")
    toks = list(range(5, 200))
    a, b = eng.logits_all(toks), eng8.logits_all(toks)
    rel = ((a - b).norm() / a.norm()).item()
    assert rel < 0.2, rel
    assert eng8.weight_bytes() < 0.7 * eng.weight_bytes()
