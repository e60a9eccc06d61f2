"""Serving engine on the native kernels: paged decode == contiguous forward, int8 tracks bf16."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(weights="bf16", kv="bf16"):
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
    return QwenEngine(m, block_size=16, num_blocks=256, max_seq_len=512, max_prefill=128, weights=weights, kv_dtype=kv)


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


@pytest.mark.parametrize("hd,hq,hk", [(128, 8, 2), (64, 6, 2)])
def test_int8_kv_kernels_match_reference(hd, hq, hk):
    """kv_append_i8 == torch quantisation (row scale min(absmax, ceiling)/127); kv_gather_i8 returns
    the dequantised rows; paged_decode_i8 == fp32 attention over the dequantised cache."""
    from brain_b200.ops import reference as ref
    from brain_b200.ops._cuda import call, stream_ptr, check_error
    torch.manual_seed(2)
    bs, nb, n = 16, 40, 300
    k = torch.randn(n, hk * hd, device="cuda").bfloat16()
    v = (torch.randn(n, hk * hd, device="cuda") * 3).bfloat16()
    clip = torch.tensor([[2.5] * hk, [1e30] * hk], device="cuda")
    table = torch.randperm(nb)[:20].to("cuda", torch.int32)
    t = torch.arange(n, device="cuda")
    slots = (table[(t // bs).long()] * bs + (t % bs).int()).to(torch.int32)
    kc = torch.zeros(nb, hk, bs, hd, device="cuda", dtype=torch.int8)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(nb, hk, bs, device="cuda")
    vs = torch.zeros_like(ks)
    call("kv_append_i8", k, k.stride(0), v, v.stride(0), slots, kc, vc, ks, vs, clip, n, hk, hd, bs, stream_ptr())
    check_error()
    blk, off = (slots // bs).long(), (slots % bs).long()
    for x, pool, sc, ceil in ((k, kc, ks, 2.5), (v, vc, vs, 1e30)):
        xf = x.float().reshape(n, hk, hd)
        scale = xf.abs().amax(-1).clamp(max=ceil) / 127
        want = torch.clamp(torch.round(xf / scale[..., None]), -127, 127)
        got = pool[blk, :, off].float()
        assert torch.allclose(sc[blk, :, off], scale, rtol=1e-6, atol=0)
        assert (got - want).abs().max().item() <= 1.0     # round-half ties may differ by one step
        assert ((got - want).abs() > 0).float().mean().item() < 1e-3
    ok = torch.empty(n, hk * hd, device="cuda", dtype=torch.bfloat16)
    ov = torch.empty_like(ok)
    call("kv_gather_i8", kc, vc, ks, vs, table, ok, ov, n, hk, hd, bs, stream_ptr())
    check_error()
    dk = (kc[blk, :, off].float() * ks[blk, :, off][..., None]).reshape(n, -1)
    dv = (vc[blk, :, off].float() * vs[blk, :, off][..., None]).reshape(n, -1)
    assert torch.allclose(ok.float(), dk, rtol=1e-2, atol=1e-3) and torch.allclose(ov.float(), dv, rtol=1e-2, atol=1e-3)

    B = 3
    lens = [7, 129, 300]
    q = torch.randn(B, hq * hd, device="cuda").bfloat16()
    bts = table[None, :].expand(B, -1).contiguous()
    seqlens = torch.tensor(lens, device="cuda", dtype=torch.int32)
    for splits in (1, 3):
        out = torch.empty(B, hq * hd, device="cuda", dtype=torch.bfloat16)
        po = torch.empty(B * hq * splits * hd, device="cuda")
        pm = torch.empty(B * hq * splits * 2, device="cuda")
        call("paged_decode_i8", q, q.stride(0), kc, vc, ks, vs, bts, bts.shape[1], seqlens, out, out.stride(0),
             po, pm, B, hq, hk, hd, bs, splits, float(hd ** -0.5), stream_ptr())
        check_error()
        for b in range(B):
            S = lens[b]
            want = ref.attention(q[b].float().reshape(1, 1, hq, hd), dk[:S].reshape(1, S, hk, hd),
                                 dv[:S].reshape(1, S, hk, hd), causal=False)
            err = ((out[b].float() - want.reshape(-1)).norm() / want.norm()).item()
            assert err < 1e-2, (splits, b, err)


def test_engine_int8_kv_tracks_bf16_kv():
    from brain_b200.ops import _cuda
    base, e8 = _engine(), _engine(kv="int8")
    toks = np.arange(5, 205, dtype=np.int32)
    bt = np.arange(base.max_blocks, dtype=np.int32)
    outs = []
    for e in (base, e8):
        e.prefill_chunk(toks[:128], 0, bt, False)
        e.prefill_chunk(toks[128:], 128, bt, True)
        _, c = e.decode(np.array([7], dtype=np.int32), np.array([200], dtype=np.int32), bt[None, :], greedy=False)
        outs.append(dict(c[0]))
    _cuda.check_error()
    common = set(outs[0]) & set(outs[1])
    assert len(common) >= 32
    spread = max(outs[0].values()) - min(outs[0].values())
    assert max(abs(outs[0][t] - outs[1][t]) for t in common) < 0.1 * spread


def _same_candidates(ca, cb):
    """Top-k candidate lists agree: the same tokens apart from ties at the tail of the list, and
    logits within a couple of bf16 steps."""
    a, b = dict(ca), dict(cb)
    common = set(a) & set(b)
    assert len(common) >= len(a) - 4
    spread = max(a.values()) - min(a.values())
    assert max(abs(a[t] - b[t]) for t in common) <= 0.02 * spread + 1e-3
    assert max(a, key=a.get) == max(b, key=b.get)


@pytest.mark.parametrize("weights,kv", [("bf16", "bf16"), ("int8", "int8")])
def test_native_forward_matches_python_path(weights, kv):
    """The native layer sequence issues the same kernels in the same order as the Python wrappers:
    prefill (fresh chunk, chunk with a past, packed chunks), eager decode and graph decode agree."""
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.ops import _cuda
    from brain_b200.serve.engine import QwenEngine
    cfg = QwenConfig(vocab=512, block_size=512, n_layers=3, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512)
    m = Qwen3(cfg).init_weights(3)
    with torch.no_grad():
        for p in m.parameters():
            p.mul_(3.0)
    m = m.to("cuda", torch.bfloat16)
    mk = lambda native, graphs: QwenEngine(m, block_size=16, num_blocks=128, max_seq_len=512, max_prefill=256,
                                           weights=weights, kv_dtype=kv, native=native, cuda_graphs=graphs)
    e_py, e_nat, e_graph = mk(False, False), mk(True, False), mk(True, True)
    assert e_py.native is None and e_nat.native is not None
    rng = np.random.default_rng(0)
    toks = rng.integers(0, 512, 200).astype(np.int32)
    bt0, bt1, bt2 = (np.arange(32, dtype=np.int32) + 32 * i for i in range(3))
    res = []
    for e in (e_py, e_nat, e_graph):
        r = {}
        e.prefill_chunk(toks[:128], 0, bt0, False)
        r["first"], r["cand"] = e.prefill_chunk(toks[128:], 128, bt0, True, greedy=False)
        items = [(toks[:70], 0, bt1, True, True), (toks[50:141], 0, bt2, True, True)]
        r["packed"] = [t for t, _ in e.prefill_batch(items)]
        r["verify"] = e.verify_chunk(toks[10:30], 200, bt0).tolist()
        tok = np.array([r["first"], r["packed"][0], r["packed"][1]], dtype=np.int32)
        pos = np.array([220, 70, 91], dtype=np.int32)
        bts = np.stack([bt0, bt1, bt2])
        out, _ = e.decode(tok, pos, bts, window=3, greedy=True)
        r["decode"] = out
        _, c = e.decode(np.array([5, 6, 7], dtype=np.int32), pos + 3, bts, window=1, greedy=False)
        r["dcand"] = c
        # one forward carrying a fresh prompt AND a decode row per running sequence gives what the
        # two separate forwards give (same inputs, so the pages are rewritten with the same values)
        bt3 = np.arange(32, dtype=np.int32) + 96
        nxt = np.array([8, 9, 10], dtype=np.int32)
        sep_first, _ = e.prefill_chunk(toks[:60], 0, bt3, True)
        sep_dec, _ = e.decode(nxt, pos + 4, bts, window=1, greedy=True)
        mres, mdec, mc = e.mixed_step([(toks[:60], 0, bt3, True, True)], nxt, pos + 4, bts, True)
        assert mc is None and mres[0][0] == sep_first and mdec == sep_dec
        r["mixed"] = (mres[0][0], mdec)
        res.append(r)
    _cuda.check_error()
    py, nat, gr = res
    assert e_graph.graph_replays >= 1
    for other in (nat, gr):
        assert other["first"] == py["first"] and other["packed"] == py["packed"] and other["verify"] == py["verify"]
        assert other["decode"] == py["decode"] and other["mixed"] == py["mixed"]
        _same_candidates(py["cand"], other["cand"])
        for ca, cb in zip(py["dcand"], other["dcand"]):
            _same_candidates(ca, cb)


def test_w4a8_unpack_kernel_and_engine():
    """The nibble-expansion kernel is exact against the PyTorch restatement, and the W4A8 engine
    (4-bit weights expanded per projection into the shared int8 scratch, CUDA-graph decode included)
    picks tokens whose logits the bf16 engine ranks close to its own best."""
    from brain_b200.ops import _cuda, functional as F
    from brain_b200.serve.quantize import quantize_weight_q4
    torch.manual_seed(0)
    w = torch.randn(96, 256)
    words, sw = quantize_weight_q4(w)
    want = F.unpack_q4(words)                                   # CPU restatement
    got = F.unpack_q4(words.cuda())
    assert torch.equal(got.cpu(), want) and int(want.abs().max()) <= 7
    # the W4A8 engine on the GPU against the same engine on the CPU backend (same 4-bit weights and
    # the same dynamic int8 activations; bf16 vs fp32 arithmetic around them)
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.serve.engine import QwenEngine
    cfg = QwenConfig(vocab=512, block_size=512, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512)
    m = Qwen3(cfg).init_weights(3)
    with torch.no_grad():
        for p in m.parameters():
            p.copy_((p * 3.0).bfloat16().float())              # values both dtypes hold exactly
    mk = lambda mod: QwenEngine(mod, block_size=16, num_blocks=64, max_seq_len=512, max_prefill=128, weights="int4")
    e_cpu = mk(m)
    import copy
    e4 = mk(copy.deepcopy(m).to("cuda", torch.bfloat16))
    assert e4.native is None and all(l["qkv"].int4 for l in e4.layers)
    assert torch.equal(e4.layers[0]["qkv"].words.cpu(), e_cpu.layers[0]["qkv"].words)
    toks = np.random.RandomState(0).randint(0, 512, 48).astype(np.int32)
    bt = np.arange(32, dtype=np.int32)
    for e in (e4, e_cpu):
        e.prefill_chunk(toks, 0, bt, True)
    nxt = np.array([7], dtype=np.int32)
    pos = np.array([48], dtype=np.int32)
    _, c4 = e4.decode(nxt, pos, bt[None, :], greedy=False)
    _, cc = e_cpu.decode(nxt, pos, bt[None, :], greedy=False)
    d4, dc = dict(c4[0]), dict(cc[0])
    common = set(d4) & set(dc)
    spread = max(dc.values()) - min(dc.values())
    assert len(common) >= 24, len(common)
    worst = max(abs(d4[t] - dc[t]) for t in common)
    assert worst < 0.1 * spread, (worst, spread)
    g1, _ = e4.decode(nxt, pos, bt[None, :], greedy=True)       # graph path: same scratch, same result twice
    g2, _ = e4.decode(nxt, pos, bt[None, :], greedy=True)
    assert g1 == g2
    _cuda.check_error()
