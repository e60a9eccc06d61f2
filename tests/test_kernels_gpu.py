"""sm_100a kernels vs the plain PyTorch fp32 reference of the same op (small + odd shapes)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from brain_b200.ops import _cuda, functional as F, reference as ref  # noqa: E402


def dev():
    return torch.device("cuda:0")


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.fixture(autouse=True)
def _check_device_error():
    yield
    _cuda.check_error()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 1024), (300, 200, 136), (4096, 1024, 1024),
                                   (1024, 3072, 1024), (64, 64, 64), (129, 1000, 72)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_bf16(M, N, K, a_mn, b_mn):
    torch.manual_seed(M + N + K)
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operand needs a 16-byte row pitch")
    a = torch.randn(M, K, device=dev()).bfloat16()
    b = torch.randn(N, K, device=dev()).bfloat16()
    want = a.float() @ b.float().t()
    aa = a.t().contiguous() if a_mn else a
    bb = b.t().contiguous() if b_mn else b
    got = F.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn)
    assert rel_err(got, want) < 1e-2
    got32 = F.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert rel_err(got32, want) < 2e-3


def _gemm_pair(aa, bb, out, a_mn, b_mn, out_mode, alpha=1.0, split_k=1):
    """The CTA-pair (cta_group::2) kernel through its own entry point."""
    from brain_b200.ops._cuda import call, stream_ptr
    M, N = out.shape
    K = aa.shape[0] if a_mn else aa.shape[1]
    call("gemm_bf16_pair", aa, bb, out, M, N, K, aa.stride(0), bb.stride(0), out.stride(0), int(a_mn), int(b_mn),
         out_mode, float(alpha), split_k, 0, stream_ptr())


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (300, 520, 136), (4096, 1024, 1024),
                                   (264, 1000, 72)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_pair_kernel(M, N, K, a_mn, b_mn):
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operand needs a 16-byte row pitch")
    torch.manual_seed(M + N + K + 1)
    a = torch.randn(M, K, device=dev()).bfloat16()
    b = torch.randn(N, K, device=dev()).bfloat16()
    want = a.float() @ b.float().t()
    aa = a.t().contiguous() if a_mn else a
    bb = b.t().contiguous() if b_mn else b
    # bf16 output inside a canary frame: partial tiles at the right and bottom edges must be clipped
    pad = torch.full((M + 2, N + 16), 7.0, device=dev(), dtype=torch.bfloat16)
    out = pad[1:M + 1, 8:8 + N]
    _gemm_pair(aa, bb, out, a_mn, b_mn, 0)
    assert rel_err(out, want) < 1e-2
    assert (pad[0] == 7).all() and (pad[-1] == 7).all() and (pad[:, :8] == 7).all() and (pad[:, 8 + N:] == 7).all()
    out32 = torch.empty(M, N, device=dev())
    _gemm_pair(aa, bb, out32, a_mn, b_mn, 1, alpha=0.5)
    assert rel_err(out32, 0.5 * want) < 2e-3


def test_gemm_pair_accumulate_split_k_and_dispatch():
    torch.manual_seed(5)
    M, N, K = 1024, 512, 8192                      # a weight-gradient shape: long K, both operands [K][rows]
    a = torch.randn(K, M, device=dev()).bfloat16()
    b = torch.randn(K, N, device=dev()).bfloat16()
    base = torch.randn(M, N, device=dev())
    want = base + a.float().t() @ b.float()
    for sk in (1, 4):
        out = base.clone()
        _gemm_pair(a, b, out, True, True, 2, split_k=sk)
        assert rel_err(out, want) < 2e-3
    # the public op picks the pair kernel for large plain GEMMs; same numbers either way
    x = torch.randn(8192, 1024, device=dev()).bfloat16()
    w = torch.randn(4096, 1024, device=dev()).bfloat16()
    n0 = _cuda.launch_count
    y = F.gemm(x, w)
    assert _cuda.launch_count == n0 + 1
    assert rel_err(y, x.float() @ w.float().t()) < 1e-2


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_widths_and_accumulate(bn):
    torch.manual_seed(0)
    M, N, K = 640, 768, 512
    a = torch.randn(M, K, device=dev()).bfloat16()
    b = torch.randn(N, K, device=dev()).bfloat16()
    base = torch.randn(M, N, device=dev())
    out = base.clone()
    F.gemm(a, b, out=out, accumulate=True, bn=bn)
    want = base + a.float() @ b.float().t()
    assert rel_err(out, want) < 2e-3
    bias = torch.randn(N, device=dev())
    got = F.gemm(a, b, bias=bias, alpha=0.5, bn=bn)
    assert rel_err(got, 0.5 * (a.float() @ b.float().t()) + bias) < 1e-2


def test_gemm_strided_views_and_canaries():
    torch.manual_seed(1)
    M, N, K = 200, 328, 256
    big = torch.randn(M, K + 64, device=dev()).bfloat16()
    a = big[:, 32:32 + K]
    w = torch.randn(N, K, device=dev()).bfloat16()
    pad = torch.full((M + 2, N + 16), 7.0, device=dev(), dtype=torch.bfloat16)
    out = pad[1:M + 1, 8:8 + N]
    F.gemm(a, w, out=out)
    assert rel_err(out, a.float() @ w.float().t()) < 1e-2
    assert (pad[0] == 7).all() and (pad[-1] == 7).all()
    assert (pad[:, :8] == 7).all() and (pad[:, 8 + N:] == 7).all()


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 1024), (70, 200, 384), (512, 1536, 4096),
                                   (300, 520, 400), (1024, 768, 4096)])   # the last four run on CTA pairs
def test_gemm_i8(M, N, K):
    torch.manual_seed(2)
    x = torch.randn(M, K, device=dev())
    w = torch.randn(N, K, device=dev()) * 0.05
    xq, sx = ref.quant_rows(x)
    wq, sw = ref.quant_rows(w)
    want = (xq.float() @ wq.float().t()) * sx[:, None] * sw[None, :]
    got = F.gemm_i8(xq, wq, sx, sw)
    assert rel_err(got, want) < 1e-2
    assert rel_err(got, x @ w.t()) < 5e-2
    # output inside a sentinel frame: partial tiles at the right and bottom edges must be clipped
    pad = torch.full((M + 2, N + 16), 7.0, device=dev(), dtype=torch.bfloat16)
    out = pad[1:M + 1, 8:8 + N]
    F.gemm_i8(xq, wq, sx, sw, out=out)
    assert rel_err(out, want) < 1e-2
    assert (pad[0] == 7).all() and (pad[-1] == 7).all()
    assert (pad[:, :8] == 7).all() and (pad[:, 8 + N:] == 7).all()


def test_linear_autograd_matches_reference():
    torch.manual_seed(3)
    x = torch.randn(4, 96, 256, device=dev()).bfloat16().requires_grad_()
    w = torch.randn(384, 256, device=dev()).bfloat16().requires_grad_()
    b = torch.randn(384, device=dev()).bfloat16().requires_grad_()
    y = F.linear(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = ref.linear(xr, wr, br)
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2
    assert rel_err(x.grad, xr.grad) < 1e-2
    assert rel_err(w.grad, wr.grad) < 1e-2
    assert rel_err(b.grad, br.grad) < 1e-2


def test_linear_main_grad_accumulates():
    torch.manual_seed(4)
    x = torch.randn(512, 128, device=dev()).bfloat16().requires_grad_()
    w = torch.randn(256, 128, device=dev()).bfloat16().requires_grad_()
    w.main_grad = torch.ones(256, 128, device=dev())
    dy = torch.randn(512, 256, device=dev()).bfloat16()
    F.linear(x, w).backward(dy)
    assert w.grad is None
    assert rel_err(w.main_grad, 1 + dy.float().t() @ x.detach().float()) < 2e-3


@pytest.mark.parametrize("rows,d", [(37, 1024), (1000, 64), (5, 5120), (4096, 768)])
def test_rmsnorm(rows, d):
    torch.manual_seed(5)
    x = torch.randn(rows, d, device=dev()).bfloat16().requires_grad_()
    r = torch.randn(rows, d, device=dev()).bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(d, device=dev())).bfloat16().requires_grad_()
    y, h = F.rmsnorm(x, w, 1e-6, residual=r)
    dy, dh = torch.randn_like(y), torch.randn_like(h)
    (y * dy).sum().backward(retain_graph=True)
    (h * dh).sum().backward()
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    hr = (xr + rr)
    yr = ref.rmsnorm(hr, wr, 1e-6)
    ((yr * dy.float()).sum() + (hr * dh.float()).sum()).backward()
    assert rel_err(y, yr) < 1e-2 and rel_err(h, hr) < 1e-2
    assert rel_err(x.grad, xr.grad) < 2e-2
    assert rel_err(r.grad, rr.grad) < 2e-2
    assert rel_err(w.grad, wr.grad) < 2e-2
    y2 = F.rmsnorm(x.detach(), w.detach(), 1e-6)
    assert rel_err(y2, ref.rmsnorm(x.detach().float(), w.detach().float())) < 1e-2


@pytest.mark.parametrize("rows,d", [(33, 768), (512, 64)])
def test_layernorm(rows, d):
    torch.manual_seed(6)
    x = torch.randn(rows, d, device=dev()).bfloat16().requires_grad_()
    g = (1 + 0.1 * torch.randn(d, device=dev())).bfloat16().requires_grad_()
    b = (0.1 * torch.randn(d, device=dev())).bfloat16().requires_grad_()
    y = F.layernorm(x, g, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, gr, br = (t.detach().float().requires_grad_() for t in (x, g, b))
    yr = ref.layernorm(xr, gr, br)
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2
    assert rel_err(x.grad, xr.grad) < 2e-2
    assert rel_err(g.grad, gr.grad) < 2e-2
    assert rel_err(b.grad, br.grad) < 2e-2


@pytest.mark.parametrize("hd,hq,hk,extra", [(128, 4, 2, 256), (64, 6, 2, 128), (128, 2, 2, 0)])
@pytest.mark.parametrize("norm", [True, False])
def test_qknorm_rope(hd, hq, hk, extra, norm):
    torch.manual_seed(7)
    n = 77
    width = (hq + hk) * hd + extra
    qkv = torch.randn(n, width, device=dev()).bfloat16().requires_grad_()
    wq = (1 + 0.1 * torch.randn(hd, device=dev())).bfloat16().requires_grad_() if norm else None
    wk = (1 + 0.1 * torch.randn(hd, device=dev())).bfloat16().requires_grad_() if norm else None
    cos, sin = ref.rope_tables(128, hd, 1e6, device=dev())
    pos = torch.randint(0, 128, (n,), device=dev(), dtype=torch.int32)
    out = F.qknorm_rope(qkv, wq, wk, cos, sin, pos, hq, hk, hd)
    do = torch.randn_like(out)
    out.backward(do)
    qr = qkv.detach().float().requires_grad_()
    wqr = wq.detach().float().requires_grad_() if norm else None
    wkr = wk.detach().float().requires_grad_() if norm else None
    outr = ref.qknorm_rope(qr[:, :(hq + hk) * hd], wqr, wkr, cos, sin, pos.long(), hq, hk, hd)
    outr.backward(do.float())
    assert rel_err(out, outr) < 1e-2
    assert rel_err(qkv.grad, qr.grad) < 2e-2
    if norm:
        assert rel_err(wq.grad, wqr.grad) < 2e-2
        assert rel_err(wk.grad, wkr.grad) < 2e-2


def test_swiglu_gelu_embedding():
    torch.manual_seed(8)
    gu = torch.randn(130, 2 * 96, device=dev()).bfloat16().requires_grad_()
    h = F.swiglu(gu)
    dh = torch.randn_like(h)
    h.backward(dh)
    gr = gu.detach().float().requires_grad_()
    hr = ref.swiglu(gr)
    hr.backward(dh.float())
    assert rel_err(h, hr) < 1e-2 and rel_err(gu.grad, gr.grad) < 2e-2

    x = torch.randn(50, 64, device=dev()).bfloat16().requires_grad_()
    y = F.gelu(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = ref.gelu_tanh(xr)
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2 and rel_err(x.grad, xr.grad) < 2e-2

    emb = torch.randn(100, 64, device=dev()).bfloat16().requires_grad_()
    pos = torch.randn(16, 64, device=dev()).bfloat16().requires_grad_()
    tok = torch.randint(0, 100, (3, 16), device=dev())
    e = F.embedding(tok, emb, pos, 16)
    de = torch.randn_like(e)
    e.backward(de)
    er, pr = emb.detach().float().requires_grad_(), pos.detach().float().requires_grad_()
    want = er[tok] + pr[None]
    want.backward(de.float())
    assert rel_err(e, want) < 1e-2
    assert rel_err(emb.grad, er.grad) < 1e-2 and rel_err(pos.grad, pr.grad) < 1e-2


@pytest.mark.parametrize("n,V", [(9, 64), (130, 50304), (64, 151936)])
def test_cross_entropy(n, V):
    torch.manual_seed(9)
    logits = (3 * torch.randn(n, V, device=dev())).bfloat16().requires_grad_()
    tgt = torch.randint(0, V, (n,), device=dev())
    tgt[::5] = -1
    loss = F.cross_entropy(logits, tgt)
    loss.backward()
    lr = logits.detach().float().requires_grad_()
    lossr = ref.cross_entropy(lr, tgt)
    lossr.backward()
    assert abs(loss.item() - lossr.item()) < 2e-3 * max(1.0, abs(lossr.item()))
    assert rel_err(logits.grad, lr.grad) < 2e-2


def test_lm_head_ce_fused():
    torch.manual_seed(10)
    n, d, V = 300, 128, 1000
    x = (0.5 * torch.randn(n, d, device=dev())).bfloat16().requires_grad_()
    w = (0.1 * torch.randn(V, d, device=dev())).bfloat16().requires_grad_()
    tgt = torch.randint(0, V, (n,), device=dev())
    tgt[:7] = -1
    loss = F.lm_head_ce(x, w, tgt, chunk_rows=128)
    loss.backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lossr = ref.cross_entropy(ref.linear(xr, wr), tgt)
    lossr.backward()
    assert abs(loss.item() - lossr.item()) < 1e-2 * abs(lossr.item())
    assert rel_err(x.grad, xr.grad) < 3e-2
    assert rel_err(w.grad, wr.grad) < 3e-2


def test_lm_head_ce_weighted():
    """Per-position weights (both signs, zeros) in the fused LM head + CE."""
    torch.manual_seed(12)
    n, d, V = 260, 128, 1000
    x = (0.5 * torch.randn(n, d, device=dev())).bfloat16().requires_grad_()
    w = (0.1 * torch.randn(V, d, device=dev())).bfloat16().requires_grad_()
    tgt = torch.randint(0, V, (n,), device=dev())
    tgt[:5] = -1
    wts = torch.randn(n, device=dev())
    wts[10:20] = 0
    loss = F.lm_head_ce(x, w, tgt, chunk_rows=128, weights=wts)
    loss.backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    rows = ref.cross_entropy(ref.linear(xr, wr), tgt, reduction="none")
    lossr = (rows * wts).sum() / (tgt >= 0).sum()
    lossr.backward()
    assert abs(loss.item() - lossr.item()) < 2e-2 * max(abs(lossr.item()), 0.1)
    assert rel_err(x.grad, xr.grad) < 3e-2
    assert rel_err(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("rows,d", [(37, 1024), (300, 4096), (5, 2048), (64, 768)])
def test_fused_norm_and_swiglu_quant_are_bit_identical_to_the_unfused_pairs(rows, d):
    """rmsnorm_q8 == quant_rows(rmsnorm(...)) and swiglu_q8 == quant_rows(swiglu(...)), bit for bit,
    including the residual sum the norm writes out."""
    torch.manual_seed(21)
    x = torch.randn(rows, d, device=dev()).bfloat16()
    r = torch.randn(rows, d, device=dev()).bfloat16()
    w = (1 + 0.1 * torch.randn(d, device=dev())).bfloat16()
    s = _cuda.stream_ptr()
    for res in (None, r):
        if res is None:
            y = F.rmsnorm(x, w, 1e-6)
            h = None
        else:
            y, h = F.rmsnorm(x, w, 1e-6, residual=res)
        q_want, s_want = F.quant_rows(y)
        q = torch.empty(rows, d, device=dev(), dtype=torch.int8)
        sc = torch.empty(rows, device=dev())
        h_out = torch.empty_like(x) if res is not None else None
        _cuda.call("rmsnorm_q8", x, res, w, h_out, q, sc, rows, d, 1e-6, s)
        assert torch.equal(q, q_want) and torch.equal(sc, s_want)
        if res is not None:
            assert torch.equal(h_out, h)
    gu = torch.randn(rows, 2 * d, device=dev()).bfloat16()
    q_want, s_want = F.quant_rows(F.swiglu(gu))
    q = torch.empty(rows, d, device=dev(), dtype=torch.int8)
    sc = torch.empty(rows, device=dev())
    _cuda.call("swiglu_q8", gu, q, sc, rows, d, s)
    assert torch.equal(q, q_want) and torch.equal(sc, s_want)
    _cuda.check_error()


def test_adamw_and_gradnorm():
    torch.manual_seed(11)
    n = 100003
    npad = (n + 3) // 4 * 4
    p = torch.randn(npad, device=dev())
    g = torch.randn(npad, device=dev())
    m = torch.zeros(npad, device=dev())
    v = torch.zeros(npad, device=dev())
    w16 = torch.empty(npad, device=dev(), dtype=torch.bfloat16)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    scratch = torch.empty(1024, device=dev())
    ss = torch.zeros(1, device=dev())
    coef = torch.empty(1, device=dev())
    norm = torch.empty(1, device=dev())
    s = _cuda.stream_ptr()
    _cuda.call("sumsq", g, _cuda.L(n), scratch, ss, 0, s)
    _cuda.call("clip_coef", ss, 1.0, 1.0, coef, norm, s)
    want_norm = g[:n].norm().item()
    assert abs(norm.item() - want_norm) < 1e-3 * want_norm
    want_coef = min(1.0, 1.0 / (want_norm + 1e-6))
    assert abs(coef.item() - want_coef) < 1e-5
    for step in (1, 2, 3):
        _cuda.call("adamw", p, m, v, g, w16, _cuda.L(n), 3e-4, 0.9, 0.95, 1e-8, 0.1, step, coef, s)
        ref.adamw_(pr[:n], mr[:n], vr[:n], g[:n], 3e-4, 0.9, 0.95, 1e-8, 0.1, step, want_coef)
    assert rel_err(p[:n], pr[:n]) < 1e-5
    assert rel_err(m[:n], mr[:n]) < 1e-4 and rel_err(v[:n], vr[:n]) < 1e-4
    assert rel_err(w16[:n], pr[:n]) < 1e-2


@pytest.mark.parametrize("E,k", [(128, 8), (8, 2), (60, 4)])
def test_router_topk(E, k):
    torch.manual_seed(12)
    n = 333
    logits = torch.randn(n, E, device=dev())
    logits[5, :] = 0.0  # full tie -> lowest indices win
    counts = torch.zeros(E, device=dev(), dtype=torch.int32)
    probs, idx, w, lse = F.router_topk(logits, k, True, 1.0, counts=counts)
    pr, ir, wr, lr = ref.router_topk(logits, k, True, 1.0)
    assert torch.allclose(probs, pr, atol=1e-5)
    assert (idx == ir).all()
    assert torch.allclose(w, wr, atol=1e-5) and torch.allclose(lse, lr, atol=1e-4)
    assert (idx[5] == torch.arange(k, device=dev())).all()
    assert (counts.long() == torch.bincount(ir.flatten(), minlength=E)).all()


def test_quant_and_argmax():
    torch.manual_seed(13)
    for k in (520, 4096, 516):          # 16-byte vector path (k % 8 == 0) and the scalar fallback
        x = torch.randn(100, k, device=dev()).bfloat16()
        q, s = F.quant_rows(x)
        qr, sr = ref.quant_rows(x)
        assert torch.allclose(s, sr, rtol=1e-6) and (q.int() - qr.int()).abs().max() <= 1
        assert ((q.int() - qr.int()).abs() > 0).float().mean() < 1e-3
    lg = torch.randn(7, 151936, device=dev()).bfloat16()
    assert (F.argmax_rows(lg).long() == lg.float().argmax(-1)).all()
    # top-k rows: values descending and equal to the library's; among equal values lowest index first
    idx, val = F.topk_rows(lg, 64)
    want_v, _ = torch.topk(lg.float(), 64, dim=-1)
    assert torch.equal(val, want_v)
    assert torch.equal(lg.float().gather(1, idx.long()), val)
    small = torch.tensor([[1.0, 3.0, 3.0, -2.0, 3.0, 0.5, 0.5, 7.0]], device=dev()).bfloat16()
    i2, v2 = F.topk_rows(small, 8)
    assert i2[0].tolist() == [7, 1, 2, 4, 0, 5, 6, 3] and v2[0, 0].item() == 7.0


def test_adamw_tracks_the_fp32_oracle_over_twenty_steps():
    """The optimiser kernel is compiled without fast-math: 20 steps on the device stay within fp32
    rounding of the PyTorch restatement (master weights and both moments)."""
    from brain_b200.ops._cuda import L, call, stream_ptr
    torch.manual_seed(11)
    n = 1 << 16
    p0 = torch.randn(n)
    pm, m, v = p0.clone().cuda(), torch.zeros(n, device=dev()), torch.zeros(n, device=dev())
    w16 = torch.empty(n, device=dev(), dtype=torch.bfloat16)
    rp, rm, rv = p0.clone().double(), torch.zeros(n).double(), torch.zeros(n).double()
    coef = torch.ones(1, device=dev())
    lr, b1, b2, eps, wd = 3e-4, 0.9, 0.95, 1e-8, 0.1
    for t in range(1, 21):
        g = torch.randn(n) * (0.1 + 0.05 * t)
        call("adamw", pm, m, v, g.cuda(), w16, L(n), lr, b1, b2, eps, wd, t, coef, stream_ptr())
        gd = g.double()
        rm = b1 * rm + (1 - b1) * gd
        rv = b2 * rv + (1 - b2) * gd * gd
        rp = rp - lr * ((rm / (1 - b1 ** t)) / ((rv / (1 - b2 ** t)).sqrt() + eps) + wd * rp)
    torch.cuda.synchronize()
    assert float((pm.cpu().double() - rp).abs().max()) < 2e-6
    assert float((m.cpu().double() - rm).abs().max()) < 1e-6 and float((v.cpu().double() - rv).abs().max()) < 1e-6
    assert rel_err(w16.cpu(), rp.float()) < 4e-3
