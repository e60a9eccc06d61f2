"""Out-of-bounds write checks without a memory checker: every kernel output of these tests is a view
cut out of the middle of a larger buffer pre-filled with a sentinel.  After the launch the frame
around the view (rows above and below, columns left and right, the scratch tensors' tails) must
still hold the sentinel bit for bit, and the view itself must be fully overwritten and correct.
Shapes are ragged on purpose (partial tiles, odd token counts, pools with unused blocks)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from brain_b200.ops import _cuda, reference as ref  # noqa: E402
from brain_b200.ops._cuda import L, call, stream_ptr  # noqa: E402

SENT = 123.0   # exactly representable in bf16 and fp32; far outside every expected output


class Framed:
    """A [rows, cols] view with ``pad`` sentinel rows above/below and 8 sentinel columns on each side
    (8 elements keep 16-byte alignment of bf16 rows)."""

    def __init__(self, rows, cols, dtype=torch.bfloat16, pad=3, cpad=8):
        self.buf = torch.full((rows + 2 * pad, cols + 2 * cpad), SENT, device="cuda", dtype=dtype)
        self.view = self.buf[pad:pad + rows, cpad:cpad + cols]
        self.pad, self.cpad, self.rows, self.cols = pad, cpad, rows, cols

    def assert_frame_intact(self, what):
        b, p, c = self.buf, self.pad, self.cpad
        edges = [b[:p], b[p + self.rows:]] + ([b[:, :c], b[:, c + self.cols:]] if c else [])
        for e in edges:
            assert bool((e == SENT).all()), f"{what}: a write landed outside the output view"

    def assert_fully_written(self, what):
        assert not bool((self.view == SENT).any()), f"{what}: part of the output was never written"


def flat_canary(n, dtype, tail=64):
    buf = torch.full((n + tail,), SENT, device="cuda", dtype=dtype)
    return buf, buf[:n], buf[n:]


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.fixture(autouse=True)
def _check_device_error():
    yield
    _cuda.check_error()


@pytest.mark.parametrize("B,T,hq,hk,hd", [(2, 200, 2, 1, 128), (1, 333, 4, 2, 64), (1, 128, 2, 2, 128)])
def test_flash_forward_and_backward_stay_inside_their_outputs(B, T, hq, hk, hd):
    torch.manual_seed(T)
    q = torch.randn(B * T, hq * hd, device="cuda").bfloat16()
    k = torch.randn(B * T, hk * hd, device="cuda").bfloat16()
    v = torch.randn(B * T, hk * hd, device="cuda").bfloat16()
    do = torch.randn(B * T, hq * hd, device="cuda").bfloat16()
    scale = hd ** -0.5
    out = Framed(B * T, hq * hd)
    lse_buf, lse, lse_tail = flat_canary(B * hq * T, torch.float32)
    call("flash_fwd", q, q.stride(0), k, k.stride(0), v, v.stride(0), out.view, out.view.stride(0), lse,
         B, T, T, hq, hk, hd, float(scale), 1, stream_ptr())
    torch.cuda.synchronize()
    out.assert_frame_intact("flash forward O")
    out.assert_fully_written("flash forward O")
    assert bool((lse_tail == SENT).all()) and not bool((lse == SENT).any())
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    want = ref.attention(qr.reshape(B, T, hq, hd), kr.reshape(B, T, hk, hd), vr.reshape(B, T, hk, hd),
                         True).reshape(B * T, hq * hd)
    assert rel_err(out.view, want) < 2e-2
    want.backward(do.float())
    dq, dk, dv = Framed(B * T, hq * hd), Framed(B * T, hk * hd), Framed(B * T, hk * hd)
    d_buf, delta, d_tail = flat_canary(B * hq * T, torch.float32)
    o = out.view
    call("flash_bwd", q, q.stride(0), k, k.stride(0), v, v.stride(0), o, o.stride(0), do, do.stride(0),
         lse, delta, dq.view, dq.view.stride(0), dk.view, dk.view.stride(0), dv.view, dv.view.stride(0),
         B, T, T, hq, hk, hd, float(scale), 1, stream_ptr())
    torch.cuda.synchronize()
    for f, name, g in ((dq, "dQ", qr.grad), (dk, "dK", kr.grad), (dv, "dV", vr.grad)):
        f.assert_frame_intact("flash backward " + name)
        f.assert_fully_written("flash backward " + name)
        assert rel_err(f.view, g) < 3e-2, name
    assert bool((d_tail == SENT).all())


@pytest.mark.parametrize("kv8", [False, True])
def test_paged_kv_append_and_decode_stay_inside_their_outputs(kv8):
    torch.manual_seed(3)
    B, hq, hk, hd, bs = 3, 8, 2, 128, 16
    lens = [5, 130, 257]
    max_blocks, nb = 20, 64
    # pools: blocks 0 and nb+1 are never named by a slot or a table and must keep the sentinel
    dt = torch.int8 if kv8 else torch.bfloat16
    fill = 77 if kv8 else SENT
    kc_all = torch.full((nb + 2, hk, bs, hd), fill, device="cuda", dtype=dt)
    vc_all = torch.full((nb + 2, hk, bs, hd), fill, device="cuda", dtype=dt)
    kc, vc = kc_all[1:nb + 1], vc_all[1:nb + 1]
    ks_all = torch.full(((nb + 2) * hk * bs,), SENT, device="cuda")
    vs_all = torch.full(((nb + 2) * hk * bs,), SENT, device="cuda")
    ks, vs = ks_all[hk * bs:(nb + 1) * hk * bs], vs_all[hk * bs:(nb + 1) * hk * bs]
    perm = torch.randperm(nb)[:B * max_blocks].reshape(B, max_blocks).to("cuda", torch.int32)
    # append every token of every sequence through its slot (block * bs + offset)
    ref_k, ref_v = [], []
    for b, S in enumerate(lens):
        kn = torch.randn(S, hk * hd, device="cuda").bfloat16()
        vn = torch.randn(S, hk * hd, device="cuda").bfloat16()
        t = torch.arange(S, device="cuda")
        slots = (perm[b][(t // bs).long()].long() * bs + t % bs).to(torch.int32)
        if kv8:
            call("kv_append_i8", kn, kn.stride(0), vn, vn.stride(0), slots, kc, vc, ks, vs, None, S, hk, hd, bs,
                 stream_ptr())
        else:
            call("kv_append", kn, kn.stride(0), vn, vn.stride(0), slots, kc, vc, S, hk, hd, bs, stream_ptr())
        ref_k.append(kn)
        ref_v.append(vn)
    torch.cuda.synchronize()
    for pool in (kc_all, vc_all):
        assert bool((pool[0] == fill).all()) and bool((pool[nb + 1] == fill).all()), "append left its pool"
    used = set(int(x) for b, S in enumerate(lens) for x in perm[b][: (S + bs - 1) // bs].tolist())
    unused = [i for i in range(nb) if i not in used]
    assert bool((kc[unused] == fill).all()) and bool((vc[unused] == fill).all()), "append wrote a block no slot names"
    if kv8:
        assert bool((ks_all[:hk * bs] == SENT).all()) and bool((ks_all[(nb + 1) * hk * bs:] == SENT).all())
        assert bool((vs_all[:hk * bs] == SENT).all()) and bool((vs_all[(nb + 1) * hk * bs:] == SENT).all())
    # decode: framed output, scratch with tails
    q = torch.randn(B, hq * hd, device="cuda").bfloat16()
    seqlens = torch.tensor(lens, device="cuda", dtype=torch.int32)
    for splits in (1, 4):
        out = Framed(B, hq * hd, pad=2)
        po_buf, po, po_tail = flat_canary(B * hq * splits * hd, torch.float32)
        pm_buf, pm, pm_tail = flat_canary(B * hq * splits * 2, torch.float32)
        if kv8:
            call("paged_decode_i8", q, q.stride(0), kc, vc, ks, vs, perm, max_blocks, seqlens, out.view,
                 out.view.stride(0), po, pm, B, hq, hk, hd, bs, splits, float(hd ** -0.5), stream_ptr())
        else:
            call("paged_decode", q, q.stride(0), kc, vc, perm, max_blocks, seqlens, out.view, out.view.stride(0),
                 po, pm, B, hq, hk, hd, bs, splits, float(hd ** -0.5), stream_ptr())
        torch.cuda.synchronize()
        out.assert_frame_intact("paged decode")
        out.assert_fully_written("paged decode")
        assert bool((po_tail == SENT).all()) and bool((pm_tail == SENT).all())
        for b, S in enumerate(lens):
            want = ref.attention(q[b].float().reshape(1, 1, hq, hd), ref_k[b].float().reshape(1, S, hk, hd),
                                 ref_v[b].float().reshape(1, S, hk, hd), causal=False)
            assert rel_err(out.view[b], want.reshape(-1)) < (6e-2 if kv8 else 2e-2), (splits, b)


def test_moe_gather_grouped_gemm_and_combine_stay_inside_their_outputs():
    """The expert-sorted operand buffer, both grouped GEMM outputs and the combined output, each cut
    out of a sentinel frame; token count and expert loads chosen so that every expert's last tile
    is partial and one expert gets no token at all."""
    from brain_b200.ops.moe_cuda import _u64
    torch.manual_seed(5)
    n, d, E, k, ff = 301, 136, 5, 2, 72
    x = torch.randn(n, d, device="cuda").bfloat16()
    idx = torch.randint(0, E - 1, (n, k), device="cuda", dtype=torch.int32)      # expert E-1 stays empty
    idx[:, 1] = (idx[:, 0] + 1) % (E - 1)
    w = torch.rand(n, k, device="cuda", dtype=torch.float32)
    w_gu = (torch.randn(E, 2 * ff, d, device="cuda") * 0.1).bfloat16()
    w_dn = (torch.randn(E, d, ff, device="cuda") * 0.1).bfloat16()
    counts = torch.bincount(idx.flatten().long(), minlength=E).to(torch.int32)
    max_rows = (n * k + E * 127 + 127) // 128 * 128
    max_tiles = max_rows // 128
    offsets = torch.empty(E + 1, device="cuda", dtype=torch.int32)
    tg_buf, tile_group, tg_tail = flat_canary(max_tiles, torch.int32)
    call("moe_plan", counts, E, offsets, tile_group, max_tiles, stream_ptr())
    pp_buf, pos_of_pair, pp_tail = flat_canary(n * k, torch.int32)
    pq_buf, pair_of_pos, pq_tail = flat_canary(max_rows, torch.int32)
    pos_of_pair.fill_(-1)
    pair_of_pos.fill_(-1)
    call("moe_positions", idx, L(n * k), 0, E, offsets, pos_of_pair, pair_of_pos, stream_ptr())
    xp = Framed(max_rows, d, cpad=0)      # the kernel's output is contiguous: rows above and below only
    call("moe_gather", _u64([x.data_ptr()]), 1, n, pair_of_pos, None, k, xp.view, offsets, E, d, max_rows,
         stream_ptr())
    torch.cuda.synchronize()
    for t in (tg_tail, pp_tail, pq_tail):
        assert bool((t == SENT).all()), "routing metadata kernel wrote past its array"
    xp.assert_frame_intact("moe_gather")
    # reference from the routing tables
    pop = pair_of_pos.cpu()
    rows = (pop >= 0).nonzero().flatten()
    assert rows.numel() == n * k
    xpc = xp.view.cpu().float()
    assert torch.equal(xpc[rows], x.cpu().float()[(pop[rows] // k).long()])
    y = Framed(n, d, cpad=0)
    pairs = pos_of_pair.cpu().long().reshape(n, k)
    from brain_b200.ops.moe_cuda import grouped_gemm_rows
    gu = grouped_gemm_rows(xp.view, w_gu.view(E * 2 * ff, d), tile_group, 2 * ff, 2 * ff)
    hc = torch.empty(max_rows, ff, device="cuda", dtype=torch.bfloat16)
    call("swiglu_fwd", gu, hc, L(max_rows), ff, stream_ptr())
    yp = grouped_gemm_rows(hc, w_dn.view(E * d, ff), tile_group, d, d)
    call("moe_combine", _u64([yp.data_ptr()]), _u64([pos_of_pair.data_ptr()]), 1, idx, L(0), w.contiguous(),
         k, E, y.view, n, d, stream_ptr())
    torch.cuda.synchronize()
    y.assert_frame_intact("moe_combine")
    y.assert_fully_written("moe_combine")
    want = torch.zeros(n, d)
    xf = x.cpu().float()
    for t in range(n):
        for s in range(k):
            e = int(idx[t, s])
            g_u = w_gu[e].cpu().float() @ xf[t]
            a = torch.nn.functional.silu(g_u[:ff]) * g_u[ff:]
            want[t] += float(w[t, s]) * (w_dn[e].cpu().float() @ a)
    assert rel_err(y.view.cpu(), want) < 3e-2
    assert pairs.min() >= 0
    # the same down projection with the combine's transfer as its epilogue: every output row is stored
    # into the slot of its (token, choice) pair, padding rows are dropped, nothing else is touched
    slots = Framed(n * k, d, cpad=0)
    call("gemm_bf16_grouped_scatter", hc, w_dn.view(E * d, ff), max_rows, d, ff, hc.stride(0), ff, d, 0, tile_group,
         d, E * d, pair_of_pos, _u64([slots.view.data_ptr()]), 1, n * k, stream_ptr())
    torch.cuda.synchronize()
    slots.assert_frame_intact("grouped GEMM with combine epilogue")
    slots.assert_fully_written("grouped GEMM with combine epilogue")
    assert torch.equal(slots.view.cpu()[pop[rows].long()], yp.cpu()[rows]), "slot rows differ from the plain GEMM's rows"
    y2 = Framed(n, d, cpad=0)
    ident = torch.arange(n * k, device="cuda", dtype=torch.int32)
    call("moe_combine", _u64([slots.view.data_ptr()]), _u64([ident.data_ptr()]), 1, torch.zeros_like(ident), L(0),
         w.contiguous(), k, 1, y2.view, n, d, stream_ptr())
    torch.cuda.synchronize()
    y2.assert_frame_intact("slot sum")
    assert torch.equal(y2.view, y.view)
