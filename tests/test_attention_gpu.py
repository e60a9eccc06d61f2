"""Flash attention kernels vs the materialised-scores fp32 reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from brain_b200.ops import _cuda, reference as ref  # noqa: E402
from brain_b200.ops.attention import flash_attention  # noqa: E402


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.fixture(autouse=True)
def _check_device_error():
    yield
    _cuda.check_error()


CASES = [
    # B, T, hq, hk, hd, causal
    (1, 128, 2, 1, 128, True),
    (2, 256, 4, 2, 128, True),
    (1, 512, 4, 4, 64, True),
    (2, 200, 2, 1, 128, True),     # ragged tail tile
    (1, 384, 2, 2, 128, False),
    (1, 1024, 8, 2, 128, True),
]


@pytest.mark.parametrize("B,T,hq,hk,hd,causal", CASES)
def test_flash_fwd(B, T, hq, hk, hd, causal):
    torch.manual_seed(B * T + hq)
    dev = "cuda"
    width = (hq + 2 * hk) * hd
    qkv = torch.randn(B * T, width, device=dev).bfloat16()
    q, k, v = qkv[:, :hq * hd], qkv[:, hq * hd:(hq + hk) * hd], qkv[:, (hq + hk) * hd:]
    out = flash_attention(q, k, v, B, T, hq, hk, hd, causal)
    want = ref.attention(q.float().reshape(B, T, hq, hd), k.float().reshape(B, T, hk, hd),
                         v.float().reshape(B, T, hk, hd), causal).reshape(B * T, hq * hd)
    assert rel_err(out, want) < 2e-2


@pytest.mark.parametrize("B,T,hq,hk,hd,causal", CASES)
def test_flash_bwd(B, T, hq, hk, hd, causal):
    torch.manual_seed(B * T + hq + 1)
    dev = "cuda"
    q = torch.randn(B * T, hq * hd, device=dev).bfloat16().requires_grad_()
    k = torch.randn(B * T, hk * hd, device=dev).bfloat16().requires_grad_()
    v = torch.randn(B * T, hk * hd, device=dev).bfloat16().requires_grad_()
    out = flash_attention(q, k, v, B, T, hq, hk, hd, causal)
    do = torch.randn_like(out)
    out.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    want = ref.attention(qr.reshape(B, T, hq, hd), kr.reshape(B, T, hk, hd),
                         vr.reshape(B, T, hk, hd), causal).reshape(B * T, hq * hd)
    want.backward(do.float())
    assert rel_err(q.grad, qr.grad) < 3e-2
    assert rel_err(k.grad, kr.grad) < 3e-2
    assert rel_err(v.grad, vr.grad) < 3e-2


@pytest.mark.parametrize("form", ["1"])
def test_flash_fwd_first_form_still_matches(form):
    """BB_FA_FWD=1 selects the single-buffer forward kernel (the one with timeline stamps); the
    switch is read once per process, so the check runs in a child process."""
    import os
    import subprocess
    import sys
    code = (
        "import math, torch\n"
        "from brain_b200.ops import _cuda, reference as ref\n"
        "from brain_b200.ops.attention import flash_attention\n"
        "torch.manual_seed(0)\n"
        "for (B,T,hq,hk,hd,S) in ((2,256,4,2,128,256),(1,200,2,1,64,200),(1,72,4,2,64,200)):\n"
        "    q=torch.randn(B*T,hq*hd,device='cuda').bfloat16(); k=torch.randn(B*S,hk*hd,device='cuda').bfloat16(); v=torch.randn(B*S,hk*hd,device='cuda').bfloat16()\n"
        "    o=flash_attention(q,k,v,B,T,hq,hk,hd,True,S=S); _cuda.check_error()\n"
        "    w=ref.attention(q.float().reshape(B,T,hq,hd),k.float().reshape(B,S,hk,hd),v.float().reshape(B,S,hk,hd),True,1/math.sqrt(hd)).reshape(B*T,hq*hd)\n"
        "    assert ((o.float()-w).norm()/w.norm()).item() < 2e-2\n"
        "print('ok')\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, BB_FA_FWD=form, PYTHONPATH=root),
                       capture_output=True, text=True, timeout=300, cwd=root)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


def test_flash_fwd_prefix_offset():
    """Queries are the last T positions of an S-long context (chunked prefill shape)."""
    torch.manual_seed(5)
    B, T, S, hq, hk, hd = 1, 128, 384, 2, 1, 128
    q = torch.randn(B * T, hq * hd, device="cuda").bfloat16()
    k = torch.randn(B * S, hk * hd, device="cuda").bfloat16()
    v = torch.randn(B * S, hk * hd, device="cuda").bfloat16()
    out = flash_attention(q, k, v, B, T, hq, hk, hd, True, S=S)
    want = ref.attention(q.float().reshape(B, T, hq, hd), k.float().reshape(B, S, hk, hd),
                         v.float().reshape(B, S, hk, hd), True).reshape(B * T, hq * hd)
    assert rel_err(out, want) < 2e-2


@pytest.mark.parametrize("B,T,hq,hk,hd,norm", [(2, 256, 4, 2, 128, True), (1, 384, 4, 4, 64, False),
                                                (1, 200, 2, 1, 128, True)])
def test_attention_from_fused_qkv(B, T, hq, hk, hd, norm):
    """The single-node qk-norm + rope + attention op against the fp32 CPU composition, including
    the gradient of the whole qkv buffer (q|k through the rope backward, v written in place)."""
    from brain_b200.ops.attention import attention_qkv
    torch.manual_seed(7 * T + hd)
    width = (hq + 2 * hk) * hd
    qkv = (torch.randn(B * T, width) * 0.7)
    wq = (1.0 + 0.1 * torch.randn(hd)) if norm else None
    wk = (1.0 + 0.1 * torch.randn(hd)) if norm else None
    cos, sin = ref.rope_tables(T, hd, 1e6)
    pos = torch.arange(T, dtype=torch.int32).repeat(B)
    do = torch.randn(B * T, hq * hd)

    def run(dev, dt):
        x = qkv.to(dev, dt).requires_grad_()
        gq = wq.to(dev, dt).requires_grad_() if norm else None
        gk = wk.to(dev, dt).requires_grad_() if norm else None
        o = attention_qkv(x, gq, gk, cos.to(dev), sin.to(dev), pos.to(dev), B, T, hq, hk, hd, 1e-6)
        o.backward(do.to(dev, dt))
        return o.detach(), x.grad, (gq.grad if norm else None), (gk.grad if norm else None)

    o1, dx1, dq1, dk1 = run("cuda", torch.bfloat16)
    o0, dx0, dq0, dk0 = run("cpu", torch.float32)
    assert rel_err(o1.cpu(), o0) < 2e-2
    qkw = (hq + hk) * hd
    assert rel_err(dx1.cpu()[:, :qkw], dx0[:, :qkw]) < 4e-2
    assert rel_err(dx1.cpu()[:, qkw:], dx0[:, qkw:]) < 3e-2
    if norm:
        assert rel_err(dq1.cpu(), dq0) < 5e-2 and rel_err(dk1.cpu(), dk0) < 5e-2


@pytest.mark.parametrize("hd,block_rows", [(128, 16), (64, 32)])
def test_paged_varlen_flash_forward(hd, block_rows):
    """One launch over packed sequences of different lengths whose keys and values live in a paged
    pool (shuffled blocks, cached prefixes of different lengths) against plain attention per sequence."""
    import math
    from brain_b200.ops import _cuda, reference as ref
    from brain_b200.ops._cuda import call, stream_ptr
    torch.manual_seed(7)
    hq, hk = 4, 2
    seqs = [(0, 200), (48, 130), (300, 17), (16, 256)]            # (cached prefix, new rows)
    max_blocks = 40
    pool_blocks = 160
    kc = torch.randn(pool_blocks, hk, block_rows, hd, device="cuda").bfloat16()
    vc = torch.randn(pool_blocks, hk, block_rows, hd, device="cuda").bfloat16()
    perm = torch.randperm(pool_blocks).tolist()
    tables, row0, ctx, tiles, qs, wants = [], [0], [], [], [], []
    used = 0
    for si, (start, new) in enumerate(seqs):
        S = start + new
        nb = -(-S // block_rows)
        blocks = perm[used:used + nb]
        used += nb
        tables.append(blocks + [-1] * (max_blocks - nb))
        k = torch.cat([kc[b] for b in blocks], dim=1)[:, :S]      # [hk, S, hd]
        v = torch.cat([vc[b] for b in blocks], dim=1)[:, :S]
        q = torch.randn(new, hq * hd, device="cuda").bfloat16()
        qs.append(q)
        w = ref.attention(q.float().reshape(1, new, hq, hd), k.float().transpose(0, 1).reshape(1, S, hk, hd),
                          v.float().transpose(0, 1).reshape(1, S, hk, hd), True, 1 / math.sqrt(hd)).reshape(new, hq * hd)
        wants.append(w)
        row0.append(row0[-1] + new)
        ctx.append(S)
        tiles += [(si, t) for t in range(-(-new // 128))]
    q = torch.cat(qs)
    n = q.shape[0]
    pad = torch.full((n + 2, hq * hd), 9.0, device="cuda", dtype=torch.bfloat16)   # canary rows around the output
    out = pad[1:n + 1]
    dev_i = lambda x: torch.tensor(x, device="cuda", dtype=torch.int32)
    call("flash_fwd_paged", q, q.stride(0), kc, vc, out, out.stride(0), dev_i(tables), max_blocks, block_rows, pool_blocks,
         dev_i(row0), dev_i(ctx), dev_i([t[0] for t in tiles]), dev_i([t[1] for t in tiles]), len(tiles), n, hq, hk, hd,
         float(hd ** -0.5), stream_ptr())
    torch.cuda.synchronize()
    _cuda.check_error()
    want = torch.cat(wants)
    assert ((out.float() - want).norm() / want.norm()).item() < 2e-2
    assert (pad[0] == 9).all() and (pad[-1] == 9).all()
