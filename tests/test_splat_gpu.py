"""Gaussian-splat rasteriser kernels vs the C++ CPU oracle, the device scan / radix sort
primitives, and a finite-difference check of the differentiable path."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from brain_b200.ops import _cuda  # noqa: E402
from brain_b200.ops._cuda import L, call, stream_ptr  # noqa: E402
from brain_b200.splat import reference as ref  # noqa: E402
from brain_b200.splat.render import render, render_diff  # noqa: E402
from brain_b200.splat.types import Camera, RenderOpts, Splats  # noqa: E402


@pytest.fixture(autouse=True)
def _check_device_error():
    yield
    _cuda.check_error()


@pytest.mark.parametrize("n", [5, 1024, 1025, 300_000])
def test_scan_u32(n):
    x = torch.randint(0, 50, (n,), device="cuda", dtype=torch.int32)
    out = torch.empty_like(x)
    scratch = torch.zeros(n // 1024 + n // (1 << 20) + 8, device="cuda", dtype=torch.int32)
    call("scan_u32", x, out, L(n), scratch, stream_ptr())
    want = torch.cumsum(x.long(), 0) - x.long()
    assert torch.equal(out.long(), want)


@pytest.mark.parametrize("n,bits", [(1, 40), (2047, 40), (2049, 48), (200_000, 44)])
def test_radix_sort_pairs_is_stable(n, bits):
    g = torch.Generator(device="cuda").manual_seed(n)
    keys = torch.randint(0, 1 << 20, (n,), device="cuda", generator=g, dtype=torch.int64) << (bits - 20)
    keys |= torch.randint(0, 4, (n,), device="cuda", generator=g, dtype=torch.int64)       # many duplicates in the low bits
    vals = torch.arange(n, device="cuda", dtype=torch.int32)
    k, v = keys.clone(), vals.clone()
    nblocks = (n + 2047) // 2048
    hist = torch.zeros(256 * nblocks, device="cuda", dtype=torch.int32)
    scr = torch.zeros(256 * nblocks // 1024 + 16, device="cuda", dtype=torch.int32)
    call("radix_sort_pairs", k, v, torch.empty_like(k), torch.empty_like(v), L(n), bits, hist, scr, stream_ptr())
    want_k, idx = torch.sort(keys, stable=True)
    assert torch.equal(k, want_k) and torch.equal(v.long(), idx)


@pytest.mark.parametrize("n,wh,depth,aa", [(500, (64, 48), False, False), (4000, (160, 112), False, True),
                                            (4000, (130, 70), True, False)])
def test_render_matches_cpu_oracle(n, wh, depth, aa):
    s = Splats.random(n, seed=n)
    cam = Camera.look_at([0.3, 0.2, -3.0], [0, 0, 0], [0, 1, 0], 55.0, *wh)
    opts = RenderOpts(bg=(0.1, 0.2, 0.3), depth=depth, antialiased=aa)
    want = ref.render(s, cam, opts)
    got = render(s.to("cuda"), cam, opts).cpu()
    assert got.shape == want.shape
    err = (got - want).abs()
    # identical math in fp32; a pixel can differ only where a contribution sits on a threshold
    assert float(err.mean()) < 2e-4 and float((err > 2e-2).float().mean()) < 2e-3


def test_render_diff_gradients_match_finite_differences():
    torch.manual_seed(0)
    s = Splats.random(60, seed=3)
    s.scales = s.scales * 3.0
    cam = Camera.look_at([0, 0, -3.0], [0, 0, 0], [0, 1, 0], 50.0, 48, 48)
    opts = RenderOpts(bg=(0.05, 0.05, 0.05))
    dev = "cuda"
    fields = {k: getattr(s, k).to(dev).double().float().requires_grad_() for k in ("means", "quats", "scales", "opacities", "colors")}
    wimg = torch.rand(48, 48, 4, device=dev)

    def loss_of(f):
        img = render_diff(Splats(f["means"], f["quats"], f["scales"], f["opacities"], f["colors"]), cam, opts)
        return (img * wimg).sum()

    loss = loss_of(fields)
    loss.backward()
    base = render(Splats(*(fields[k].detach() for k in ("means", "quats", "scales", "opacities", "colors"))), cam, opts)
    assert float((render_diff(Splats(*(fields[k].detach() for k in ("means", "quats", "scales", "opacities", "colors"))), cam, opts) - base).abs().max()) < 1e-3
    g = torch.Generator().manual_seed(1)
    for name, eps in (("colors", 1e-2), ("opacities", 2e-3), ("means", 2e-3), ("scales", 1e-3), ("quats", 2e-3)):
        p = fields[name]
        v = (torch.randint(0, 2, p.shape, generator=g).float() * 2 - 1).to(dev)
        analytic = float((p.grad * v).sum())
        with torch.no_grad():
            plus = dict(fields); plus[name] = p.detach() + eps * v
            minus = dict(fields); minus[name] = p.detach() - eps * v
            plus = {k: t.detach() for k, t in plus.items()}
            minus = {k: t.detach() for k, t in minus.items()}
            numeric = float((loss_of(plus) - loss_of(minus)) / (2 * eps))
        assert abs(analytic - numeric) <= 0.02 * max(abs(analytic), abs(numeric)) + 0.05, (name, analytic, numeric)
