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


def _composite_dense(xy, conic_op, colors, depth, rad, H, W, bg):
    """Dense PyTorch restatement of the compositing (every Gaussian against every pixel, sorted by
    depth), differentiable by autograd; the skip tests are masks, exactly like the kernel."""
    order = torch.argsort(depth)
    xy, conic_op, colors, rad = xy[order], conic_op[order], colors[order], rad[order]
    ys, xs = torch.meshgrid(torch.arange(H, device=xy.device) + 0.5, torch.arange(W, device=xy.device) + 0.5, indexing="ij")
    dx = xy[:, 0, None, None] - xs[None]
    dy = xy[:, 1, None, None] - ys[None]
    sigma = 0.5 * (conic_op[:, 0, None, None] * dx * dx + conic_op[:, 2, None, None] * dy * dy) + conic_op[:, 1, None, None] * dx * dy
    alpha = torch.clamp(conic_op[:, 3, None, None] * torch.exp(-sigma), max=0.99)
    keep = (dx.abs() <= rad[:, 0, None, None]) & (dy.abs() <= rad[:, 1, None, None]) & (sigma >= 0) & (alpha >= 1.0 / 255.0)
    alpha = torch.where(keep, alpha, torch.zeros_like(alpha))
    T = torch.ones(H, W, device=xy.device)
    C = torch.zeros(H, W, 3, device=xy.device)
    alive = torch.ones(H, W, dtype=torch.bool, device=xy.device)
    for k in range(xy.shape[0]):
        nt = T * (1 - alpha[k])
        alive = alive & ~((nt <= 1e-4) & (alpha[k] > 0))
        a_k = torch.where(alive, alpha[k], torch.zeros_like(alpha[k]))
        C = C + (a_k * T)[..., None] * colors[k]
        T = T * (1 - a_k)
    return torch.cat([C + T[..., None] * torch.tensor(bg, device=xy.device), (1 - T)[..., None]], dim=-1)


def test_render_diff_gradients_match_autograd_reference_and_finite_differences():
    """Analytic gradients of the CUDA rasteriser against autograd through a dense PyTorch
    restatement (both treat the contribution tests as fixed masks), then a finite-difference check
    on the fields whose loss is smooth (colours exactly linear; means, where the moving cut-off
    boundary gains on one side what it loses on the other)."""
    from brain_b200.splat.render import _Binned, project_torch
    torch.manual_seed(0)
    s = Splats.random(60, seed=3)
    s.scales = s.scales * 3.0
    H = W = 48
    cam = Camera.look_at([0, 0, -3.0], [0, 0, 0], [0, 1, 0], 50.0, W, H)
    opts = RenderOpts(bg=(0.05, 0.1, 0.15))
    dev = "cuda"
    names = ("means", "quats", "scales", "opacities", "colors")
    wimg = torch.rand(H, W, 4, device=dev)

    def leaves():
        return {k: getattr(s, k).to(dev).clone().requires_grad_() for k in names}
    f1 = leaves()
    img = render_diff(Splats(*(f1[k] for k in names)), cam, opts)
    (img * wimg).sum().backward()
    f2 = leaves()
    b = _Binned(Splats(*(f2[k].detach() for k in names)), cam, opts)
    xy, conic_op = project_torch(f2["means"], f2["quats"], f2["scales"], f2["opacities"], cam, opts)
    live = b.touched > 0
    ref_img = _composite_dense(xy[live], conic_op[live], f2["colors"][live], b.depth[live], b.rad[live], H, W, opts.bg)
    assert float((ref_img - img.detach()).abs().max()) < 2e-3
    (ref_img * wimg).sum().backward()
    for k in names:
        ga, gr = f1[k].grad, f2[k].grad
        assert float((ga - gr).norm() / gr.norm().clamp_min(1e-6)) < 2e-3, k

    def loss_of(f):
        return float((render_diff(Splats(*(f[k] for k in names)), cam, opts) * wimg).sum())
    g = torch.Generator().manual_seed(1)
    for name, eps, tol in (("colors", 1e-2, 0.01), ("means", 2e-3, 0.15)):
        p = f1[name]
        v = (torch.randint(0, 2, p.shape, generator=g).float() * 2 - 1).to(dev)
        analytic = float((p.grad * v).sum())
        with torch.no_grad():
            plus = {k: t.detach() for k, t in f1.items()}
            minus = dict(plus)
            plus[name] = p.detach() + eps * v
            minus[name] = p.detach() - eps * v
            numeric = (loss_of(plus) - loss_of(minus)) / (2 * eps)
        assert abs(analytic - numeric) <= tol * max(abs(analytic), abs(numeric)) + 0.05, (name, analytic, numeric)
