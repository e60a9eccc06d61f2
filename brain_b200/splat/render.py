"""Gaussian-splat renderer on the GPU (headless: the image is a device tensor).

``render`` is the inference path — every stage is one of the kernels in ``csrc/kernels/splat.cu``
(project -> scan -> emit -> radix sort -> tile ranges -> rasterise).  ``render_diff`` is the
training path: the per-Gaussian projection is restated in PyTorch ops so autograd carries gradients
to means / rotations / scales / opacities, while tile binning, rasterisation and its backward stay
native.  On CPU tensors both fall back to the C++ oracle (forward only).

Reference: crates/splat/src/renderer.rs (stage order, 16x16 tiles, keys = tile << 32 | depth bits),
crates/splat/src/sort.rs (device scan + radix sort), crates/splat/src/reference.rs (math)."""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from ..ops._cuda import L, call, stream_ptr
from . import reference as ref
from .types import Camera, RenderOpts, Splats

TILE = 16


def _fptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


class _Binned:
    """Projection + tile binning of one view (device buffers kept for the rasteriser/backward)."""

    def __init__(self, s: Splats, cam: Camera, opts: RenderOpts):
        dev = s.means.device
        n = len(s)
        self.n, self.cam, self.opts = n, cam, opts
        self.camp, self.optp = cam.packed(), opts.packed()
        f32 = dict(device=dev, dtype=torch.float32)
        self.xy = torch.zeros(n, 2, **f32)
        self.conic_op = torch.zeros(n, 4, **f32)
        self.depth = torch.zeros(n, **f32)
        self.rad = torch.zeros(n, 2, **f32)
        self.rect = torch.zeros(n, 4, device=dev, dtype=torch.int32)
        self.touched = torch.zeros(n, device=dev, dtype=torch.int32)
        self.offs = torch.zeros(n, device=dev, dtype=torch.int32)
        scratch = torch.zeros(n // 1024 + n // (1 << 20) + 8, device=dev, dtype=torch.int32)
        m, q, sc, op = (t.detach().contiguous().float() for t in (s.means, s.quats, s.scales, s.opacities))
        call("splat_project", m, q, sc, op, n, _fptr(self.camp), cam.width, cam.height, _fptr(self.optp), opts.flags(),
             self.xy, self.conic_op, self.depth, self.rad, self.rect, self.touched, self.offs, scratch, stream_ptr())
        self.tiles_x = (cam.width + TILE - 1) // TILE
        self.tiles_y = (cam.height + TILE - 1) // TILE
        n_pairs = int(self.offs[-1].item()) + int(self.touched[-1].item()) if n else 0
        self.n_pairs = n_pairs
        np_alloc = max(n_pairs, 1)
        self.keys = torch.zeros(np_alloc, device=dev, dtype=torch.int64)
        self.order = torch.zeros(np_alloc, device=dev, dtype=torch.int32)
        self.ranges = torch.zeros(self.tiles_x * self.tiles_y, 2, device=dev, dtype=torch.int32)
        if n_pairs:
            call("splat_emit", self.rect, self.depth, self.touched, self.offs, n, self.tiles_x, self.keys, self.order,
                 stream_ptr())
            keys_tmp, vals_tmp = torch.empty_like(self.keys), torch.empty_like(self.order)
            nblocks = (n_pairs + 2047) // 2048
            hist = torch.zeros(256 * nblocks, device=dev, dtype=torch.int32)
            scr = torch.zeros(256 * nblocks // 1024 + 16, device=dev, dtype=torch.int32)
            tile_bits = max(1, int(self.tiles_x * self.tiles_y - 1).bit_length())
            call("radix_sort_pairs", self.keys, self.order, keys_tmp, vals_tmp, L(n_pairs), 32 + tile_bits, hist, scr,
                 stream_ptr())

    def rasterise(self, xy, conic_op, colors, want_aux: bool):
        cam, dev = self.cam, xy.device
        img = torch.empty(cam.height, cam.width, 4, device=dev, dtype=torch.float32)
        final_t = torch.empty(cam.height, cam.width, device=dev, dtype=torch.float32) if want_aux else None
        ncon = torch.empty(cam.height, cam.width, device=dev, dtype=torch.int32) if want_aux else None
        self.ranges.zero_()
        call("splat_raster", self.keys, self.order, L(self.n_pairs), self.ranges, xy, conic_op, self.depth, self.rad,
             colors, cam.width, cam.height, _fptr(self.optp), self.opts.flags(), img, final_t, ncon, stream_ptr())
        return img, final_t, ncon


def render(s: Splats, cam: Camera, opts: RenderOpts = RenderOpts()) -> torch.Tensor:
    """[H, W, 4] fp32 (rgb or depth x3, alpha)."""
    if not s.means.is_cuda:
        return ref.render(s, cam, opts)
    b = _Binned(s, cam, opts)
    img, _, _ = b.rasterise(b.xy, b.conic_op, s.colors.detach().contiguous().float(), False)
    return img


# ------------------------------------------------------------------------------------ differentiable path
def project_torch(means, quats, scales, opac, cam: Camera, opts: RenderOpts):
    """The projection as differentiable tensor ops -> (xy [N,2], conic_op [N,4]); culled Gaussians
    get zero opacity (they are not binned, so their values never matter)."""
    dev = means.device
    v = torch.from_numpy(cam.viewmat()).to(dev).view(3, 4)
    W, t = v[:, :3], v[:, 3]
    pc = means @ W.T + t
    x, y, z = pc[:, 0], pc[:, 1], pc[:, 2].clamp_min(1e-6)
    qn = quats / (quats.norm(dim=1, keepdim=True) + 1e-8)
    qw, qx, qy, qz = qn.unbind(1)
    R = torch.stack([1 - 2 * (qy * qy + qz * qz), 2 * (qx * qy - qw * qz), 2 * (qx * qz + qw * qy),
                     2 * (qx * qy + qw * qz), 1 - 2 * (qx * qx + qz * qz), 2 * (qy * qz - qw * qx),
                     2 * (qx * qz - qw * qy), 2 * (qy * qz + qw * qx), 1 - 2 * (qx * qx + qy * qy)], dim=1).view(-1, 3, 3)
    M = R * scales[:, None, :]
    sig = M @ M.transpose(1, 2)
    cc = W @ sig @ W.T
    w, h = float(cam.width), float(cam.height)
    tfx, tfy = 0.5 * w / cam.fx, 0.5 * h / cam.fy
    lxp, lxn = (w - cam.cx) / cam.fx + 0.3 * tfx, cam.cx / cam.fx + 0.3 * tfx
    lyp, lyn = (h - cam.cy) / cam.fy + 0.3 * tfy, cam.cy / cam.fy + 0.3 * tfy
    rz = 1.0 / z
    txc = z * torch.minimum(torch.maximum(x * rz, torch.tensor(-lxn, device=dev)), torch.tensor(lxp, device=dev))
    tyc = z * torch.minimum(torch.maximum(y * rz, torch.tensor(-lyn, device=dev)), torch.tensor(lyp, device=dev))
    j00, j02 = cam.fx * rz, -cam.fx * txc * rz * rz
    j11, j12 = cam.fy * rz, -cam.fy * tyc * rz * rz
    sa = j00 * j00 * cc[:, 0, 0] + 2 * j00 * j02 * cc[:, 0, 2] + j02 * j02 * cc[:, 2, 2]
    sb = j00 * (cc[:, 0, 1] * j11 + cc[:, 0, 2] * j12) + j02 * (cc[:, 2, 1] * j11 + cc[:, 2, 2] * j12)
    sc = j11 * j11 * cc[:, 1, 1] + 2 * j11 * j12 * cc[:, 1, 2] + j12 * j12 * cc[:, 2, 2]
    det0 = sa * sc - sb * sb
    sa, sc = sa + opts.eps2d, sc + opts.eps2d
    det = (sa * sc - sb * sb).clamp_min(1e-12)
    op = opac
    if opts.antialiased:
        op = op * torch.sqrt((det0 / det).clamp_min(0.005 * 0.005))
    xy = torch.stack([cam.fx * x * rz + cam.cx, cam.fy * y * rz + cam.cy], dim=1)
    conic_op = torch.stack([sc / det, -sb / det, sa / det, op], dim=1)
    return xy, conic_op


class _Rasterise(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xy, conic_op, colors, binned: _Binned):
        xy, conic_op, colors = xy.contiguous().float(), conic_op.contiguous().float(), colors.contiguous().float()
        img, final_t, ncon = binned.rasterise(xy, conic_op, colors, True)
        ctx.save_for_backward(xy, conic_op, colors, final_t, ncon)
        ctx.binned = binned
        return img

    @staticmethod
    def backward(ctx, dimg):
        xy, conic_op, colors, final_t, ncon = ctx.saved_tensors
        b = ctx.binned
        n = xy.shape[0]
        d_colors = torch.zeros(n, 3, device=xy.device)
        d_opac = torch.zeros(n, device=xy.device)
        d_conic = torch.zeros(n, 3, device=xy.device)
        d_xy = torch.zeros(n, 2, device=xy.device)
        call("splat_raster_bwd", b.ranges, b.order, xy, conic_op, b.rad, colors, b.cam.width, b.cam.height,
             _fptr(b.optp), final_t, ncon, dimg.contiguous().float(), d_colors, d_opac, d_conic, d_xy, stream_ptr())
        return d_xy, torch.cat([d_conic, d_opac[:, None]], dim=1), d_colors, None


def render_diff(s: Splats, cam: Camera, opts: RenderOpts = RenderOpts()) -> torch.Tensor:
    """Differentiable colour render (``opts.depth`` must be False): gradients reach every field of
    ``s`` that requires grad."""
    assert not opts.depth, "the differentiable path renders colour"
    assert s.means.is_cuda, "the differentiable path needs a CUDA device"
    b = _Binned(s, cam, opts)
    xy, conic_op = project_torch(s.means.float(), s.quats.float(), s.scales.float(), s.opacities.float(), cam, opts)
    return _Rasterise.apply(xy, conic_op, s.colors, b)
