"""``brain splat <render|train>`` — headless Gaussian-splat rendering and a small fitting loop
(reference: crates/cli/src/splat_cli.rs; the reference's viewer window and wgpu surface are left
out: images go to ``.npy`` / binary PPM files)."""
from __future__ import annotations

import sys
import time
from typing import List

from .args import Args


def _save(img, path: str) -> None:
    import numpy as np
    a = img.detach().cpu().numpy()
    if path.endswith(".npy"):
        np.save(path, a)
        return
    rgb = (np.clip(a[..., :3], 0.0, 1.0) * 255.0 + 0.5).astype(np.uint8)
    with open(path, "wb") as f:
        f.write(f"P6 {rgb.shape[1]} {rgb.shape[0]} 255\n".encode())
        f.write(rgb.tobytes())


def run_splat(argv: List[str], device: str = "auto") -> int:
    import torch
    from ..splat.render import render, render_diff
    from ..splat.types import Camera, RenderOpts, Splats
    from ..train import pick_device
    verb = argv[0] if argv else None
    a = Args(argv[1:])
    n = a.int_or("--n", 20000)
    w, h = a.int_or("--width", 640), a.int_or("--height", 480)
    seed = a.int_or("--seed", 0)
    out = a.str_or("--out", "splat.ppm")
    dev = pick_device(device)
    cam = Camera.look_at([0.0, 0.0, -3.0], [0, 0, 0], [0, 1, 0], a.float_or("--fov", 50.0), w, h)
    if verb == "render":
        depth = a.take_flag("--depth")
        a.finish()
        s = Splats.random(n, seed).to(dev)
        opts = RenderOpts(depth=depth)
        t0 = time.perf_counter()
        img = render(s, cam, opts)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        _save(img, out)
        print(f"rendered {n} gaussians at {w}x{h} on {dev} in {dt * 1e3:.1f} ms -> {out}")
        return 0
    if verb == "train":
        steps, lr = a.int_or("--steps", 200), a.float_or("--lr", 2e-2)
        a.finish()
        if dev.type != "cuda":
            print("brain splat train needs a CUDA device (the CPU oracle is forward-only)", file=sys.stderr)
            return 1
        target = render(Splats.random(n, seed).to(dev), cam, RenderOpts())
        s = Splats.random(n, seed + 1).to(dev)
        params = [t.requires_grad_() for t in s.tensors()]
        opt = torch.optim.Adam(params, lr=lr)
        first = last = None
        for step in range(steps):
            opt.zero_grad()
            with torch.no_grad():
                s.opacities.clamp_(0.02, 0.98)
                s.scales.clamp_(1e-3, 2.0)
            loss = ((render_diff(s, cam, RenderOpts()) - target) ** 2).mean()
            loss.backward()
            opt.step()
            last = float(loss)
            first = last if first is None else first
            if (step + 1) % max(steps // 10, 1) == 0:
                print(f"step {step + 1:>6}  loss {last:.6f}")
        _save(render(s, cam, RenderOpts()), out)
        print(f"trained: loss {first:.6f} -> {last:.6f}; image -> {out}")
        return 0
    print(f"usage: brain splat <render|train> [--n N --width W --height H --seed S --out F.ppm|.npy --depth]  (got {verb!r})",
          file=sys.stderr)
    return 2
