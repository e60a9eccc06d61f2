"""Scene, camera and options of the Gaussian-splat renderer (reference: crates/splat/src/types.rs —
``Camera`` with a camera-to-world matrix and pinhole intrinsics, ``look_at``, ``Splats`` as flat
per-Gaussian arrays with quaternions in wxyz order, ``RenderOpts``)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Tuple

import numpy as np
import torch


@dataclass
class Camera:
    c2w: np.ndarray           # [4, 4] row-major camera-to-world (columns: right, down, forward, eye)
    fx: float
    fy: float
    cx: float
    cy: float
    width: int
    height: int

    def viewmat(self) -> np.ndarray:
        """World-to-camera as 12 floats (row-major 3x4): R^T and -R^T t."""
        m = np.asarray(self.c2w, dtype=np.float64).reshape(4, 4)
        r = m[:3, :3].T
        t = -r @ m[:3, 3]
        return np.concatenate([r, t[:, None]], axis=1).reshape(-1).astype(np.float32)

    def packed(self) -> np.ndarray:
        return np.concatenate([self.viewmat(), [self.fx, self.fy, self.cx, self.cy]]).astype(np.float32)

    @staticmethod
    def look_at(eye, target, up, fov_y_deg: float, width: int, height: int) -> "Camera":
        eye, target, up = (np.asarray(v, dtype=np.float64) for v in (eye, target, up))

        def norm(v):
            return v / max(np.linalg.norm(v), 1e-12)
        f = norm(target - eye)
        r = norm(np.cross(f, up))
        d = norm(np.cross(f, r))
        c2w = np.eye(4)
        c2w[:3, 0], c2w[:3, 1], c2w[:3, 2], c2w[:3, 3] = r, d, f, eye
        fy = 0.5 * height / math.tan(0.5 * math.radians(fov_y_deg))
        return Camera(c2w.astype(np.float32), fy, fy, width / 2.0, height / 2.0, width, height)


@dataclass
class RenderOpts:
    bg: Tuple[float, float, float] = (0.0, 0.0, 0.0)
    depth: bool = False
    antialiased: bool = False
    eps2d: float = 0.3
    near: float = 0.01
    far: float = 1e10

    def packed(self) -> np.ndarray:
        return np.asarray([*self.bg, self.eps2d, self.near, self.far], dtype=np.float32)

    def flags(self) -> int:
        return int(self.depth) | (int(self.antialiased) << 1)


@dataclass
class Splats:
    means: torch.Tensor       # [N, 3]
    quats: torch.Tensor       # [N, 4] wxyz
    scales: torch.Tensor      # [N, 3] (linear, not log)
    opacities: torch.Tensor   # [N] in (0, 1)
    colors: torch.Tensor      # [N, 3]

    def __len__(self) -> int:
        return int(self.opacities.shape[0])

    def to(self, device) -> "Splats":
        return Splats(*(t.to(device) for t in (self.means, self.quats, self.scales, self.opacities, self.colors)))

    def tensors(self):
        return (self.means, self.quats, self.scales, self.opacities, self.colors)

    @staticmethod
    def random(n: int, seed: int = 0, extent: float = 1.0, device="cpu") -> "Splats":
        g = torch.Generator().manual_seed(seed)
        means = (torch.rand(n, 3, generator=g) * 2 - 1) * extent
        quats = torch.randn(n, 4, generator=g)
        scales = torch.exp(torch.rand(n, 3, generator=g) * 1.5 - 3.5) * extent
        opac = torch.rand(n, generator=g) * 0.8 + 0.15
        colors = torch.rand(n, 3, generator=g)
        return Splats(means, quats, scales, opac, colors).to(device)
