"""CPU oracle of the splat renderer: thin wrapper over the native C++ restatement
(``csrc/runtime/splat_ref.cpp``; reference: crates/splat/src/reference.rs)."""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch

from .. import _host
from .types import Camera, RenderOpts, Splats

_host.register({
    "bbh_splat_render": (ctypes.c_int, [ctypes.c_void_p] * 5 + [ctypes.c_int64, ctypes.c_void_p, ctypes.c_int,
                                                                 ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                                                 ctypes.c_void_p, ctypes.c_int]),
})


def render(s: Splats, cam: Camera, opts: RenderOpts = RenderOpts(), threads: int = 0) -> torch.Tensor:
    """[H, W, 4] fp32 image (rgb or depth x3, alpha)."""
    arrs = [np.ascontiguousarray(t.detach().cpu().numpy(), dtype=np.float32) for t in s.tensors()]
    camp, op = cam.packed(), opts.packed()
    img = np.zeros((cam.height, cam.width, 4), dtype=np.float32)
    _host.lib().bbh_splat_render(*(a.ctypes.data for a in arrs), len(s), camp.ctypes.data, cam.width, cam.height,
                                 op.ctypes.data, opts.flags(), img.ctypes.data, threads or min(16, os.cpu_count() or 1))
    return torch.from_numpy(img)
