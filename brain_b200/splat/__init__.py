"""3D Gaussian splatting: scene types, the CPU oracle and the CUDA rasteriser (headless)."""
from .types import Camera, RenderOpts, Splats  # noqa: F401
