"""Block-diffusion decoding: denoising schedule, per-request canvas state
(python/minisgl/diffusion/__init__.py, python/minisgl/diffusion/sampler.py)."""
from .sampler import Canvas, DenoiseConfig, entropy_bound_accept

__all__ = ["Canvas", "DenoiseConfig", "entropy_bound_accept"]
