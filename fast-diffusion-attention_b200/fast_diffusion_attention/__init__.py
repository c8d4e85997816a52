"""Block-diffusion attention for NVIDIA B200 (sm_100a): drop-in for the `fast_diffusion_attention` package."""

from .version import __version__  # noqa: F401
from .interface import diffusion_attn_func, diffusion_attn_varlen_func  # noqa: F401

__all__ = ["diffusion_attn_func", "diffusion_attn_varlen_func", "__version__"]
