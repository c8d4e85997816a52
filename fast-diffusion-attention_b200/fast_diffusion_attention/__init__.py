"""Block-diffusion attention for NVIDIA B200 (sm_100a): drop-in for the `fast_diffusion_attention` package."""

from .version import __version__  # noqa: F401
from .interface import (  # noqa: F401
    diffusion_attn_func,
    diffusion_attn_varlen_func,
    diffusion_attn_qkvpacked_func,
    diffusion_attn_varlen_qkvpacked_func,
)

__all__ = ["diffusion_attn_func", "diffusion_attn_varlen_func", "diffusion_attn_qkvpacked_func",
           "diffusion_attn_varlen_qkvpacked_func", "__version__"]
