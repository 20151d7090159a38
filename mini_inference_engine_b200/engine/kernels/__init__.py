"""GPU operators of the hot path, under the reference's names."""

from .sm89_fp8 import install_sm89_fp8_dispatch, sm89_available, sm89_fp8_linear

__all__ = ["install_sm89_fp8_dispatch", "sm89_available", "sm89_fp8_linear"]
