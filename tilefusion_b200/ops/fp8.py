"""Bulk conversion between fp16/bf16 tensors and 8-bit floating-point storage.

TileFusion declares ``__fp8_e4m3`` / ``__fp8_e5m2`` and converts single values
(``include/types/base.hpp:13-39`` and ``:70-107``); these operators convert
whole tensors on the device, which is what writing and reading an 8-bit K/V
cache needs.  Rounding is to nearest even and saturating (values beyond the
largest finite one map to it), like the CUDA constructors TileFusion uses.
"""

from __future__ import annotations

import torch

from .._torch_ops import ensure_loaded

__all__ = ["fp8_quantize", "fp8_dequantize"]

_FP8 = (torch.float8_e4m3fn, torch.float8_e5m2)


def fp8_quantize(x: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn, factor: float = 1.0) -> torch.Tensor:
    """``fp8(x * factor)`` for a contiguous fp16/bf16 CUDA tensor ``x``; read it
    back with ``k_scale`` / ``v_scale`` ``= 1 / factor``."""
    if dtype not in _FP8:
        raise TypeError("dtype must be torch.float8_e4m3fn or torch.float8_e5m2")
    ensure_loaded()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    torch.ops.tilefusion.fp8_quantize(x.contiguous(), out, factor)
    return out


def fp8_dequantize(x: torch.Tensor, dtype: torch.dtype = torch.float16, factor: float = 1.0) -> torch.Tensor:
    """``dtype(float(x) * factor)`` for a contiguous float8 CUDA tensor ``x``."""
    if x.dtype not in _FP8:
        raise TypeError("x must be a torch.float8_e4m3fn or torch.float8_e5m2 tensor")
    ensure_loaded()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    torch.ops.tilefusion.fp8_dequantize(x.contiguous(), out, factor)
    return out
