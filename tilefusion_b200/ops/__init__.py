"""Attention operators (mirrors TileFusion's ``python/ops/__init__.py``)."""

from .flash_attention import FlashAttention, flash_attention, flash_attention_autograd, flash_attention_bwd
from .flash_decoding import FlashDecoding, flash_decoding
from .fp8 import fp8_dequantize, fp8_quantize
from .fused_two_gemms import fused_two_gemms

__all__ = ["FlashAttention", "flash_attention", "flash_attention_bwd", "flash_attention_autograd",
           "FlashDecoding", "flash_decoding", "fused_two_gemms", "fp8_quantize", "fp8_dequantize"]
