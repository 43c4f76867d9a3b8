"""Flash decoding operator (split-KV partials + log-sum-exp combine).

TileFusion has no decode operator; this one is added next to
``flash_attention`` and registered with the dispatcher the same way.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .._torch_ops import ensure_loaded

__all__ = ["FlashDecoding", "flash_decoding"]


class FlashDecoding:
    """Callable holding the chunk size, split count and scale."""

    def __init__(self, kv_chunk: int = 0, num_splits: int = 0,
                 softmax_scale: Optional[float] = None, k_scale: float = 1.0, v_scale: float = 1.0) -> None:
        self.kv_chunk = kv_chunk
        self.num_splits = num_splits
        self.softmax_scale = softmax_scale
        self.k_scale = k_scale
        self.v_scale = v_scale

    def __call__(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                 block_table: Optional[torch.Tensor] = None,
                 kv_len: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``query [B, H, 1, D]``; ``key``/``value`` ``[B, H_kv, Lk, D]`` with ``H_kv``
        dividing ``H`` (grouped-query attention when smaller), or -- with
        ``block_table`` (int32 ``[B, max_pages]``) and ``kv_len`` -- a paged cache
        ``[num_pages, H_kv, page_size, D]`` whose page ``block_table[b, i]`` holds keys
        ``[i * page_size, (i + 1) * page_size)`` of batch entry ``b``.  ``key`` / ``value``
        may be ``torch.float8_e4m3fn`` or ``torch.float8_e5m2``: the cache is read as
        ``k_scale * key`` and ``v_scale * value`` (with grouped-query heads every query
        head then streams its KV head's bytes itself).

        Returns ``O [B, H, 1, D]`` and ``LSE [B, H, 1]`` (fp32, natural log).
        """
        ensure_loaded()
        scale = self.softmax_scale
        if scale is None:
            scale = 1.0 / math.sqrt(query.size(-1))
        b, h, _, d = query.shape
        out = torch.empty(b, h, 1, d, dtype=query.dtype, device=query.device)
        lse = torch.empty(b, h, 1, dtype=torch.float32, device=query.device)
        if block_table is not None:
            if kv_len is None:
                raise ValueError("kv_len is required with a block_table")
            torch.ops.tilefusion.flash_decoding_paged(
                query, key, value, block_table, kv_len, out, lse, self.kv_chunk, self.num_splits, scale,
                self.k_scale, self.v_scale
            )
            return out, lse
        torch.ops.tilefusion.flash_decoding(
            query, key, value, out, lse, self.kv_chunk, self.num_splits, scale, self.k_scale, self.v_scale
        )
        return out, lse


def flash_decoding(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                   kv_chunk: int = 0, num_splits: int = 0,
                   softmax_scale: Optional[float] = None, block_table: Optional[torch.Tensor] = None,
                   kv_len: Optional[int] = None, k_scale: float = 1.0,
                   v_scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """One-query-row attention over a long KV sequence.

    Args:
        query: ``[B, H, 1, D]``.
        key, value: ``[B, H_kv, Lk, D]``, rows contiguous (``H_kv`` divides ``H``); or
            pages ``[num_pages, H_kv, page_size, D]`` when ``block_table`` is given.
        kv_chunk: keys per chunk (multiple of 128, at most 1024); 0: 512, or 1024 for a
            ``float8`` cache.
        num_splits: partial rows per (batch, head); 0 lets the registry choose.
        softmax_scale: defaults to ``1/sqrt(D)``.
        block_table, kv_len: paged KV cache (``page_size`` a multiple of 128).
        k_scale, v_scale: dequantisation factors of a ``float8`` cache.
    """
    return FlashDecoding(kv_chunk, num_splits, softmax_scale, k_scale, v_scale)(query, key, value, block_table, kv_len)
