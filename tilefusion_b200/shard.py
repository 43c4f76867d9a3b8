"""Single-node multi-GPU layer: one process per GPU over ``torch.distributed``.

TileFusion has no distributed code; this layer adds the two partitionings the
attention path needs.

* Prefill shards by (batch x heads): the heads are independent problems, so a
  rank runs the same kernel on its contiguous slice and **no collective** is
  involved (``head_slice`` / ``prefill_sharded``).
* Long-context decode shards by KV length: every rank holds a contiguous slice
  of the keys, produces one partial ``(O, m, l)`` row per (batch, head) written
  straight into its slot of a gather buffer, one NCCL all-gather (in place)
  moves ``B*H*(D+2)`` fp32 per rank over NVLink, and every rank then runs the
  log-sum-exp combine over the gathered slots (``ShardedDecoder``).

The compute steps are the CUDA operators; they are parameters only so that
the host logic (slicing, buffer layout, collective plumbing) can be exercised
with ``gloo`` ranks on a machine without GPUs.
"""

from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["head_slice", "kv_slice", "prefill_sharded", "ShardedDecoder"]


def head_slice(n_heads_total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous ``[begin, end)`` slice of the flattened (batch x heads) axis."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_heads_total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def kv_slice(len_kv: int, rank: int, world: int, align: int = 128) -> Tuple[int, int]:
    """Contiguous ``[begin, end)`` slice of the key axis, boundaries on
    multiples of ``align`` keys (the last rank takes the ragged tail)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    blocks = (len_kv + align - 1) // align
    b0, b1 = head_slice(blocks, rank, world)
    return min(len_kv, b0 * align), min(len_kv, b1 * align)


def _default_attention(q, k, v, scale, causal):
    from .ops.flash_attention import FlashAttention

    # q [n, Lq, D], k [n, Lk, D], v [n, Lk, Dv]; the operator wants key as [.., D, Lk]
    return FlashAttention(0, 0, 0, 0, scale, causal)(q, k.transpose(-1, -2), v)


def prefill_sharded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
                    causal: bool = False, rank: Optional[int] = None, world: Optional[int] = None,
                    attention_fn: Callable = _default_attention) -> Tuple[torch.Tensor, Tuple[int, int]]:
    """Runs this rank's slice of a ``[BH, L, D]`` problem; no communication.

    ``q``, ``k``, ``v`` are the full (or already local) tensors flattened over
    (batch x heads).  Returns the local output and the slice it covers.
    """
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    b0, b1 = head_slice(q.size(0), rank, world)
    out = attention_fn(q[b0:b1], k[b0:b1], v[b0:b1], softmax_scale, causal)
    return out, (b0, b1)


def _default_partial(q, k, v, slot, kv_chunk, num_splits, scale):
    from ._torch_ops import ensure_loaded

    ensure_loaded()
    torch.ops.tilefusion.flash_decoding_partial(q, k, v, slot, kv_chunk, num_splits, scale)


def _default_gathered(slots, out, lse):
    from ._torch_ops import ensure_loaded

    ensure_loaded()
    torch.ops.tilefusion.flash_decoding_gathered(slots, out, lse)


class ShardedDecoder:
    """Flash decoding with the KV sequence sharded across the ranks of a group.

    The gather buffer ``[world, B*H*(D+2)]`` fp32 is allocated once; a step is
    partial kernel -> in-place all-gather -> combine kernel, all stream-ordered
    on the current stream with no host synchronisation.
    """

    def __init__(self, batch: int, heads: int, head_dim: int, dtype: torch.dtype, device,
                 group=None, kv_chunk: int = 512, num_splits: int = 0,
                 partial_fn: Callable = _default_partial,
                 gathered_fn: Callable = _default_gathered) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.batch, self.heads, self.head_dim = batch, heads, head_dim
        self.dtype = dtype
        self.kv_chunk, self.num_splits = kv_chunk, num_splits
        self.slot_floats = batch * heads * (head_dim + 2)
        self.gather = torch.zeros(self.world, self.slot_floats, dtype=torch.float32, device=device)
        self._partial = partial_fn
        self._gathered = gathered_fn

    def __call__(self, query: torch.Tensor, key_local: torch.Tensor, value_local: torch.Tensor,
                 softmax_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``query [B, H, 1, D]`` (replicated), ``key_local``/``value_local``
        ``[B, H, Lk_local, D]``.  Returns ``O [B, H, 1, D]`` and ``LSE [B, H, 1]``
        on every rank."""
        scale = 1.0 / math.sqrt(self.head_dim) if softmax_scale is None else softmax_scale
        slot = self.gather[self.rank]
        self._partial(query, key_local, value_local, slot, self.kv_chunk, self.num_splits, scale)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gather.view(-1), slot, group=self.group)
        out = torch.empty(self.batch, self.heads, 1, self.head_dim, dtype=self.dtype, device=query.device)
        lse = torch.empty(self.batch, self.heads, 1, dtype=torch.float32, device=query.device)
        self._gathered(self.gather, out, lse)
        return out, lse
