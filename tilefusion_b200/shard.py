"""Single-node multi-GPU layer: one process per GPU over ``torch.distributed``.

TileFusion has no distributed code; this layer adds the two partitionings the
attention path needs.

* Prefill shards by (batch x heads): the heads are independent problems, so a
  rank runs the same kernel on its contiguous slice and **no collective** is
  involved (``head_slice`` / ``prefill_sharded``).
* Long-context decode shards by KV length: every rank holds a contiguous slice
  of the keys and produces one partial ``(O, m, l)`` row per (batch, head);
  the rows of all ranks (``B*H*(D+2)`` fp32 each) are gathered over NVLink and
  every rank runs the log-sum-exp combine over them (``ShardedDecoder``).  Two
  transports: ``"p2p"`` -- the merge kernel stores its rows straight into every
  rank's symmetric-memory gather buffer and raises a flag there, and the
  combine kernel waits (bounded) on the flags, so the exchange is fused into
  the two kernels and no collective is launched; ``"nccl"`` -- the rows go to
  the local slot and one in-place ``all_gather_into_tensor`` moves them.

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

    ``transport="p2p"`` (default when symmetric memory can be set up): a
    symmetric buffer holds two gather areas ``[world, B*H*(D+2)]`` (alternated
    between consecutive steps, so a fast rank never overwrites rows a slow rank
    is still reading) and one flag word per sender.  ``transport="nccl"``: one
    gather buffer and an in-place all-gather.  Either way a step is stream-ordered
    on the current stream with no host synchronisation.
    """

    def __init__(self, batch: int, heads: int, head_dim: int, dtype: torch.dtype, device,
                 group=None, kv_chunk: int = 512, num_splits: int = 0,
                 partial_fn: Callable = _default_partial,
                 gathered_fn: Callable = _default_gathered, transport: Optional[str] = None) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.batch, self.heads, self.head_dim = batch, heads, head_dim
        self.dtype = dtype
        self.kv_chunk, self.num_splits = kv_chunk, num_splits
        self.slot_floats = batch * heads * (head_dim + 2)
        self._partial = partial_fn
        self._gathered = gathered_fn
        self._step = 0
        custom = partial_fn is not _default_partial or gathered_fn is not _default_gathered
        if transport is None:
            transport = "nccl" if (custom or self.world == 1) else "p2p"
        self.transport = transport
        if transport == "p2p":
            try:
                self._setup_symmetric(device)
            except Exception as exc:  # symmetric memory unavailable (no P2P mapping, old torch ...)
                self.transport = "nccl"
                self.transport_fallback_reason = f"{type(exc).__name__}: {exc}"
        if self.transport == "nccl":
            self.gather = torch.zeros(self.world, self.slot_floats, dtype=torch.float32, device=device)

    def _setup_symmetric(self, device) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        from ._torch_ops import ensure_loaded

        ensure_loaded()
        area = self.world * self.slot_floats
        self._flag_offset = 2 * area
        total = 2 * area + max(32, self.world)
        buf = symm_mem.empty(total, dtype=torch.float32, device=device)
        group = self.group if self.group is not None else dist.group.WORLD
        handle = symm_mem.rendezvous(buf, group)
        buf.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)      # every rank's flags are zero before any peer writes
        self._symm_buf, self._symm_handle = buf, handle
        self._peer_table = int(handle.buffer_ptrs_dev)
        self._areas = [buf[i * area:(i + 1) * area].view(self.world, self.slot_floats) for i in range(2)]
        self._flags = buf[self._flag_offset:self._flag_offset + self.world].view(torch.int32)
        self.gather = self._areas[0]

    def __call__(self, query: torch.Tensor, key_local: torch.Tensor, value_local: torch.Tensor,
                 softmax_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``query [B, H, 1, D]`` (replicated), ``key_local``/``value_local``
        ``[B, H, Lk_local, D]``.  Returns ``O [B, H, 1, D]`` and ``LSE [B, H, 1]``
        on every rank."""
        scale = 1.0 / math.sqrt(self.head_dim) if softmax_scale is None else softmax_scale
        out = torch.empty(self.batch, self.heads, 1, self.head_dim, dtype=self.dtype, device=query.device)
        lse = torch.empty(self.batch, self.heads, 1, dtype=torch.float32, device=query.device)
        if self.transport == "p2p":
            self._step += 1
            parity = self._step & 1
            slot_offset = (parity * self.world + self.rank) * self.slot_floats
            torch.ops.tilefusion.flash_decoding_partial_scatter(
                query, key_local, value_local, self._peer_table, self.rank, self.world, slot_offset,
                self._flag_offset, self._step, self.kv_chunk, self.num_splits, scale)
            self.gather = self._areas[parity]
            torch.ops.tilefusion.flash_decoding_gathered_wait(self.gather, self._flags, self._step, out, lse)
            return out, lse
        slot = self.gather[self.rank]
        self._partial(query, key_local, value_local, slot, self.kv_chunk, self.num_splits, scale)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gather.view(-1), slot, group=self.group)
        self._gathered(self.gather, out, lse)
        return out, lse
