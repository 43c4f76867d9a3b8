"""Single-node multi-GPU layer: one process per GPU.

TileFusion has no distributed code; this layer adds the two partitionings the
attention path needs.  The host logic lives in the native library
(``csrc/shard.cc``: ``tf_shard_*``, ``tf_decode_sharded``, ``tf_prefill_sharded``);
this module is its torch-facing caller.

* Prefill shards by (batch x heads): the heads are independent problems, so a
  rank runs the same kernel on its contiguous slice and **no collective** is
  involved (``head_slice`` / ``prefill_sharded``).
* Long-context decode shards by KV length: every rank holds a contiguous slice
  of the keys and produces one partial ``(O, m, l)`` row per (batch, head);
  the rows of all ranks (``B*H*(D+2)`` fp32 each) are exchanged over NVLink and
  every rank ends with the full answer (``ShardedDecoder``).  Two transports:
  ``"p2p"`` -- one kernel launch per step: the decode kernel stores its merged
  rows straight into every rank's gather buffer (mapped through CUDA IPC),
  raises a flag there, waits (bounded) for the other ranks' flags and writes
  the result; ``"nccl"`` -- the rows go to the local slot, one in-place
  ``ncclAllGather`` moves them and a combine kernel finishes.

``torch.distributed`` is used once, to carry the 128-byte NCCL id from rank 0
to the others when a decoder is created.  The compute steps are parameters of
``ShardedDecoder`` only so that the slicing and gather plumbing can be
exercised with ``gloo`` ranks on a machine without GPUs.
"""

from __future__ import annotations

import ctypes as C
import math
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["head_slice", "kv_slice", "prefill_sharded", "ShardedDecoder"]


def _slice_call(fn_name: str, *args) -> Tuple[int, int]:
    from . import _cabi

    b, e = C.c_int64(0), C.c_int64(0)
    rc = getattr(_cabi.lib(), fn_name)(*args, C.byref(b), C.byref(e))
    if rc != 0:
        raise ValueError(_cabi.lib().tf_last_error().decode())
    return b.value, e.value


def head_slice(n_heads_total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous ``[begin, end)`` slice of the flattened (batch x heads) axis
    (``tf_shard_head_slice``)."""
    return _slice_call("tf_shard_head_slice", n_heads_total, rank, world)


def kv_slice(len_kv: int, rank: int, world: int, align: int = 128) -> Tuple[int, int]:
    """Contiguous ``[begin, end)`` slice of the key axis, boundaries on
    multiples of ``align`` keys; trailing ranks may be empty (``tf_shard_kv_slice``)."""
    return _slice_call("tf_shard_kv_slice", len_kv, rank, world, align)


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


class ShardedDecoder:
    """Flash decoding with the KV sequence sharded across the ranks of a group.

    By default a thin wrapper around a native ``TfShardCtx``: creation is
    collective (NCCL communicator, gather buffers mapped into every process for
    ``transport="p2p"``), a step is one ``tf_decode_sharded`` call on the
    current stream -- no host synchronisation and no allocation except for the
    caller-visible ``O`` / ``LSE`` (pass ``out=`` / ``lse=`` to reuse them).

    With ``partial_fn`` / ``gathered_fn`` given, the compute steps are the
    caller's and the rows travel through ``torch.distributed`` (any backend);
    this is how the host logic is tested without GPUs.
    """

    def __init__(self, batch: int, heads: int, head_dim: int, dtype: torch.dtype, device,
                 group=None, kv_chunk: int = 512, num_splits: int = 0,
                 partial_fn: Optional[Callable] = None,
                 gathered_fn: Optional[Callable] = None, transport: Optional[str] = None,
                 k_scale: float = 1.0, v_scale: float = 1.0) -> None:
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.batch, self.heads, self.head_dim = batch, heads, head_dim
        self.dtype = dtype
        self.kv_chunk, self.num_splits = kv_chunk, num_splits
        self.k_scale, self.v_scale = k_scale, v_scale     # dequantisation factors of a float8 cache
        self.slot_floats = batch * heads * (head_dim + 2)
        self._partial, self._gathered = partial_fn, gathered_fn
        self._ctx = None
        self.transport_note = ""
        if partial_fn is not None or gathered_fn is not None:
            if partial_fn is None or gathered_fn is None:
                raise ValueError("partial_fn and gathered_fn must be given together")
            self.transport = "collective"
            self.gather = torch.zeros(self.world, self.slot_floats, dtype=torch.float32, device=device)
            return
        self._create_native(torch.device(device), transport)

    # ------------------------------------------------------------- native ctx --
    def _create_native(self, device: torch.device, transport: Optional[str]) -> None:
        from . import _cabi

        if transport not in (None, "p2p", "nccl"):
            raise ValueError(f"transport must be 'p2p', 'nccl' or None, got {transport!r}")
        lib = _cabi.lib()
        ident = torch.zeros(_cabi.TF_NCCL_ID_BYTES, dtype=torch.uint8)
        if self.world > 1:
            if self.rank == 0:
                buf = (C.c_ubyte * _cabi.TF_NCCL_ID_BYTES)()
                _cabi.check(lib.tf_shard_unique_id(buf))
                ident = torch.tensor(list(buf), dtype=torch.uint8)
            # the id travels over the group's own backend (device tensors for NCCL)
            carrier = ident.to(device) if dist.get_backend(self.group) == "nccl" else ident
            src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
            dist.broadcast(carrier, src=src, group=self.group)
            ident = carrier.cpu()
        id_bytes = (C.c_ubyte * _cabi.TF_NCCL_ID_BYTES)(*ident.tolist())
        code = {None: _cabi.TF_TRANSPORT_AUTO, "p2p": _cabi.TF_TRANSPORT_P2P, "nccl": _cabi.TF_TRANSPORT_NCCL}[transport]
        dtype_code = {torch.float16: _cabi.TF_F16, torch.bfloat16: _cabi.TF_BF16}[self.dtype]
        ctx = C.c_void_p()
        with torch.cuda.device(device):
            rc = lib.tf_shard_create(self.rank, self.world, id_bytes if self.world > 1 else None, code,
                                     self.batch, self.heads, self.head_dim, dtype_code, C.byref(ctx))
        _cabi.check(rc)
        self._ctx = ctx
        self._lib = lib
        self._device = device
        self.transport = "p2p" if lib.tf_shard_transport(ctx) == _cabi.TF_TRANSPORT_P2P else "nccl"
        self.transport_note = lib.tf_shard_note(ctx).decode()

    def close(self) -> None:
        """Frees the native context.  Every rank calls it, after the last step
        of every rank has completed (e.g. behind a barrier)."""
        if self._ctx is not None:
            with torch.cuda.device(self._device):
                self._lib.tf_shard_destroy(self._ctx)
            self._ctx = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ step --
    def __call__(self, query: torch.Tensor, key_local: torch.Tensor, value_local: torch.Tensor,
                 softmax_scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                 lse: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``query [B, H, 1, D]`` (replicated), ``key_local``/``value_local``
        ``[B, H_kv, Lk_local, D]`` in the query's dtype, or ``float8_e4m3fn`` /
        ``float8_e5m2`` with ``H_kv == H`` (read as ``k_scale * key``, ``v_scale * value``).
        Returns ``O [B, H, 1, D]`` and ``LSE [B, H, 1]`` on every rank."""
        scale = 1.0 / math.sqrt(self.head_dim) if softmax_scale is None else softmax_scale
        if out is None:
            out = torch.empty(self.batch, self.heads, 1, self.head_dim, dtype=self.dtype, device=query.device)
        if lse is None:
            lse = torch.empty(self.batch, self.heads, 1, dtype=torch.float32, device=query.device)
        if self._ctx is None:
            slot = self.gather[self.rank]
            self._partial(query, key_local, value_local, slot, self.kv_chunk, self.num_splits, scale)
            if self.world > 1:
                dist.all_gather_into_tensor(self.gather.view(-1), slot, group=self.group)
            self._gathered(self.gather, out, lse)
            return out, lse
        from . import _cabi

        d = _cabi.TfDecodeDesc()
        d.dtype = _cabi.TF_F16 if self.dtype == torch.float16 else _cabi.TF_BF16
        d.batch, d.heads, d.head_dim = self.batch, self.heads, self.head_dim
        d.heads_kv = key_local.size(1)
        d.len_kv = key_local.size(2)
        d.kv_chunk, d.num_splits, d.softmax_scale = self.kv_chunk, self.num_splits, scale
        fp8 = {torch.float8_e4m3fn: _cabi.TF_FP8_E4M3, torch.float8_e5m2: _cabi.TF_FP8_E5M2}.get(key_local.dtype)
        if fp8 is not None:
            d.kv_dtype, d.k_scale, d.v_scale = fp8, self.k_scale, self.v_scale
        d.q_stride_b, d.q_stride_h = query.stride(0), query.stride(1)
        d.k_stride_b, d.k_stride_h = key_local.stride(0), key_local.stride(1)
        d.v_stride_b, d.v_stride_h = value_local.stride(0), value_local.stride(1)
        d.o_stride_b, d.o_stride_h = out.stride(0), out.stride(1)
        has_keys = key_local.numel() > 0
        if has_keys and (key_local.stride(3) != 1 or key_local.stride(2) != self.head_dim or
                         value_local.stride(3) != 1 or value_local.stride(2) != self.head_dim):
            raise ValueError("rows of key_local / value_local must be contiguous and D elements apart")
        rc = self._lib.tf_decode_sharded(
            self._ctx, query.data_ptr(), key_local.data_ptr() if has_keys else None,
            value_local.data_ptr() if has_keys else None, out.data_ptr(), lse.data_ptr(), C.byref(d),
            torch.cuda.current_stream(query.device).cuda_stream)
        _cabi.check(rc)
        return out, lse
