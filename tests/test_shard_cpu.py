"""The multi-GPU host logic with two gloo ranks on CPU.

The CUDA operators are replaced by the oracle's split/combine restatement so
that slicing, slot layout and the all-gather plumbing run without a GPU.
"""

import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as orc
from tilefusion_b200.shard import ShardedDecoder, head_slice, kv_slice, prefill_sharded


def test_head_slice_partitions_exactly():
    for total, world in [(1024, 8), (1024, 3), (5, 8), (256, 1)]:
        spans = [head_slice(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        head_slice(8, 8, 8)


def test_kv_slice_is_aligned_and_complete():
    for lk, world in [(131072, 8), (5000, 4), (100, 8), (129, 2)]:
        spans = [kv_slice(lk, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == lk
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(b % 128 == 0 for b, e in spans if e > b)   # empty tail slices sit at len_kv


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_partial(q, k, v, slot, kv_chunk, num_splits, scale):
    b, h, _, d = q.shape
    po, pml = orc.decode_split(q.squeeze(2), k, v, scale, kv_chunk)
    _, _, merged = orc.decode_combine(po, pml)                      # [B, H, D+2]
    slot[: b * h * d] = merged[..., :d].reshape(-1)
    slot[b * h * d:] = merged[..., d:].reshape(-1)


def _oracle_gathered(slots, out, lse):
    b, h, _, d = out.shape
    n = slots.size(0)
    po = slots[:, : b * h * d].view(n, b, h, d).permute(1, 2, 0, 3)
    pml = slots[:, b * h * d:].view(n, b, h, 2).permute(1, 2, 0, 3)
    o, l, _ = orc.decode_combine(po, pml)
    out.copy_(o.unsqueeze(2).to(out.dtype))
    lse.copy_(l.unsqueeze(2))


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ---- decode sharded by KV length ----
        b, h, lk, d = 2, 3, 1500, 64
        q, k, v = orc.seeded_inputs(31, (b, h, 1, d), (b, h, lk, d), (b, h, lk, d), 1.0)
        k0, k1 = kv_slice(lk, rank, world)
        dec = ShardedDecoder(b, h, d, torch.float16, "cpu", kv_chunk=512,
                             partial_fn=_oracle_partial, gathered_fn=_oracle_gathered)
        o, lse = dec(q, k[:, :, k0:k1], v[:, :, k0:k1])
        ref, lse_ref = orc.decode_fp32(q, k, v)
        ok_dec = orc.max_abs(o, ref) <= 2e-3 and orc.max_abs(lse, lse_ref) <= 1e-4
        # every rank must hold every rank's slot after the in-place all-gather
        ok_gather = bool(torch.isfinite(dec.gather).all()) and dec.gather.shape == (world, b * h * (d + 2))

        # ---- prefill sharded by heads: no collective ----
        n, l = 5, 64
        q2, k2, v2 = orc.seeded_inputs(32, (n, l, d), (n, l, d), (n, l, d), 0.5)
        fn = lambda a, bb, c, s, causal: orc.attention_fp32(a, bb, c, s, causal)[0]
        out, (h0, h1) = prefill_sharded(q2, k2, v2, 0.125, False, attention_fn=fn)
        full = orc.attention_fp32(q2, k2, v2, 0.125)[0]
        ok_pre = orc.max_abs(out, full[h0:h1]) <= 1e-6 and (h0, h1) == head_slice(n, rank, world)
        ret[rank] = (ok_dec, ok_gather, ok_pre)
    finally:
        dist.destroy_process_group()


def test_two_rank_decode_and_prefill():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}
