"""Parity of the CUDA flash-decoding kernels with the oracle, through the C-ABI.

Tolerances: max-abs <= 2e-2, relative-L2 <= 1e-3 for fp16; for bf16 outputs,
whose rounding alone is ~1.7e-3, the bound is computed from the reference
(oracle.rel_l2_bound: 1.15 x the rounding floor of the exact result, in
quadrature with the rounding of P where the tensor-core path rounds it);
|LSE error| <= 1e-3; fp32 partials are compared with relative-L2 <= 1e-5.
"""

import math

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
REL_L2_FP16 = 1e-3
LSE_ABS = 1e-3


def _inputs(seed, b, h, lk, d, dtype=torch.float16):
    return orc.seeded_inputs(seed, (b, h, 1, d), (b, h, lk, d), (b, h, lk, d), 1.0, dtype)


def _check(o, lse, ref_o, ref_lse, dtype, p_rounded=False):
    """p_rounded: the grouped-query path runs on the tensor cores and rounds P to
    the 16-bit dtype; the one-head-per-KV-head kernel keeps P in fp32."""
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    assert orc.max_abs(o.cpu(), ref_o) <= MAX_ABS
    assert orc.rel_l2(o.cpu(), ref_o) <= orc.rel_l2_bound(ref_o, dtype, p_rounded)
    assert orc.max_abs(lse.cpu(), ref_lse) <= LSE_ABS


CASES = [
    # B, H, Lk, D, kv_chunk, num_splits
    (1, 1, 512, 128, 512, 0),
    (2, 3, 1000, 128, 512, 0),     # ragged last chunk and stage
    (1, 2, 1, 128, 512, 0),        # a single key
    (2, 2, 130, 64, 128, 0),
    (4, 8, 4096, 128, 512, 0),
    (4, 8, 4096, 128, 512, 3),     # 8 chunks over 3 splits: uneven splits
    (1, 4, 3000, 64, 256, 0),
    (2, 2, 2048, 128, 1024, 1),    # one split walks two chunks: running (m, l)
    (3, 5, 777, 128, 128, 0),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c)))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_decode_matches_oracle(case, dtype):
    from cabi_helpers import decode, device_status

    b, h, lk, d, chunk, splits = case
    q, k, v = _inputs(21, b, h, lk, d, dtype)
    o, lse = decode(q.cuda(), k.cuda(), v.cuda(), None, chunk, splits)
    ref, lse_ref = orc.decode_fp32(q, k, v)
    _check(o, lse, ref, lse_ref, dtype)
    assert device_status() == 0


@pytest.mark.parametrize("lk,chunk,splits", [(4096, 512, 0), (1000, 256, 2), (2048, 512, 1)])
def test_split_partials_match_oracle(lk, chunk, splits):
    from cabi_helpers import decode_split

    b, h, d = 2, 4, 128
    q, k, v = _inputs(22, b, h, lk, d)
    part_o, part_ml, plan = decode_split(q.cuda(), k.cuda(), v.cuda(), None, chunk, splits)
    ref_o, ref_ml = orc.decode_split(q.squeeze(2), k, v, 1.0 / math.sqrt(d), plan.kv_chunk * plan.chunks_per_split)
    assert part_o.shape == ref_o.shape
    # m is a maximum over the same keys; l and O are sums in a different order
    assert orc.max_abs(part_ml[..., 0].cpu(), ref_ml[..., 0]) <= 1e-4
    assert orc.rel_l2(part_ml[..., 1].cpu(), ref_ml[..., 1]) <= 1e-5
    assert orc.rel_l2(part_o.cpu(), ref_o) <= 1e-5


@pytest.mark.parametrize("n_shards", [2, 4, 8])
def test_sharded_partial_then_gathered(n_shards):
    """The multi-GPU decode path on one GPU: each KV shard writes its slot, the
    gathered combine merges them (the all-gather is the identity here)."""
    from cabi_helpers import decode_gathered, decode_partial_into
    from tilefusion_b200.shard import kv_slice

    b, h, lk, d = 2, 4, 5000, 128
    q, k, v = _inputs(23, b, h, lk, d)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    slots = torch.full((n_shards, b * h * (d + 2)), float("nan"), dtype=torch.float32, device="cuda")
    for r in range(n_shards):
        k0, k1 = kv_slice(lk, r, n_shards)
        decode_partial_into(qc, kc[:, :, k0:k1].contiguous(), vc[:, :, k0:k1].contiguous(), slots[r])
    o, lse = decode_gathered(slots, b, h, d, torch.float16)
    ref, lse_ref = orc.decode_fp32(q, k, v)
    _check(o, lse, ref, lse_ref, torch.float16)


def test_empty_shard_contributes_nothing():
    from cabi_helpers import decode_gathered, decode_partial_into

    b, h, lk, d = 1, 2, 300, 128
    q, k, v = _inputs(24, b, h, lk, d)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    slots = torch.full((2, b * h * (d + 2)), float("nan"), dtype=torch.float32, device="cuda")
    decode_partial_into(qc, kc, vc, slots[0])
    decode_partial_into(qc, kc[:, :, :0].contiguous(), vc[:, :, :0].contiguous(), slots[1])
    o, lse = decode_gathered(slots, b, h, d, torch.float16)
    ref, lse_ref = orc.decode_fp32(q, k, v)
    _check(o, lse, ref, lse_ref, torch.float16)


GQA_CASES = [
    # B, Hq, Hkv, Lk, D
    (2, 8, 2, 1000, 128),      # group of 4, ragged last tile
    (1, 8, 1, 4096, 128),      # multi-query: all 8 heads share one KV head
    (3, 6, 3, 130, 64),        # group of 2, D = 64
    (2, 32, 8, 8192, 128),
    (1, 16, 2, 1, 128),        # a single key: three of the four row copies see no key at all
    (1, 64, 2, 700, 128),      # group of 32: the largest that is replicated in the lane quarters
    (1, 128, 2, 700, 128),     # group of 64: not replicated
    (2, 12, 4, 40, 64),        # fewer keys than one quarter holds in the last copy
]


@pytest.mark.parametrize("case", GQA_CASES, ids=lambda c: "x".join(map(str, c)))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_grouped_query_decode(case, dtype):
    """Query heads that share a KV head (K/V are [B, H_kv, Lk, D])."""
    from cabi_helpers import decode, device_status

    b, hq, hkv, lk, d = case
    q, k, v = orc.seeded_inputs(27, (b, hq, 1, d), (b, hkv, lk, d), (b, hkv, lk, d), 1.0, dtype)
    o, lse = decode(q.cuda(), k.cuda(), v.cuda())
    g = hq // hkv
    ref, lse_ref = orc.decode_fp32(q, k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1))
    _check(o, lse, ref, lse_ref, dtype, p_rounded=True)
    assert device_status() == 0


def test_grouped_query_python_api():
    import tilefusion_b200 as tilefusion

    q, k, v = orc.seeded_inputs(28, (2, 16, 1, 128), (2, 4, 3000, 128), (2, 4, 3000, 128), 1.0)
    o, lse = tilefusion.ops.flash_decoding(q.cuda(), k.cuda(), v.cuda())
    ref, lse_ref = orc.decode_fp32(q, k.repeat_interleave(4, dim=1), v.repeat_interleave(4, dim=1))
    _check(o, lse, ref, lse_ref, torch.float16)


def _paginate(k, v, page_size, seed):
    """Scatters contiguous K/V [B, H, Lk, D] into a shuffled page pool; returns
    (k_pages, v_pages, block_table).  Unused rows of the last page are zero."""
    b, h, lk, d = k.shape
    per_seq = -(-lk // page_size)
    n_pages = b * per_seq + 3                        # a few pages nobody uses
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g)[: b * per_seq].view(b, per_seq)
    kp = torch.zeros(n_pages, h, page_size, d, dtype=k.dtype)
    vp = torch.zeros_like(kp)
    for bi in range(b):
        for i in range(per_seq):
            n = min(page_size, lk - i * page_size)
            kp[perm[bi, i], :, :n] = k[bi, :, i * page_size:i * page_size + n]
            vp[perm[bi, i], :, :n] = v[bi, :, i * page_size:i * page_size + n]
    return kp, vp, perm.to(torch.int32)


@pytest.mark.parametrize("case", [
    # B, Hq, Hkv, Lk, D, page_size
    (2, 4, 4, 1000, 128, 256),      # MHA, ragged last page
    (3, 4, 4, 4096, 128, 512),
    (2, 8, 2, 1500, 128, 128),      # grouped-query, one tile per page
    (2, 8, 2, 3000, 64, 1024),
], ids=lambda c: "x".join(map(str, c)))
def test_paged_kv_cache(case):
    import tilefusion_b200 as tilefusion

    b, hq, hkv, lk, d, page = case
    q, k, v = orc.seeded_inputs(29, (b, hq, 1, d), (b, hkv, lk, d), (b, hkv, lk, d), 1.0)
    kp, vp, table = _paginate(k, v, page, 5)
    o, lse = tilefusion.ops.flash_decoding(q.cuda(), kp.cuda(), vp.cuda(), block_table=table.cuda(), kv_len=lk)
    g = hq // hkv
    ref, lse_ref = orc.decode_fp32(q, k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1))
    _check(o, lse, ref, lse_ref, torch.float16)


def test_python_api_matches_oracle():
    import tilefusion_b200 as tilefusion

    q, k, v = _inputs(25, 2, 4, 2500, 128)
    o, lse = tilefusion.ops.flash_decoding(q.cuda(), k.cuda(), v.cuda())
    ref, lse_ref = orc.decode_fp32(q, k, v)
    assert o.shape == (2, 4, 1, 128) and lse.shape == (2, 4, 1)
    _check(o, lse, ref, lse_ref, torch.float16)


def test_config3_size_properties_and_subset():
    """Full decode config (B32 H32 Lk8192 D128, seed 2): a subset of (b, h)
    against the CPU oracle, all of them against the fp32 expression on the GPU,
    and the V = 1 property."""
    from cabi_helpers import decode, device_status

    b, h, lk, d = 32, 32, 8192, 128
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(b, h, 1, d, generator=g, device="cuda").half()
    k = torch.randn(b, h, lk, d, generator=g, device="cuda").half()
    v = torch.randn(b, h, lk, d, generator=g, device="cuda").half()
    o, lse = decode(q, k, v)
    assert device_status() == 0
    for (bi, hi) in [(0, 0), (13, 7), (31, 31)]:
        ref, lse_ref = orc.decode_fp32(q[bi:bi + 1, hi:hi + 1].cpu(), k[bi:bi + 1, hi:hi + 1].cpu(),
                                       v[bi:bi + 1, hi:hi + 1].cpu())
        _check(o[bi:bi + 1, hi:hi + 1], lse[bi:bi + 1, hi:hi + 1], ref, lse_ref, torch.float16)
    worst, num, den = 0.0, 0.0, 0.0
    for bi in range(b):
        ref, lse_ref = orc.decode_fp32(q[bi:bi + 1], k[bi:bi + 1], v[bi:bi + 1])
        diff = o[bi:bi + 1].float() - ref
        worst = max(worst, diff.abs().max().item())
        num += diff.double().pow(2).sum().item()
        den += ref.double().pow(2).sum().item()
        assert (lse[bi:bi + 1] - lse_ref).abs().max().item() <= LSE_ABS
    assert worst <= MAX_ABS and math.sqrt(num / den) <= REL_L2_FP16
    o1, _ = decode(q[:2], k[:2], torch.ones_like(v[:2]))
    assert (o1.float() - 1.0).abs().max().item() <= 2e-3


def test_config4_size_subset_sharded_and_properties():
    """Long-context decode config (B4 H32 Lk131072 D128, seed 3): the full 8 GiB
    problem on one GPU against the fp32 expression on the GPU for every (b, h),
    the CPU oracle on one of them, and the same problem through the KV-sharded
    path (8 shards written into slots, then the gathered combine)."""
    from cabi_helpers import decode, decode_gathered, decode_partial_into, device_status
    from tilefusion_b200.shard import kv_slice

    free, _ = torch.cuda.mem_get_info()
    if free < 12 << 30:
        pytest.skip("needs 12 GiB of free device memory")
    b, h, lk, d = 4, 32, 131072, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(b, h, 1, d, generator=g, device="cuda").half()
    k = torch.empty(b, h, lk, d, dtype=torch.float16, device="cuda")
    v = torch.empty_like(k)
    for t in (k, v):
        for bi in range(b):
            t[bi] = torch.randn(h, lk, d, generator=g, device="cuda").half()
    o, lse = decode(q, k, v)
    assert device_status() == 0
    worst, num, den = 0.0, 0.0, 0.0
    for bi in range(b):
        for h0 in range(0, h, 8):
            ref, lse_ref = orc.decode_fp32(q[bi:bi + 1, h0:h0 + 8], k[bi:bi + 1, h0:h0 + 8], v[bi:bi + 1, h0:h0 + 8])
            diff = o[bi:bi + 1, h0:h0 + 8].float() - ref
            worst = max(worst, diff.abs().max().item())
            num += diff.double().pow(2).sum().item()
            den += ref.double().pow(2).sum().item()
            assert (lse[bi:bi + 1, h0:h0 + 8] - lse_ref).abs().max().item() <= LSE_ABS
    assert worst <= MAX_ABS and math.sqrt(num / den) <= REL_L2_FP16
    ref, lse_ref = orc.decode_fp32(q[2:3, 5:6].cpu(), k[2:3, 5:6].cpu(), v[2:3, 5:6].cpu())
    _check(o[2:3, 5:6], lse[2:3, 5:6], ref, lse_ref, torch.float16)
    # the sharded path on the same tensors (views of the shards, no copies)
    n_shards = 8
    slots = torch.full((n_shards, b * h * (d + 2)), float("nan"), dtype=torch.float32, device="cuda")
    for r in range(n_shards):
        k0, k1 = kv_slice(lk, r, n_shards)
        decode_partial_into(q, k[:, :, k0:k1], v[:, :, k0:k1], slots[r])
    o2, lse2 = decode_gathered(slots, b, h, d, torch.float16)
    assert (o2.float() - o.float()).abs().max().item() <= 2e-3
    assert (lse2 - lse).abs().max().item() <= 1e-4


def test_bad_arguments_report_errors():
    from cabi_helpers import decode
    from tilefusion_b200._cabi import TileFusionError, TF_ERR_UNSUPPORTED

    q, k, v = _inputs(26, 1, 1, 256, 128)
    with pytest.raises(TileFusionError) as e:
        decode(q.cuda(), k.cuda(), v.cuda(), None, 100, 0)
    assert e.value.code == TF_ERR_UNSUPPORTED and "kv_chunk" in str(e.value)


def test_missing_peer_is_reported_not_hung():
    """Failure detection: the combine of a KV-sharded decode waits for a flag per
    sending rank.  Here one sender never shows up (its flag stays 0); the bounded
    wait must give up, the kernel must return NaN rows rather than a plausible
    result, the status word (and its host-visible mirror, without a
    synchronisation) must name the wait, and the context must stay usable."""
    import ctypes as C
    import time

    from cabi_helpers import decode, device_status
    from tilefusion_b200 import _cabi

    lib = _cabi.lib()
    assert lib.tf_set_wait_limit_ms(0) == _cabi.TF_ERR_BAD_ARG
    assert lib.tf_set_wait_limit_ms(300) == 0       # the limit is configurable; 0.3 s keeps the test short
    try:
        b, h, d, n_ranks = 1, 2, 128, 2
        slots = torch.zeros(n_ranks, b * h * (d + 2), dtype=torch.float32, device="cuda")
        flags = torch.zeros(n_ranks, dtype=torch.int32, device="cuda")
        flags[0] = 1                                   # rank 0 "arrived", rank 1 never does
        o = torch.zeros(b, h, 1, d, dtype=torch.float16, device="cuda")
        lse = torch.zeros(b, h, 1, dtype=torch.float32, device="cuda")
        t0 = time.perf_counter()
        rc = lib.tf_decode_gathered_wait(slots.data_ptr(), flags.data_ptr(), n_ranks, 1, b, h, d, _cabi.TF_F16,
                                         o.data_ptr(), o.stride(0), o.stride(1), lse.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
        assert rc == 0                                 # the launch itself succeeds
        # the host sees the failure without synchronising: poll the mirror word
        code = C.c_int32(0)
        while lib.tf_device_status_peek(C.byref(code)) == 0 and time.perf_counter() - t0 < 10.0:
            time.sleep(0.01)
        assert code.value == 401 and time.perf_counter() - t0 < 5.0
        assert "earlier launch gave up" in lib.tf_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isnan(o.float()).all() and torch.isnan(lse).all()   # no plausible-looking garbage
        rc = lib.tf_device_status(C.byref(code))       # synchronises, reports and clears
        assert rc == _cabi.TF_ERR_DEVICE_TIMEOUT and code.value == 401
        assert "wait gave up" in lib.tf_last_error().decode()
        assert device_status() == 0                    # the word is cleared by the read
        assert lib.tf_device_status_peek(C.byref(code)) == 0 and code.value == 0
    finally:
        assert lib.tf_set_wait_limit_ms(2000) == 0
    # the context is intact: an ordinary decode still runs and is correct
    q, k, v = _inputs(30, 1, 2, 512, 128)
    out, l2 = decode(q.cuda(), k.cuda(), v.cuda())
    ref, lse_ref = orc.decode_fp32(q, k, v)
    _check(out, l2, ref, lse_ref, torch.float16)


@pytest.mark.parametrize("transport", ["p2p", "nccl"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_sharded_context_single_rank(transport, dtype):
    """tf_shard_create / tf_decode_sharded with a world of one: the p2p transport
    runs split, merge, exchange and final combine in ONE launch (the rank is its
    own only peer), the nccl transport runs the fused merge into the local slot
    and the gathered combine.  Several steps reuse the two gather areas, the
    flags and the arrival counters; a second, longer problem grows the workspace."""
    from cabi_helpers import device_status
    from tilefusion_b200.shard import ShardedDecoder

    b, h, d = 2, 8, 128
    dec = ShardedDecoder(b, h, d, dtype, "cuda", transport=transport)
    assert dec.transport == transport and dec.world == 1
    try:
        for step, lk in enumerate([3000, 3000, 700, 9000, 9000]):
            q, k, v = _inputs(60 + step, b, h, lk, d, dtype)
            out = torch.full((b, h, 1, d), float("nan"), dtype=dtype, device="cuda")
            lse = torch.full((b, h, 1), float("nan"), dtype=torch.float32, device="cuda")
            dec(q.cuda(), k.cuda(), v.cuda(), out=out, lse=lse)
            ref, lse_ref = orc.decode_fp32(q, k, v)
            _check(out, lse, ref, lse_ref, dtype)
        assert device_status() == 0
    finally:
        dec.close()


def test_sharded_context_grouped_query_and_head_dim_64():
    """The grouped-query form takes the three-launch route through the same
    context; head_dim 64 takes the fused one."""
    from cabi_helpers import device_status
    from tilefusion_b200.shard import ShardedDecoder

    b, hq, hkv, lk, d = 2, 8, 2, 2048, 128
    q, _, _ = _inputs(70, b, hq, 128, d)
    _, k, v = _inputs(71, b, hkv, lk, d)
    dec = ShardedDecoder(b, hq, d, torch.float16, "cuda", transport="p2p")
    try:
        for _ in range(3):
            out, lse = dec(q.cuda(), k.cuda(), v.cuda())
        ref, lse_ref = orc.decode_fp32(q, k.repeat_interleave(hq // hkv, 1), v.repeat_interleave(hq // hkv, 1))
        _check(out, lse, ref, lse_ref, torch.float16)
    finally:
        dec.close()
    q, k, v = _inputs(72, 3, 5, 1500, 64)
    dec = ShardedDecoder(3, 5, 64, torch.float16, "cuda")
    try:
        for _ in range(2):
            out, lse = dec(q.cuda(), k.cuda(), v.cuda())
        ref, lse_ref = orc.decode_fp32(q, k, v)
        _check(out, lse, ref, lse_ref, torch.float16)
        assert device_status() == 0
    finally:
        dec.close()
