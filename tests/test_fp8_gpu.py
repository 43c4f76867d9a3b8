"""8-bit K/V storage on the GPU, through the C-ABI and the torch operators.

* tf_fp8_quantize / tf_fp8_dequantize: BIT-EXACT against the format oracle
  (oracle/fp8_oracle.py, itself pinned to TileFusion's test_fp8.cu answers and
  to torch's float8 casts).
* Decoding over an 8-bit cache: the stored bytes are exact inputs, so the
  oracle is the fp32 closed form over the dequantised values and the bounds are
  the ones of the 16-bit cache (max-abs <= 2e-2, relative-L2 <= the dtype's
  computed bound, |LSE| <= 1e-3, fp32 partials relative-L2 <= 1e-5): the kernel
  keeps q, scores, softmax and accumulators in fp32 and only widens K/V.
"""

import math

import pytest
import torch

from oracle import attention_oracle as orc
from oracle import fp8_oracle as f8

pytestmark = pytest.mark.gpu

KINDS = {f8.E4M3: torch.float8_e4m3fn, f8.E5M2: torch.float8_e5m2}
MAX_ABS = 2e-2
LSE_ABS = 1e-3


def _as_fp8(codes: torch.Tensor, kind: str) -> torch.Tensor:
    return codes.view(KINDS[kind])


# ------------------------------------------------------------- conversions --
@pytest.mark.parametrize("kind", list(KINDS))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("n", [1, 15, 16, 17, 4099, (1 << 20) + 3])
def test_quantize_is_bit_exact(kind, dtype, n):
    from cabi_helpers import fp8_convert

    gen = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=gen) * 4.0
    x[::7] *= 1e-3                                    # subnormal results
    x[::11] *= 300.0                                  # beyond e4m3's range: saturation
    x = x.to(dtype)
    for factor in (1.0, 0.37):
        dst = torch.zeros(n, dtype=torch.uint8, device="cuda").view(KINDS[kind])
        fp8_convert(x.cuda(), dst, factor)
        want = f8.quantize(x, kind, factor)
        assert torch.equal(dst.view(torch.uint8).cpu(), want)


@pytest.mark.parametrize("kind", list(KINDS))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_dequantize_is_bit_exact_on_every_code(kind, dtype):
    from cabi_helpers import fp8_convert

    codes = torch.arange(256, dtype=torch.uint8).repeat(9)[: 256 * 9 - 5]      # ragged length
    finite = torch.isfinite(f8.decode(codes, kind))
    for factor in (1.0, 0.125, 3.0):
        dst = torch.zeros(codes.numel(), dtype=dtype, device="cuda")
        fp8_convert(_as_fp8(codes, kind).cuda(), dst, factor)
        want = f8.dequantize(codes, kind, factor, dtype)
        got = dst.cpu()
        assert torch.equal(got[finite].view(torch.int16), want[finite].view(torch.int16))
        assert torch.equal(torch.isnan(got), torch.isnan(want))


def test_round_trip_operator_and_empty_input():
    import tilefusion_b200 as tilefusion

    x = (torch.randn(3, 5, 64, generator=torch.Generator().manual_seed(2)) * 2).to(torch.bfloat16)
    q8 = tilefusion.ops.fp8_quantize(x.cuda(), torch.float8_e4m3fn, factor=4.0)
    assert q8.dtype == torch.float8_e4m3fn and q8.shape == x.shape
    assert torch.equal(q8.view(torch.uint8).cpu(), f8.quantize(x, f8.E4M3, 4.0))
    back = tilefusion.ops.fp8_dequantize(q8, torch.bfloat16, factor=0.25)
    assert torch.equal(back.cpu().view(torch.int16),
                       f8.dequantize(q8.view(torch.uint8).cpu(), f8.E4M3, 0.25, torch.bfloat16).view(torch.int16))
    empty = tilefusion.ops.fp8_quantize(torch.empty(0, dtype=torch.float16, device="cuda"))
    assert empty.numel() == 0


def test_conversion_arguments_are_checked():
    from tilefusion_b200 import _cabi

    lib = _cabi.lib()
    buf = torch.zeros(64, dtype=torch.float16, device="cuda")
    out = torch.zeros(64, dtype=torch.uint8, device="cuda")
    assert lib.tf_fp8_quantize(buf.data_ptr(), out.data_ptr(), 64, _cabi.TF_F16, _cabi.TF_F16, 1.0, None) == _cabi.TF_ERR_UNSUPPORTED
    assert lib.tf_fp8_quantize(buf.data_ptr(), out.data_ptr(), 64, _cabi.TF_FP8_E4M3, _cabi.TF_FP8_E4M3, 1.0, None) == _cabi.TF_ERR_UNSUPPORTED
    assert lib.tf_fp8_quantize(buf.data_ptr(), out.data_ptr(), -1, _cabi.TF_F16, _cabi.TF_FP8_E4M3, 1.0, None) == _cabi.TF_ERR_BAD_ARG
    assert lib.tf_fp8_quantize(buf.data_ptr(), out.data_ptr(), 64, _cabi.TF_F16, _cabi.TF_FP8_E4M3, 0.0, None) == _cabi.TF_ERR_BAD_ARG
    assert lib.tf_fp8_quantize(buf.data_ptr() + 2, out.data_ptr(), 32, _cabi.TF_F16, _cabi.TF_FP8_E4M3, 1.0, None) == _cabi.TF_ERR_UNSUPPORTED
    assert lib.tf_fp8_quantize(None, out.data_ptr(), 0, _cabi.TF_F16, _cabi.TF_FP8_E4M3, 1.0, None) == 0


# ------------------------------------------------------------------ decode --
def _cache(seed, b, h, lk, d, kind, dtype, k_factor=1.0, v_factor=1.0):
    """Seeded q (16-bit) and an 8-bit cache; returns the device inputs and the
    exact fp32 values the cache stands for."""
    q, k, v = orc.seeded_inputs(seed, (b, h, 1, d), (b, h, lk, d), (b, h, lk, d), 1.0, dtype)
    k8, v8 = f8.quantize(k, kind, k_factor), f8.quantize(v, kind, v_factor)
    k_exact = f8.decode(k8, kind) / k_factor
    v_exact = f8.decode(v8, kind) / v_factor
    return q, _as_fp8(k8, kind), _as_fp8(v8, kind), k_exact, v_exact


def _check(o, lse, ref_o, ref_lse, dtype):
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    assert orc.max_abs(o.cpu(), ref_o) <= MAX_ABS
    assert orc.rel_l2(o.cpu(), ref_o) <= orc.rel_l2_bound(ref_o, dtype, p_rounded=False)
    assert orc.max_abs(lse.cpu(), ref_lse) <= LSE_ABS


CASES = [
    # B, H, Lk, D, kv_chunk, num_splits
    (1, 1, 512, 128, 512, 0),
    (2, 3, 1000, 128, 512, 0),     # ragged last chunk and stage
    (1, 2, 1, 128, 512, 0),        # a single key
    (2, 2, 130, 64, 128, 0),
    (4, 8, 4096, 128, 512, 0),
    (4, 8, 4096, 128, 1024, 3),    # uneven splits, the largest chunk
    (1, 4, 3000, 64, 256, 0),
    (2, 2, 2048, 64, 1024, 1),     # one split walks two chunks: running (m, l)
    (3, 5, 777, 128, 128, 0),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c)))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("kind", list(KINDS))
def test_decode_over_8bit_cache_matches_oracle(case, dtype, kind):
    from cabi_helpers import decode, device_status

    b, h, lk, d, chunk, splits = case
    q, k8, v8, k_exact, v_exact = _cache(31, b, h, lk, d, kind, dtype, k_factor=2.0, v_factor=4.0)
    o, lse = decode(q.cuda(), k8.cuda(), v8.cuda(), None, chunk, splits, k_scale=0.5, v_scale=0.25)
    ref, lse_ref = orc.decode_fp32(q, k_exact, v_exact)
    _check(o, lse, ref, lse_ref, dtype)
    assert device_status() == 0


@pytest.mark.parametrize("kind", list(KINDS))
@pytest.mark.parametrize("lk,chunk,splits,d", [(4096, 512, 0, 128), (1000, 256, 2, 128), (2048, 512, 1, 64)])
def test_split_partials_over_8bit_cache_match_oracle(kind, lk, chunk, splits, d):
    from cabi_helpers import decode_split

    q, k8, v8, k_exact, v_exact = _cache(33, 2, 3, lk, d, kind, torch.float16)
    part_o, part_ml, plan = decode_split(q.cuda(), k8.cuda(), v8.cuda(), None, chunk, splits)
    ref_o, ref_ml = orc.decode_split(q.squeeze(2), k_exact, v_exact, 1.0 / math.sqrt(d),
                                     plan.chunks_per_split * plan.kv_chunk)
    assert orc.rel_l2(part_o.cpu(), ref_o) <= 1e-5
    assert orc.max_abs(part_ml.cpu()[..., 0], ref_ml[..., 0]) <= 1e-4
    assert orc.rel_l2(part_ml.cpu()[..., 1], ref_ml[..., 1]) <= 1e-5


def test_scales_default_to_one_and_strided_cache():
    """k_scale = v_scale = 0 read as 1; kv_chunk = 0 is the registry's choice (1024 keys for an
    8-bit cache); K/V heads taken out of a wider buffer (stride_h > Lk*D)."""
    from cabi_helpers import decode

    from cabi_helpers import decode_desc, decode_plan

    b, h, lk, d = 2, 4, 2900, 128
    q, k8, v8, k_exact, v_exact = _cache(35, b, h, lk, d, f8.E4M3, torch.float16)
    assert decode_plan(decode_desc(q, k8, v8, kv_chunk=0)).kv_chunk == 1024
    assert decode_plan(decode_desc(q, q, q, kv_chunk=0)).kv_chunk == 512
    wide_k = torch.zeros(b, h, lk + 28, d, dtype=torch.uint8).view(torch.float8_e4m3fn)
    wide_v = torch.zeros_like(wide_k)
    wide_k[:, :, :lk] = k8
    wide_v[:, :, :lk] = v8
    o, lse = decode(q.cuda(), wide_k.cuda()[:, :, :lk], wide_v.cuda()[:, :, :lk], kv_chunk=0)
    ref, lse_ref = orc.decode_fp32(q, k_exact, v_exact)
    _check(o, lse, ref, lse_ref, torch.float16)


def _paginate(k, v, page_size, seed):
    b, h, lk, d = k.shape
    per_seq = -(-lk // page_size)
    n_pages = b * per_seq + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed))[: b * per_seq].view(b, per_seq)
    kp = torch.zeros(n_pages, h, page_size, d, dtype=torch.uint8)
    vp = torch.zeros_like(kp)
    for bi in range(b):
        for i in range(per_seq):
            n = min(page_size, lk - i * page_size)
            kp[perm[bi, i], :, :n] = k[bi, :, i * page_size:i * page_size + n]
            vp[perm[bi, i], :, :n] = v[bi, :, i * page_size:i * page_size + n]
    return kp, vp, perm.to(torch.int32)


@pytest.mark.parametrize("kind", list(KINDS))
@pytest.mark.parametrize("case", [(2, 4, 1000, 128, 256), (3, 4, 4096, 64, 512)], ids=lambda c: "x".join(map(str, c)))
def test_paged_8bit_cache_through_the_operator(kind, case):
    import tilefusion_b200 as tilefusion

    b, h, lk, d, page = case
    q, k8, v8, k_exact, v_exact = _cache(37, b, h, lk, d, kind, torch.bfloat16, k_factor=2.0, v_factor=2.0)
    kp, vp, table = _paginate(k8.view(torch.uint8), v8.view(torch.uint8), page, 5)
    o, lse = tilefusion.ops.flash_decoding(q.cuda(), _as_fp8(kp, kind).cuda(), _as_fp8(vp, kind).cuda(),
                                           block_table=table.cuda(), kv_len=lk, k_scale=0.5, v_scale=0.5)
    ref, lse_ref = orc.decode_fp32(q, k_exact, v_exact)
    _check(o, lse, ref, lse_ref, torch.bfloat16)


def test_sharded_context_and_static_entry_over_8bit_cache():
    """The fused one-launch sharded step (world of one) and the no-allocation
    entry point read the same descriptor fields."""
    import ctypes as C

    from cabi_helpers import decode_desc, device_status
    from tilefusion_b200 import _cabi

    b, h, lk, d = 2, 8, 3000, 128
    q, k8, v8, k_exact, v_exact = _cache(39, b, h, lk, d, f8.E4M3, torch.float16, k_factor=2.0)
    ref, lse_ref = orc.decode_fp32(q, k_exact, v_exact)
    qd, kd, vd = q.cuda(), k8.cuda(), v8.cuda()
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream

    o = torch.full((b, h, 1, d), float("nan"), dtype=torch.float16, device="cuda")
    lse = torch.full((b, h, 1), float("nan"), dtype=torch.float32, device="cuda")
    desc = decode_desc(qd, kd, vd, o, k_scale=0.5)
    _cabi.check(lib.tf_decode_static(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                     C.byref(desc), stream))
    _check(o, lse, ref, lse_ref, torch.float16)

    ctx = C.c_void_p()
    _cabi.check(lib.tf_shard_create(0, 1, None, _cabi.TF_TRANSPORT_P2P, b, h, d, _cabi.TF_F16, C.byref(ctx)))
    try:
        for _ in range(2):
            o.fill_(float("nan"))
            lse.fill_(float("nan"))
            _cabi.check(lib.tf_decode_sharded(ctx, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(),
                                              lse.data_ptr(), C.byref(desc), stream))
            _check(o, lse, ref, lse_ref, torch.float16)
    finally:
        torch.cuda.synchronize()
        lib.tf_shard_destroy(ctx)
    assert device_status() == 0


GROUPED_CASES = [
    # B, Hkv, group, Lk, D, kv_chunk, num_splits
    (2, 2, 4, 1000, 128, 512, 0),
    (1, 1, 8, 4096, 128, 1024, 0),    # multi-query: one KV head
    (3, 2, 2, 777, 64, 256, 0),
    (2, 3, 5, 2049, 128, 512, 3),     # a group size that is no power of two, uneven splits
    (1, 2, 32, 300, 64, 128, 0),
]


@pytest.mark.parametrize("case", GROUPED_CASES, ids=lambda c: "x".join(map(str, c)))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("kind", list(KINDS))
def test_grouped_query_heads_over_8bit_cache_match_oracle(case, dtype, kind):
    """Query head h reads KV head h // group; every query head is a row of its own."""
    from cabi_helpers import decode, device_status

    b, hkv, g, lk, d, chunk, splits = case
    q, _, _ = orc.seeded_inputs(41, (b, hkv * g, 1, d), (1, 1, 8, d), (1, 1, 8, d), 1.0, dtype)
    _, k8, v8, k_exact, v_exact = _cache(43, b, hkv, lk, d, kind, dtype, k_factor=2.0, v_factor=4.0)
    o, lse = decode(q.cuda(), k8.cuda(), v8.cuda(), None, chunk, splits, k_scale=0.5, v_scale=0.25)
    ref, lse_ref = orc.decode_fp32(q, k_exact.repeat_interleave(g, dim=1), v_exact.repeat_interleave(g, dim=1))
    _check(o, lse, ref, lse_ref, dtype)
    assert device_status() == 0


def test_grouped_query_heads_over_paged_8bit_cache_static_and_sharded():
    """The same rows through the paged operator, the no-allocation entry point and the one-launch
    sharded step (world of one)."""
    import ctypes as C

    import tilefusion_b200 as tilefusion
    from cabi_helpers import decode_desc, device_status
    from tilefusion_b200 import _cabi

    b, hkv, g, lk, d, kind = 2, 2, 4, 1500, 128, f8.E4M3
    q, _, _ = orc.seeded_inputs(45, (b, hkv * g, 1, d), (1, 1, 8, d), (1, 1, 8, d), 1.0, torch.float16)
    _, k8, v8, k_exact, v_exact = _cache(47, b, hkv, lk, d, kind, torch.float16, k_factor=2.0)
    ref, lse_ref = orc.decode_fp32(q, k_exact.repeat_interleave(g, dim=1), v_exact.repeat_interleave(g, dim=1))

    kp, vp, table = _paginate(k8.view(torch.uint8), v8.view(torch.uint8), 256, 7)
    o, lse = tilefusion.ops.flash_decoding(q.cuda(), _as_fp8(kp, kind).cuda(), _as_fp8(vp, kind).cuda(),
                                           block_table=table.cuda(), kv_len=lk, k_scale=0.5)
    _check(o, lse, ref, lse_ref, torch.float16)

    qd, kd, vd = q.cuda(), k8.cuda(), v8.cuda()
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    o = torch.full((b, hkv * g, 1, d), float("nan"), dtype=torch.float16, device="cuda")
    lse = torch.full((b, hkv * g, 1), float("nan"), dtype=torch.float32, device="cuda")
    desc = decode_desc(qd, kd, vd, o, k_scale=0.5)
    _cabi.check(lib.tf_decode_static(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                     C.byref(desc), stream))
    _check(o, lse, ref, lse_ref, torch.float16)

    ctx = C.c_void_p()
    _cabi.check(lib.tf_shard_create(0, 1, None, _cabi.TF_TRANSPORT_P2P, b, hkv * g, d, _cabi.TF_F16, C.byref(ctx)))
    try:
        o.fill_(float("nan"))
        lse.fill_(float("nan"))
        _cabi.check(lib.tf_decode_sharded(ctx, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(),
                                          lse.data_ptr(), C.byref(desc), stream))
        _check(o, lse, ref, lse_ref, torch.float16)
    finally:
        torch.cuda.synchronize()
        lib.tf_shard_destroy(ctx)
    assert device_status() == 0


def test_unsupported_8bit_layouts_report_errors():
    from cabi_helpers import decode_desc, decode_plan
    from tilefusion_b200 import _cabi

    q = torch.zeros(1, 8, 1, 128, dtype=torch.float16, device="cuda")
    k = torch.zeros(1, 3, 256, 128, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    with pytest.raises(_cabi.TileFusionError, match="multiple of heads_kv"):
        decode_plan(decode_desc(q, k, k))
    k = torch.zeros(1, 8, 256, 128, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    d = decode_desc(q, k, k)
    d.k_stride_h += 8
    with pytest.raises(_cabi.TileFusionError, match="multiples of 16"):
        decode_plan(d)
    d = decode_desc(q, k, k)
    d.kv_dtype = 7
    with pytest.raises(_cabi.TileFusionError, match="kv_dtype"):
        decode_plan(d)
    d = decode_desc(q, k, k, k_scale=-1.0)
    with pytest.raises(_cabi.TileFusionError, match="k_scale"):
        decode_plan(d)
