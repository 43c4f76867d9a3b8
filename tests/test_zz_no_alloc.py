"""tf_decode_static: flash decoding for callers that may not allocate.

A serving runtime that owns one fixed device arena, or a plugin inside a process
whose allocator it must not touch, cannot supply the workspace that tf_decode
wants for its split-KV partial rows.  tf_decode_static keeps those rows in a
fixed array inside the library instead.  It must give the same answer as
tf_decode -- the same two kernels run, only the place of the partial rows
differs -- and because every call shares that array, a second call with a
different shape must not be disturbed by what the first one left behind.

This file is named so that pytest collects it after every other test file.
"""

import ctypes as C
import math

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
REL_L2 = 1e-3
LSE_ABS = 1e-3


def _decode_static(q, k, v, kv_chunk=512, num_splits=0):
    from cabi_helpers import decode_desc
    from tilefusion_b200 import _cabi

    b, h, _, d = q.shape
    o = torch.full((b, h, 1, d), float("nan"), dtype=q.dtype, device=q.device)
    lse = torch.full((b, h, 1), float("nan"), dtype=torch.float32, device=q.device)
    desc = decode_desc(q, k, v, o, None, kv_chunk, num_splits)
    rc = _cabi.lib().tf_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                      C.byref(desc), torch.cuda.current_stream().cuda_stream)
    _cabi.check(rc)
    return o, lse


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    from cabi_helpers import decode, device_status

    # the second problem is smaller and differently split than the first, so the
    # array still holds rows of the first call beyond the ones the second writes
    for seed, (b, h, lk, d, chunk, splits) in enumerate([(4, 8, 6000, 128, 512, 0), (2, 3, 1300, 128, 256, 2)]):
        q, k, v = orc.seeded_inputs(40 + seed, (b, h, 1, d), (b, h, lk, d), (b, h, lk, d), 1.0)
        qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
        o_ws, lse_ws = decode(qc, kc, vc, None, chunk, splits)
        o_st, lse_st = _decode_static(qc, kc, vc, chunk, splits)
        assert torch.isfinite(o_st.float()).all() and torch.isfinite(lse_st).all()
        assert orc.max_abs(o_st, o_ws) <= MAX_ABS
        assert orc.rel_l2(o_st, o_ws) <= REL_L2
        assert orc.max_abs(lse_st, lse_ws) <= LSE_ABS
        # and both agree with the oracle
        ref, lse_ref = orc.decode_fp32(q, k, v, 1.0 / math.sqrt(d))
        assert orc.max_abs(o_st.cpu(), ref) <= MAX_ABS and orc.rel_l2(o_st.cpu(), ref) <= REL_L2
        assert orc.max_abs(lse_st.cpu(), lse_ref) <= LSE_ABS
    assert device_status() == 0


def test_grouped_query_and_paged_cache_through_the_same_entry_point():
    """tf_decode_static serves every form tf_decode does.  Grouped-query heads run
    on the tensor-core kernel and a paged cache goes through the block table; in
    both cases the partial rows land in the built-in array, and the results must
    equal those of tf_decode with a caller's workspace."""
    from cabi_helpers import decode_desc, decode_plan, device_status
    from tilefusion_b200 import _cabi

    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream

    def both(q, k, v, fill):
        b, h, _, d = q.shape
        outs = []
        for static in (False, True):
            o = torch.full((b, h, 1, d), float("nan"), dtype=q.dtype, device="cuda")
            lse = torch.full((b, h, 1), float("nan"), dtype=torch.float32, device="cuda")
            desc = decode_desc(q, k, v, o)
            fill(desc)
            if static:
                rc = lib.tf_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                          C.byref(desc), stream)
            else:
                ws = torch.empty(decode_plan(desc).workspace_bytes // 4, dtype=torch.float32, device="cuda")
                rc = lib.tf_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                   ws.data_ptr(), ws.numel() * 4, C.byref(desc), stream)
            _cabi.check(rc)
            outs.append((o, lse))
        (o_ws, lse_ws), (o_st, lse_st) = outs
        assert torch.isfinite(o_st.float()).all() and torch.isfinite(lse_st).all()
        assert orc.max_abs(o_st, o_ws) <= MAX_ABS and orc.rel_l2(o_st, o_ws) <= REL_L2
        assert orc.max_abs(lse_st, lse_ws) <= LSE_ABS
        return o_st, lse_st

    # grouped-query: 8 query heads on 2 KV heads
    b, hq, hkv, lk, d = 2, 8, 2, 3000, 128
    q, k, v = orc.seeded_inputs(44, (b, hq, 1, d), (b, hkv, lk, d), (b, hkv, lk, d), 1.0)
    o, lse = both(q.cuda(), k.cuda(), v.cuda(), lambda desc: None)
    g = hq // hkv
    ref, lse_ref = orc.decode_fp32(q, k.repeat_interleave(g, 1), v.repeat_interleave(g, 1), 1.0 / math.sqrt(d))
    assert orc.max_abs(o.cpu(), ref) <= MAX_ABS and orc.rel_l2(o.cpu(), ref) <= REL_L2
    assert orc.max_abs(lse.cpu(), lse_ref) <= LSE_ABS

    # paged cache: pages of 256 keys in shuffled order, one KV head per query head
    b, h, lk, d, page = 2, 4, 1000, 128, 256
    q, k, v = orc.seeded_inputs(45, (b, h, 1, d), (b, h, lk, d), (b, h, lk, d), 1.0)
    per_seq = -(-lk // page)
    order = torch.randperm(b * per_seq + 2, generator=torch.Generator().manual_seed(7))[: b * per_seq].view(b, per_seq)
    kp = torch.zeros(b * per_seq + 2, h, page, d, dtype=k.dtype)
    vp = torch.zeros_like(kp)
    for bi in range(b):
        for i in range(per_seq):
            n = min(page, lk - i * page)
            kp[order[bi, i], :, :n] = k[bi, :, i * page:i * page + n]
            vp[order[bi, i], :, :n] = v[bi, :, i * page:i * page + n]
    kpc, vpc, table = kp.cuda(), vp.cuda(), order.to(torch.int32).cuda()

    def paged(desc):
        desc.len_kv, desc.heads_kv = lk, h
        desc.page_size, desc.max_pages, desc.num_pages = page, per_seq, kpc.size(0)
        desc.block_table = table.data_ptr()
        desc.k_stride_h, desc.v_stride_h = kpc.stride(1), vpc.stride(1)
        desc.k_stride_page, desc.v_stride_page = kpc.stride(0), vpc.stride(0)

    o, lse = both(q.cuda(), kpc, vpc, paged)
    ref, lse_ref = orc.decode_fp32(q, k, v, 1.0 / math.sqrt(d))
    assert orc.max_abs(o.cpu(), ref) <= MAX_ABS and orc.rel_l2(o.cpu(), ref) <= REL_L2
    assert orc.max_abs(lse.cpu(), lse_ref) <= LSE_ABS
    assert device_status() == 0


def test_problem_larger_than_the_built_in_scratch_is_rejected():
    from cabi_helpers import decode_desc, decode_plan
    from tilefusion_b200 import _cabi

    lib = _cabi.lib()
    cap = lib.tf_decode_static_capacity()
    assert cap == 4 << 20
    # B*H = 512 rows with 32 splits needs 512*32*130*4 = 8.5 MB of partial rows
    b, h, lk, d = 16, 32, 16384, 128
    q = torch.zeros(b, h, 1, d, dtype=torch.float16, device="cuda")
    k = torch.zeros(b, h, lk, d, dtype=torch.float16, device="cuda")
    desc = decode_desc(q, k, k, q, None, 512, 32)
    assert decode_plan(desc).workspace_bytes > cap
    rc = lib.tf_decode_static(q.data_ptr(), k.data_ptr(), k.data_ptr(), q.data_ptr(), None, C.byref(desc), None)
    assert rc == _cabi.TF_ERR_WORKSPACE
    msg = lib.tf_last_error().decode()
    assert str(cap) in msg and "scratch" in msg
