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
