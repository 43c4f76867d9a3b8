"""fused_two_gemms (the attention kernel without its softmax) against the oracle.

TileFusion's own test (tests/python/test_fused_two_gemms.py:55-108) draws
N(0.05, 0.01) fp16 matrices of size M=256, N=128, K=64, P=64 and accepts
allclose(rtol=1e-3, atol=1e-3) against ``input_a @ input_b.t() @ input_c.t()``;
that case and tolerance are reproduced here, with more shapes beside it.
"""

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def _normal(shape, mean, std, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.normal(mean=torch.full(shape, mean), std=torch.full(shape, std), generator=g).to(dtype)


def test_reference_case_through_python_api():
    import tilefusion_b200 as tilefusion

    m, n, k, p = 256, 128, 64, 64
    a = _normal((m, k), 5e-2, 1e-2, torch.float16, 1).cuda()
    b = _normal((n, k), 5e-2, 1e-2, torch.float16, 2).cuda()
    c = _normal((p, n), 5e-2, 1e-2, torch.float16, 3).cuda()
    out = torch.zeros(m, p, dtype=torch.float16, device="cuda")
    tilefusion.ops.fused_two_gemms(a, b, c, out, 64, 64, 64, 64)
    ref = orc.fused_two_gemms_fp32(a.cpu(), b.cpu(), c.cpu())
    assert torch.allclose(out.float().cpu(), ref, rtol=1e-3, atol=1e-3)
    # and against the 16-bit torch expression TileFusion's test uses, on the GPU
    assert torch.allclose(out, a @ b.t() @ c.t(), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("m,n,k,p", [(128, 128, 128, 128), (300, 200, 64, 64), (1, 8, 128, 128),
                                     (1000, 1024, 128, 128), (64, 77, 64, 64),
                                     # k != p and widths between / above the compiled 64, 128, 256
                                     (256, 128, 64, 128), (200, 264, 128, 64), (130, 96, 96, 96), (256, 256, 256, 256),
                                     (100, 512, 192, 72), (64, 64, 8, 256)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_shapes_through_cabi(m, n, k, p, dtype):
    from cabi_helpers import device_status
    from tilefusion_b200 import _cabi

    if n % 8 != 0:
        pytest.skip("C rows ([P, N]) must be 16-byte aligned for TMA: N a multiple of 8")
    a = _normal((m, k), 0.0, 1.0, dtype, 4).cuda()
    b = _normal((n, k), 0.0, 0.125, dtype, 5).cuda()
    c = _normal((p, n), 0.0, 0.125, dtype, 6).cuda()
    d = torch.full((m, p), float("nan"), dtype=dtype, device="cuda")
    code = _cabi.TF_F16 if dtype == torch.float16 else _cabi.TF_BF16
    rc = _cabi.lib().tf_fused_two_gemms(a.data_ptr(), b.data_ptr(), c.data_ptr(), d.data_ptr(), m, n, k, p, code,
                                        a.stride(0), b.stride(0), c.stride(0), d.stride(0),
                                        torch.cuda.current_stream().cuda_stream)
    _cabi.check(rc)
    ref = orc.fused_two_gemms_fp32(a.cpu(), b.cpu(), c.cpu())
    assert torch.isfinite(d.float()).all()
    # fp16: 1e-3.  bf16: the oracle rounds the intermediate product exactly as the
    # kernel does, so only the rounding of the output is left: 1.15 x its floor
    assert orc.rel_l2(d.cpu(), ref) <= orc.rel_l2_bound(ref, dtype, p_rounded=False)
    assert device_status() == 0


def test_unsupported_widths_are_reported():
    from tilefusion_b200 import _cabi

    x = torch.zeros(64, 264, dtype=torch.float16, device="cuda")
    rc = _cabi.lib().tf_fused_two_gemms(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 64, 64, 264, 264,
                                        _cabi.TF_F16, 264, 264, 264, 264, None)
    assert rc == _cabi.TF_ERR_UNSUPPORTED and "multiples of 8" in _cabi.lib().tf_last_error().decode()


def test_mma_probe_reports_plausible_clocks():
    """tf_probe_mma_clocks: back-to-back M128 K16 MMAs retire no faster than the nominal rate
    (N / 2 clocks) and within a small multiple of it, for every operand form."""
    import ctypes as C

    from tilefusion_b200 import _cabi

    lib = _cabi.lib()
    for n in (64, 128, 256):
        for a_tmem in (0, 1):
            for b_mn in (0, 1):
                for desc32, uniform in ((0, 0), (1, 0), (1, 1)):
                    issue, done = C.c_int64(0), C.c_int64(0)
                    _cabi.check(lib.tf_probe_mma_clocks(a_tmem, n, b_mn, desc32, uniform, 256, C.byref(issue), C.byref(done)))
                    per_mma = done.value / 256
                    assert 0.9 * n / 2 <= per_mma <= 6 * n, (n, a_tmem, b_mn, desc32, uniform, per_mma)
                    assert 0 < issue.value <= done.value
    assert lib.tf_probe_mma_clocks(0, 96, 0, 1, 1, 256, C.byref(issue), C.byref(done)) == _cabi.TF_ERR_BAD_ARG
    assert lib.tf_probe_mma_clocks(0, 128, 0, 1, 1, 12, C.byref(issue), C.byref(done)) == _cabi.TF_ERR_BAD_ARG


def test_mma_pair_probe_matches_the_single_cta_clocks():
    """tf_probe_mma_pair_clocks: an M256 MMA over a pair of SMs (128 rows and n / 2 of B's columns in
    each) takes, per SM, the clocks of the M128 single-CTA MMA of the same n (within 10 %): the
    two-CTA form saves shared memory, not tensor-pipe time."""
    import ctypes as C

    from tilefusion_b200 import _cabi
    from cabi_helpers import device_status

    lib = _cabi.lib()
    for n in (64, 128, 256):
        for a_tmem in (0, 1):
            for b_mn in (0, 1):
                one = []
                for probe in (lambda *o: lib.tf_probe_mma_clocks(a_tmem, n, b_mn, 1, 1, 256, *o),
                              lambda *o: lib.tf_probe_mma_pair_clocks(a_tmem, n, b_mn, 256, *o)):
                    best = None
                    for _ in range(3):
                        issue, done = C.c_int64(0), C.c_int64(0)
                        _cabi.check(probe(C.byref(issue), C.byref(done)))
                        assert 0 < issue.value <= done.value
                        best = done.value if best is None else min(best, done.value)
                    one.append(best / 256)
                assert 0.9 * n / 2 <= one[1] <= 6 * n, (n, a_tmem, b_mn, one)
                assert abs(one[1] - one[0]) <= 0.1 * one[0], (n, a_tmem, b_mn, one)
    assert device_status() == 0
    assert lib.tf_probe_mma_pair_clocks(0, 96, 0, 256, C.byref(issue), C.byref(done)) == _cabi.TF_ERR_BAD_ARG
    assert lib.tf_probe_mma_pair_clocks(0, 128, 0, 12, C.byref(issue), C.byref(done)) == _cabi.TF_ERR_BAD_ARG
