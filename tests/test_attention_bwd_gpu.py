"""Parity of the CUDA attention backward with the gradient of the fp32 closed form.

TileFusion has no backward pass, so nothing of it pins these results; the
reference is reverse-mode differentiation (torch.autograd, fp32, on the host)
of the same expression its FlashAttentionRef class pins for the forward
(oracle.attention_bwd_fp32).  The kernels round P and dS to the 16-bit input
type before the second tensor-core products, as the forward rounds P, so the
gradients carry that rounding on top of the rounding of the outputs.
Tolerances: fp16 relative-L2 <= 2e-3 per gradient; bf16: the computed bound of
oracle.rel_l2_bound (rounding floor of the exact gradient and of the rounded
operand in quadrature, +15 %), doubled because two rounded operands (P and dS)
feed dK and dQ.  Max-abs <= 2e-2 relative to the largest gradient entry.
"""

import math

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def _check_grad(name, got, ref, dtype):
    assert torch.isfinite(got.float()).all(), f"{name}: kernel left NaN/Inf"
    assert orc.max_abs(got.cpu(), ref) <= 2e-2 * max(1.0, ref.abs().max().item()), name
    if ref.float().pow(2).mean().sqrt().item() < 1e-4:
        # a gradient that is exactly zero (one key: softmax is constant) has no relative error;
        # what the kernel returns comes from the rounding of O and must stay at that level
        assert got.float().abs().max().item() <= 2e-3, name
        return
    bound = 2e-3 if dtype == torch.float16 else 2.0 * orc.rel_l2_bound(ref, dtype)
    rel = orc.rel_l2(got.cpu(), ref)
    assert rel <= bound, f"{name}: rel-L2 {rel:.3e} > {bound:.3e}"


def _run(b, h, lq, lk, d, causal, dtype, seed=3, sigma=1.0):
    from cabi_helpers import attn_bwd, attn_fwd, device_status

    q, k, v = orc.seeded_inputs(seed, (b, h, lq, d), (b, h, lk, d), (b, h, lk, d), sigma, dtype)
    d_o = (torch.randn(b, h, lq, d, generator=torch.Generator().manual_seed(seed + 100)) * sigma).to(dtype)
    scale = 1.0 / math.sqrt(d)
    qc, kc, vc, doc = q.cuda(), k.cuda(), v.cuda(), d_o.cuda()
    o, lse = attn_fwd(qc, kc, vc, scale, causal)
    dq, dk, dv = attn_bwd(qc, kc, vc, o, doc, lse, scale, causal)
    rq, rk, rv = orc.attention_bwd_fp32(q, k, v, d_o, scale, causal)
    _check_grad("dV", dv, rv, dtype)
    _check_grad("dK", dk, rk, dtype)
    _check_grad("dQ", dq, rq, dtype)
    assert device_status() == 0


BWD_SHAPES = [
    # B, H, Lq, Lk, D, causal
    (1, 1, 128, 128, 128, False),     # one tile each way
    (1, 2, 256, 384, 128, False),     # several query and key tiles: both accumulation loops
    (2, 3, 100, 200, 128, False),     # ragged tiles
    (1, 2, 384, 384, 128, True),      # causal: diagonal tiles masked, tiles above skipped
    (1, 2, 200, 456, 128, True),      # causal with more keys than queries: key tiles nobody sees get zeros
    (1, 2, 300, 200, 64, True),       # causal, more queries than keys, D = 64
    (3, 5, 257, 129, 64, False),
    (1, 1, 1, 1, 128, False),         # single query, single key
]


@pytest.mark.parametrize("shape", BWD_SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_backward_matches_autograd_of_the_closed_form(shape, dtype):
    b, h, lq, lk, d, causal = shape
    _run(b, h, lq, lk, d, causal, dtype)


def test_config1_whole_and_config2_heads():
    """The plumbing config (B1 H8 L128 D64, scale 1/8) whole, and four heads of the
    fp16 prefill config (L2048 D128, sigma 0.5)."""
    from cabi_helpers import attn_bwd, attn_fwd

    q, k, v = orc.seeded_inputs(0, (1, 8, 128, 64), (1, 8, 128, 64), (1, 8, 128, 64), 1.0)
    d_o = torch.randn(1, 8, 128, 64, generator=torch.Generator().manual_seed(7)).half()
    o, lse = attn_fwd(q.cuda(), k.cuda(), v.cuda(), 0.125, False)
    grads = attn_bwd(q.cuda(), k.cuda(), v.cuda(), o, d_o.cuda(), lse, 0.125, False)
    for name, got, ref in zip(("dQ", "dK", "dV"), grads, orc.attention_bwd_fp32(q, k, v, d_o, 0.125, False)):
        _check_grad(name, got, ref, torch.float16)
    _run(1, 4, 2048, 2048, 128, False, torch.float16, seed=1, sigma=0.5)
    _run(1, 2, 2048, 2048, 128, True, torch.float16, seed=1, sigma=0.5)


def test_strided_views_and_linearity():
    """Operands as strided views of one packed [B, L, 3, H, D] buffer; and the
    backward is linear in dO: grad(2 dO) = 2 grad(dO) exactly (power of two)."""
    from cabi_helpers import attn_bwd, attn_fwd

    b, h, l, d = 2, 3, 256, 128
    packed = (torch.randn(b, l, 3, h, d, generator=torch.Generator().manual_seed(9)) * 0.7).half().cuda()
    q, k, v = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    d_o = torch.randn(b, h, l, d, generator=torch.Generator().manual_seed(10)).half().cuda()
    scale = 1.0 / math.sqrt(d)
    o, lse = attn_fwd(q, k, v, scale, True)
    g1 = attn_bwd(q, k, v, o, d_o, lse, scale, True)
    refs = orc.attention_bwd_fp32(q.cpu(), k.cpu(), v.cpu(), d_o.cpu(), scale, True)
    for name, got, ref in zip(("dQ", "dK", "dV"), g1, refs):
        assert got.stride() == {"dQ": q, "dK": k, "dV": v}[name].stride()
        _check_grad(name, got, ref, torch.float16)
    g2 = attn_bwd(q, k, v, o, d_o * 2, lse, scale, True)
    for a, bb in zip(g1, g2):
        assert orc.rel_l2(bb.float().cpu(), 2 * a.float().cpu()) <= 1e-3


def test_autograd_through_the_python_operator():
    """tilefusion_b200.ops.flash_attention_autograd in TileFusion's argument convention
    (key given as [.., D, Lk]): .backward() runs the CUDA backward."""
    import tilefusion_b200 as tilefusion

    b, h, lq, lk, d = 2, 2, 192, 320, 128
    q, k, v = orc.seeded_inputs(21, (b, h, lq, d), (b, h, lk, d), (b, h, lk, d), 0.8)
    d_o = torch.randn(b, h, lq, d, generator=torch.Generator().manual_seed(22)).half()
    scale = 1.0 / math.sqrt(d)
    qc = q.cuda().requires_grad_(True)
    kt = k.cuda().transpose(-1, -2).contiguous().requires_grad_(True)      # key as [.., D, Lk], its own storage
    vc = v.cuda().requires_grad_(True)
    out = tilefusion.ops.flash_attention_autograd(qc, kt, vc, scale, True)
    out.backward(d_o.cuda())
    rq, rk, rv = orc.attention_bwd_fp32(q, k, v, d_o, scale, True)
    _check_grad("dQ", qc.grad, rq, torch.float16)
    _check_grad("dK", kt.grad.transpose(-1, -2), rk, torch.float16)
    _check_grad("dV", vc.grad, rv, torch.float16)


def test_bad_arguments_are_reported():
    import ctypes as C

    from cabi_helpers import attn_desc
    from tilefusion_b200 import _cabi

    lib = _cabi.lib()
    x = torch.zeros(1, 1, 128, 96, dtype=torch.float16, device="cuda")
    d = attn_desc(x, x, x, x, 0.1, False)
    p = x.data_ptr()
    rc = lib.tf_attn_bwd(p, p, p, p, p, p, p, p, p, C.byref(d), p, 1 << 20, None)
    assert rc == _cabi.TF_ERR_UNSUPPORTED and "backward" in lib.tf_last_error().decode()
    y = torch.zeros(1, 1, 128, 128, dtype=torch.float16, device="cuda")
    d = attn_desc(y, y, y, y, 0.1, False)
    p = y.data_ptr()
    rc = lib.tf_attn_bwd(p, p, p, p, p, p, p, p, p, C.byref(d), p, 16, None)
    assert rc == _cabi.TF_ERR_WORKSPACE
    rc = lib.tf_attn_bwd(p, p, p, p, p, None, p, p, p, C.byref(d), p, 1 << 20, None)
    assert rc == _cabi.TF_ERR_BAD_ARG
