"""Calls into the C-ABI with torch tensors as device memory (test plumbing)."""

from __future__ import annotations

import ctypes as C
import math

import torch

from tilefusion_b200 import _cabi


def _dtype_code(t: torch.Tensor) -> int:
    return {torch.float16: _cabi.TF_F16, torch.bfloat16: _cabi.TF_BF16}[t.dtype]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def attn_desc(q, k, v, o, scale, causal, tile_q=0, tile_kv=0) -> _cabi.TfAttnDesc:
    """q [B,H,Lq,D], k [B,H,Lk,D], v [B,H,Lk,Dv], o [B,H,Lq,Dv]; any strides."""
    d = _cabi.TfAttnDesc()
    d.dtype = _dtype_code(q)
    d.batch, d.heads, d.len_q, d.head_dim = q.shape
    d.len_kv = k.size(2)
    d.head_dim_v = v.size(3)
    d.causal = int(causal)
    d.softmax_scale = scale
    d.tile_q, d.tile_kv = tile_q, tile_kv
    d.q_stride_b, d.q_stride_h, d.q_stride_l = q.stride(0), q.stride(1), q.stride(2)
    d.k_stride_b, d.k_stride_h, d.k_stride_l, d.k_stride_d = k.stride()
    d.v_stride_b, d.v_stride_h, d.v_stride_l, d.v_stride_d = v.stride()
    d.o_stride_b, d.o_stride_h, d.o_stride_l = o.stride(0), o.stride(1), o.stride(2)
    return d


def attn_fwd(q, k, v, scale, causal=False, want_lse=True, poison=True, tile_q=0):
    """Runs tf_attn_fwd; returns (O, LSE).  Outputs are NaN-filled first so
    that any element the kernel fails to write is caught by the comparison."""
    lib = _cabi.lib()
    b, h, lq, _ = q.shape
    o = torch.empty(b, h, lq, v.size(3), dtype=q.dtype, device=q.device)
    lse = torch.empty(b, h, lq, dtype=torch.float32, device=q.device)
    if poison:
        o.fill_(float("nan"))
        lse.fill_(float("nan"))
    d = attn_desc(q, k, v, o, scale, causal, tile_q, 128 if tile_q else 0)
    rc = lib.tf_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                         lse.data_ptr() if want_lse else None, C.byref(d), _stream())
    _cabi.check(rc)
    return o, (lse if want_lse else None)


def attn_bwd(q, k, v, o, d_o, lse, scale, causal=False):
    """Runs tf_attn_bwd; q/o/d_o [B,H,Lq,D], k/v [B,H,Lk,D] (rows contiguous), lse [B,H,Lq].
    Returns (dq, dk, dv), NaN-filled before the call."""
    lib = _cabi.lib()
    d_o = d_o.contiguous() if d_o.stride() != o.stride() else d_o
    # dq / dk / dv take the strides of q / k / v (the entry point's convention)
    dq, dk, dv = (torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=t.device).fill_(float("nan"))
                  for t in (q, k, v))
    d = attn_desc(q, k, v, o, scale, causal)
    need = lib.tf_attn_bwd_workspace_bytes(C.byref(d))
    ws = torch.empty(max(1, need // 4), dtype=torch.float32, device=q.device)
    rc = lib.tf_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(),
                         dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), C.byref(d), ws.data_ptr(), ws.numel() * 4,
                         _stream())
    _cabi.check(rc)
    return dq, dk, dv


_FP8_CODES = {torch.float8_e4m3fn: _cabi.TF_FP8_E4M3, torch.float8_e5m2: _cabi.TF_FP8_E5M2}


def decode_desc(q, k, v, o=None, scale=None, kv_chunk=512, num_splits=0, k_scale=0.0, v_scale=0.0) -> _cabi.TfDecodeDesc:
    """q [B,H,1,D], k/v [B,H,Lk,D] (q's dtype, or float8 with dequantisation factors)."""
    d = _cabi.TfDecodeDesc()
    d.dtype = _dtype_code(q)
    d.kv_dtype = _FP8_CODES.get(k.dtype, 0)
    d.k_scale, d.v_scale = k_scale, v_scale
    d.batch, d.heads = q.size(0), q.size(1)
    d.heads_kv = k.size(1)
    d.len_kv = k.size(2)
    d.head_dim = q.size(3)
    d.kv_chunk, d.num_splits = kv_chunk, num_splits
    d.softmax_scale = 1.0 / math.sqrt(q.size(3)) if scale is None else scale
    d.q_stride_b, d.q_stride_h = q.stride(0), q.stride(1)
    d.k_stride_b, d.k_stride_h = k.stride(0), k.stride(1)
    d.v_stride_b, d.v_stride_h = v.stride(0), v.stride(1)
    if o is not None:
        d.o_stride_b, d.o_stride_h = o.stride(0), o.stride(1)
    return d


def decode_plan(d: _cabi.TfDecodeDesc) -> _cabi.TfDecodePlan:
    plan = _cabi.TfDecodePlan()
    _cabi.check(_cabi.lib().tf_decode_plan(C.byref(d), C.byref(plan)))
    return plan


def decode(q, k, v, scale=None, kv_chunk=512, num_splits=0, k_scale=0.0, v_scale=0.0):
    lib = _cabi.lib()
    b, h, _, dim = q.shape
    o = torch.full((b, h, 1, dim), float("nan"), dtype=q.dtype, device=q.device)
    lse = torch.full((b, h, 1), float("nan"), dtype=torch.float32, device=q.device)
    d = decode_desc(q, k, v, o, scale, kv_chunk, num_splits, k_scale, v_scale)
    plan = decode_plan(d)
    ws = torch.full((max(1, plan.workspace_bytes // 4),), float("nan"), dtype=torch.float32, device=q.device)
    rc = lib.tf_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                       ws.data_ptr(), ws.numel() * 4, C.byref(d), _stream())
    _cabi.check(rc)
    return o, lse


def decode_split(q, k, v, scale=None, kv_chunk=512, num_splits=0, k_scale=0.0, v_scale=0.0):
    """Returns (part_o [B,H,S,D], part_ml [B,H,S,2], plan)."""
    lib = _cabi.lib()
    b, h, _, dim = q.shape
    d = decode_desc(q, k, v, None, scale, kv_chunk, num_splits, k_scale, v_scale)
    plan = decode_plan(d)
    ws = torch.full((plan.workspace_bytes // 4,), float("nan"), dtype=torch.float32, device=q.device)
    rc = lib.tf_decode_split(q.data_ptr(), k.data_ptr(), v.data_ptr(), ws.data_ptr(), ws.numel() * 4,
                             C.byref(d), _stream())
    _cabi.check(rc)
    s = plan.num_splits
    part_o = ws[: b * h * s * dim].view(b, h, s, dim)
    part_ml = ws[b * h * s * dim:].view(b, h, s, 2)
    return part_o, part_ml, plan


def decode_partial_into(q, k, v, slot, scale=None, kv_chunk=512, num_splits=0):
    lib = _cabi.lib()
    d = decode_desc(q, k, v, None, scale, kv_chunk, num_splits)
    plan = decode_plan(d)
    ws = torch.empty((max(1, plan.workspace_bytes // 4),), dtype=torch.float32, device=q.device)
    rc = lib.tf_decode_partial(q.data_ptr(), k.data_ptr() if k.numel() else None,
                               v.data_ptr() if v.numel() else None, slot.data_ptr(), ws.data_ptr(),
                               ws.numel() * 4, C.byref(d), _stream())
    _cabi.check(rc)


def decode_gathered(slots, batch, heads, dim, dtype):
    lib = _cabi.lib()
    o = torch.full((batch, heads, 1, dim), float("nan"), dtype=dtype, device=slots.device)
    lse = torch.full((batch, heads, 1), float("nan"), dtype=torch.float32, device=slots.device)
    code = _cabi.TF_F16 if dtype == torch.float16 else _cabi.TF_BF16
    rc = lib.tf_decode_gathered(slots.data_ptr(), slots.size(0), batch, heads, dim, code, o.data_ptr(),
                                o.stride(0), o.stride(1), lse.data_ptr(), _stream())
    _cabi.check(rc)
    return o, lse


def fp8_convert(src, dst, factor=1.0):
    """tf_fp8_quantize (dst float8) or tf_fp8_dequantize (src float8) over flat tensors."""
    lib = _cabi.lib()
    if dst.dtype in _FP8_CODES:
        rc = lib.tf_fp8_quantize(src.data_ptr(), dst.data_ptr(), src.numel(), _dtype_code(src), _FP8_CODES[dst.dtype],
                                 factor, _stream())
    else:
        rc = lib.tf_fp8_dequantize(src.data_ptr(), dst.data_ptr(), src.numel(), _FP8_CODES[src.dtype], _dtype_code(dst),
                                   factor, _stream())
    _cabi.check(rc)


def device_status() -> int:
    code = C.c_int32(0)
    _cabi.lib().tf_device_status(C.byref(code))
    return code.value
