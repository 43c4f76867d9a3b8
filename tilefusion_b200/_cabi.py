"""ctypes view of the C-ABI in ``include/tilefusion_b200.h``.

The structures mirror the header field by field.  ``lib()`` returns the loaded
``libtilefusion_b200.so`` with argument types set; it raises if the library is
missing and cannot be built -- nothing in this package computes attention any
other way.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libtilefusion_b200.so"

TF_OK = 0
TF_ERR_BAD_ARG = -1
TF_ERR_UNSUPPORTED = -2
TF_ERR_CUDA = -3
TF_ERR_DEVICE_TIMEOUT = -4
TF_ERR_WORKSPACE = -5
TF_F16 = 0
TF_BF16 = 1
TF_FP8_E4M3 = 2
TF_FP8_E5M2 = 3

# Every symbol the header declares (checked by the CPU test-suite).
EXPORTED = (
    "tf_attn_fwd", "tf_attn_plan", "tf_decode_plan", "tf_decode_split",
    "tf_decode_combine", "tf_decode", "tf_decode_partial", "tf_decode_gathered",
    "tf_last_error", "tf_device_status", "tf_abi_version",
    "tf_decode_static", "tf_decode_static_capacity",
    "tf_decode_partial_scatter", "tf_decode_gathered_wait", "tf_fused_two_gemms",
    "tf_shard_head_slice", "tf_shard_kv_slice", "tf_prefill_sharded", "tf_shard_unique_id",
    "tf_shard_create", "tf_shard_transport", "tf_shard_note", "tf_decode_sharded", "tf_shard_destroy",
    "tf_device_status_peek", "tf_set_wait_limit_ms", "tf_attn_bwd", "tf_attn_bwd_workspace_bytes",
    "tf_fp8_quantize", "tf_fp8_dequantize", "tf_probe_mma_clocks", "tf_probe_mma_pair_clocks",
)
TF_NCCL_ID_BYTES = 128
TF_TRANSPORT_AUTO, TF_TRANSPORT_P2P, TF_TRANSPORT_NCCL = 0, 1, 2


class TfAttnDesc(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("batch", C.c_int32), ("heads", C.c_int32),
        ("len_q", C.c_int32), ("len_kv", C.c_int32), ("head_dim", C.c_int32),
        ("head_dim_v", C.c_int32), ("causal", C.c_int32),
        ("softmax_scale", C.c_float), ("tile_q", C.c_int32), ("tile_kv", C.c_int32),
        ("reserved", C.c_int32),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_l", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64), ("k_stride_l", C.c_int64),
        ("k_stride_d", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64), ("v_stride_l", C.c_int64),
        ("v_stride_d", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64), ("o_stride_l", C.c_int64),
    ]


class TfDecodeDesc(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("batch", C.c_int32), ("heads", C.c_int32),
        ("len_kv", C.c_int32), ("head_dim", C.c_int32), ("kv_chunk", C.c_int32),
        ("num_splits", C.c_int32), ("softmax_scale", C.c_float),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64),
        ("heads_kv", C.c_int32), ("page_size", C.c_int32),
        ("block_table", C.c_void_p), ("max_pages", C.c_int32), ("num_pages", C.c_int32),
        ("k_stride_page", C.c_int64), ("v_stride_page", C.c_int64),
        ("kv_dtype", C.c_int32), ("k_scale", C.c_float), ("v_scale", C.c_float),
    ]


class TfDecodePlan(C.Structure):
    _fields_ = [
        ("num_splits", C.c_int32), ("chunks_per_split", C.c_int32),
        ("kv_chunk", C.c_int32), ("grid", C.c_int32), ("stages", C.c_int32),
        ("reserved", C.c_int32), ("workspace_bytes", C.c_uint64),
    ]


class TfAttnPlan(C.Structure):
    _fields_ = [
        ("tile_q", C.c_int32), ("tile_kv", C.c_int32), ("ctas_per_sm", C.c_int32),
        ("grid", C.c_int32), ("k_mn_major", C.c_int32), ("v_mn_major", C.c_int32),
        ("head_dim_kernel", C.c_int32), ("smem_bytes", C.c_uint64),
    ]


class TileFusionError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"tilefusion_b200 error {code}: {message}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """The loaded native library (built on first use when nvcc is present)."""
    global _lib
    if _lib is not None:
        return _lib
    from .build import build_library

    build_library()     # no-op when the library matches the sources
    try:
        handle = C.CDLL(str(_LIB_PATH))
    except OSError as e:  # pragma: no cover - depends on the machine
        raise RuntimeError(f"Failed to load library from {_LIB_PATH}") from e
    vp, i32, i64, u64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64
    fp = C.c_void_p  # float* passed as raw addresses
    handle.tf_attn_fwd.argtypes = [vp, vp, vp, vp, fp, C.POINTER(TfAttnDesc), vp]
    handle.tf_attn_plan.argtypes = [C.POINTER(TfAttnDesc), C.POINTER(TfAttnPlan)]
    handle.tf_attn_bwd.argtypes = [vp, vp, vp, vp, vp, fp, vp, vp, vp, C.POINTER(TfAttnDesc), vp, u64, vp]
    handle.tf_attn_bwd_workspace_bytes.argtypes = [C.POINTER(TfAttnDesc)]
    handle.tf_decode_plan.argtypes = [C.POINTER(TfDecodeDesc), C.POINTER(TfDecodePlan)]
    handle.tf_decode_split.argtypes = [vp, vp, vp, vp, u64, C.POINTER(TfDecodeDesc), vp]
    handle.tf_decode_combine.argtypes = [
        fp, fp, i32, i64, i64, i64, i64, i32, i32, i32, i32, vp, i64, i64, fp, fp, fp, vp,
    ]
    handle.tf_decode.argtypes = [vp, vp, vp, vp, fp, vp, u64, C.POINTER(TfDecodeDesc), vp]
    handle.tf_decode_partial.argtypes = [vp, vp, vp, fp, vp, u64, C.POINTER(TfDecodeDesc), vp]
    handle.tf_decode_gathered.argtypes = [fp, i32, i32, i32, i32, i32, vp, i64, i64, fp, vp]
    handle.tf_decode_partial_scatter.argtypes = [vp, vp, vp, vp, u64, C.POINTER(TfDecodeDesc), vp, i32, i32,
                                                 i64, i64, C.c_uint32, vp]
    handle.tf_decode_gathered_wait.argtypes = [fp, vp, i32, C.c_uint32, i32, i32, i32, i32, vp, i64, i64, fp, vp]
    handle.tf_fused_two_gemms.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i64, vp]
    handle.tf_decode_static.argtypes = [vp, vp, vp, vp, fp, C.POINTER(TfDecodeDesc), vp]
    handle.tf_decode_static_capacity.argtypes = []
    handle.tf_last_error.restype = C.c_char_p
    handle.tf_device_status.argtypes = [C.POINTER(C.c_int32)]
    handle.tf_device_status_peek.argtypes = [C.POINTER(C.c_int32)]
    handle.tf_set_wait_limit_ms.argtypes = [C.c_uint32]
    handle.tf_probe_mma_clocks.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                           C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    handle.tf_probe_mma_pair_clocks.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    handle.tf_fp8_quantize.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_float, C.c_void_p]
    handle.tf_fp8_dequantize.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_float, C.c_void_p]
    handle.tf_shard_head_slice.argtypes = [i64, i32, i32, C.POINTER(i64), C.POINTER(i64)]
    handle.tf_shard_kv_slice.argtypes = [i64, i32, i32, i32, C.POINTER(i64), C.POINTER(i64)]
    handle.tf_prefill_sharded.argtypes = [i32, i32, vp, vp, vp, vp, fp, C.POINTER(TfAttnDesc), vp,
                                          C.POINTER(i64), C.POINTER(i64)]
    handle.tf_shard_unique_id.argtypes = [vp]
    handle.tf_shard_create.argtypes = [i32, i32, vp, i32, i32, i32, i32, i32, C.POINTER(vp)]
    handle.tf_shard_transport.argtypes = [vp]
    handle.tf_shard_note.argtypes = [vp]
    handle.tf_shard_note.restype = C.c_char_p
    handle.tf_decode_sharded.argtypes = [vp, vp, vp, vp, vp, fp, C.POINTER(TfDecodeDesc), vp]
    handle.tf_shard_destroy.argtypes = [vp]
    for name in EXPORTED:
        if name not in ("tf_last_error", "tf_decode_static_capacity", "tf_shard_note", "tf_attn_bwd_workspace_bytes"):
            getattr(handle, name).restype = C.c_int
    handle.tf_decode_static_capacity.restype = C.c_uint64
    handle.tf_attn_bwd_workspace_bytes.restype = C.c_uint64
    _lib = handle
    return handle


def check(rc: int) -> None:
    if rc != TF_OK:
        raise TileFusionError(rc, lib().tf_last_error().decode())


lib()
