"""The C-ABI library and the host-side logic, without a GPU.

No compute entry point is launched here: these tests check that the library
loads, exports what the header declares, validates arguments before it
touches CUDA, and that the registry plans sensibly.
"""

import ctypes as C
import re
from pathlib import Path

import pytest

from tilefusion_b200 import _cabi

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "tilefusion_b200.h").read_text()


def test_library_exports_every_declared_symbol(native_lib):
    declared = re.findall(r"TF_EXPORT\s+[\w\s\*]+?\b(tf_\w+)\s*\(", HEADER)
    assert sorted(declared) == sorted(_cabi.EXPORTED)
    for name in declared:
        assert hasattr(native_lib, name), f"{name} is declared but not exported"
    assert native_lib.tf_abi_version() == 5


def test_struct_layouts_match_header():
    # field order and types are mirrored by hand; sizes catch a drift
    assert C.sizeof(_cabi.TfAttnDesc) == 12 * 4 + 14 * 8
    assert C.sizeof(_cabi.TfDecodeDesc) == 8 * 4 + 8 * 8 + 2 * 4 + 8 + 2 * 4 + 2 * 8 + 3 * 4 + 4   # (+ tail padding)
    assert C.sizeof(_cabi.TfDecodePlan) == 6 * 4 + 8
    assert C.sizeof(_cabi.TfAttnPlan) == 7 * 4 + 4 + 8
    for struct, cname in [(_cabi.TfAttnDesc, "TfAttnDesc"), (_cabi.TfDecodeDesc, "TfDecodeDesc"),
                          (_cabi.TfDecodePlan, "TfDecodePlan"), (_cabi.TfAttnPlan, "TfAttnPlan")]:
        body = re.search(r"typedef struct " + cname + r" \{(.*?)\} " + cname, HEADER, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            decl = re.sub(r"^(const\s+)?(u?int\d+_t|float)\s*\*?\s*", "", decl)
            names += [n.strip() for n in decl.split(",")]
        assert names == [f[0] for f in struct._fields_], cname


def _attn_desc(**kw):
    d = _cabi.TfAttnDesc()
    d.dtype, d.batch, d.heads, d.len_q, d.len_kv = _cabi.TF_F16, 8, 32, 2048, 2048
    d.head_dim = d.head_dim_v = 128
    d.softmax_scale = 0.088
    d.q_stride_l = d.k_stride_l = d.v_stride_l = d.o_stride_l = 128
    d.k_stride_d = d.v_stride_d = 1
    d.q_stride_h = d.k_stride_h = d.v_stride_h = d.o_stride_h = 2048 * 128
    d.q_stride_b = d.k_stride_b = d.v_stride_b = d.o_stride_b = 32 * 2048 * 128
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_attn_plan_and_layout_detection(native_lib):
    plan = _cabi.TfAttnPlan()
    assert native_lib.tf_attn_plan(C.byref(_attn_desc()), C.byref(plan)) == 0
    # big problem: two Q tiles per CTA, persistent grid of one CTA per SM
    assert (plan.tile_q, plan.tile_kv, plan.ctas_per_sm) == (256, 128, 1)
    assert plan.grid == 148
    # a tile hint that names a compiled variant wins
    assert native_lib.tf_attn_plan(C.byref(_attn_desc(tile_q=128, tile_kv=128)), C.byref(plan)) == 0
    assert (plan.tile_q, plan.ctas_per_sm, plan.grid) == (128, 2, 16 * 32 * 8)
    # a single Q tile, or too few tile pairs to fill the GPU: one tile per CTA
    assert native_lib.tf_attn_plan(C.byref(_attn_desc(len_q=128)), C.byref(plan)) == 0
    assert plan.tile_q == 128
    assert native_lib.tf_attn_plan(C.byref(_attn_desc(batch=1, heads=8, len_q=512)), C.byref(plan)) == 0
    assert plan.tile_q == 128
    # ... unless there are at least 3/4 of an SM count of pairs and the KV loop is long (2048 keys)
    assert native_lib.tf_attn_plan(C.byref(_attn_desc(batch=1, heads=16)), C.byref(plan)) == 0      # 128 pairs
    assert plan.tile_q == 256
    assert native_lib.tf_attn_plan(C.byref(_attn_desc(batch=1, heads=16, len_kv=1024)), C.byref(plan)) == 0
    assert plan.tile_q == 128
    assert native_lib.tf_attn_plan(C.byref(_attn_desc(batch=1, heads=8)), C.byref(plan)) == 0       # 64 pairs
    assert plan.tile_q == 128
    assert native_lib.tf_attn_plan(C.byref(_attn_desc()), C.byref(plan)) == 0
    assert (plan.k_mn_major, plan.v_mn_major) == (0, 1)     # K [Lk, D], V [Lk, Dv]
    assert 0 < plan.smem_bytes * plan.ctas_per_sm <= 227 * 1024
    # the layouts TileFusion's operator receives: K [Lk, D], V^T [Dv, Lk]
    d = _attn_desc(v_stride_l=1, v_stride_d=2048)
    assert native_lib.tf_attn_plan(C.byref(d), C.byref(plan)) == 0
    assert (plan.k_mn_major, plan.v_mn_major) == (0, 0)
    # the layouts its Python wrapper receives: key [D, Lk], value [Lk, Dv]
    d = _attn_desc(k_stride_l=1, k_stride_d=2048)
    assert native_lib.tf_attn_plan(C.byref(d), C.byref(plan)) == 0
    assert (plan.k_mn_major, plan.v_mn_major) == (1, 1)


def test_head_dims_run_on_the_next_compiled_width(native_lib):
    """Kernels are compiled for head dims 64, 128 and 256; anything else that is a
    multiple of 8 runs zero-padded on the next one, and Dv may differ from D."""
    plan = _cabi.TfAttnPlan()
    for d, dv, kernel in [(64, 64, 64), (40, 40, 64), (96, 96, 128), (128, 128, 128), (64, 128, 128),
                          (128, 64, 128), (192, 192, 256), (256, 256, 256), (72, 200, 256), (8, 8, 64)]:
        desc = _attn_desc(head_dim=d, head_dim_v=dv)
        assert native_lib.tf_attn_plan(C.byref(desc), C.byref(plan)) == 0, (d, dv)
        assert plan.head_dim_kernel == kernel
        if kernel == 256:          # S (128) + O (256) fill tensor memory: one Q tile per CTA, one CTA per SM
            assert (plan.tile_q, plan.ctas_per_sm) == (128, 1)
        assert 0 < plan.smem_bytes * plan.ctas_per_sm <= 227 * 1024


@pytest.mark.parametrize("field,value,code,needle", [
    ("head_dim", 100, _cabi.TF_ERR_UNSUPPORTED, "multiples of 8"),
    ("head_dim", 264, _cabi.TF_ERR_UNSUPPORTED, "multiples of 8"),
    ("dtype", 7, _cabi.TF_ERR_UNSUPPORTED, "half-precision"),
    ("len_kv", 0, _cabi.TF_ERR_BAD_ARG, "positive"),
    ("softmax_scale", -1.0, _cabi.TF_ERR_UNSUPPORTED, "softmax_scale"),
    ("k_stride_d", 3, _cabi.TF_ERR_UNSUPPORTED, "K must be contiguous"),
])
def test_attn_validation_precedes_cuda(native_lib, field, value, code, needle):
    d = _attn_desc(**{field: value})
    if field == "head_dim":
        d.head_dim_v = value
    rc = native_lib.tf_attn_fwd(None, None, None, None, None, C.byref(d), None)
    assert rc == code and needle in native_lib.tf_last_error().decode()


def test_null_pointers_are_rejected(native_lib):
    assert native_lib.tf_attn_fwd(None, None, None, None, None, C.byref(_attn_desc()), None) == _cabi.TF_ERR_BAD_ARG
    assert native_lib.tf_attn_fwd(None, None, None, None, None, None, None) == _cabi.TF_ERR_BAD_ARG
    assert native_lib.tf_decode_plan(None, None) == _cabi.TF_ERR_BAD_ARG


def _decode_desc(b, h, lk, d=128, chunk=512, splits=0):
    x = _cabi.TfDecodeDesc()
    x.dtype, x.batch, x.heads, x.len_kv, x.head_dim = _cabi.TF_F16, b, h, lk, d
    x.kv_chunk, x.num_splits, x.softmax_scale = chunk, splits, 0.088
    x.q_stride_h = d
    x.q_stride_b = h * d
    x.k_stride_h = x.v_stride_h = lk * d
    x.k_stride_b = x.v_stride_b = h * lk * d
    return x


@pytest.mark.parametrize("b,h,lk", [(32, 32, 8192), (4, 32, 131072), (4, 32, 16384), (1, 1, 1), (2, 3, 1000)])
def test_decode_plan_covers_every_key(native_lib, b, h, lk):
    plan = _cabi.TfDecodePlan()
    assert native_lib.tf_decode_plan(C.byref(_decode_desc(b, h, lk)), C.byref(plan)) == 0
    n_chunks = -(-lk // plan.kv_chunk)
    assert plan.kv_chunk == 512
    assert plan.num_splits * plan.chunks_per_split >= n_chunks
    assert (plan.num_splits - 1) * plan.chunks_per_split < n_chunks      # no empty split
    assert plan.workspace_bytes == b * h * plan.num_splits * 130 * 4
    assert 1 <= plan.grid <= 2 * 148
    # round-robin makespan within 2 % of perfect balance when there is enough work
    items = b * h * plan.num_splits
    if items >= 4 * plan.grid:
        span = -(-items // plan.grid) * plan.chunks_per_split
        assert span * plan.grid <= 1.02 * b * h * n_chunks + plan.grid * plan.chunks_per_split


def test_grouped_query_decode_plan(native_lib):
    d = _decode_desc(32, 32, 8192)
    d.heads_kv = 8
    plan = _cabi.TfDecodePlan()
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == 0
    n_tiles = 8192 // 128
    # four query heads per KV head: the rows are replicated in the kernel, four partial rows per
    # (row, split), all counted by num_splits
    assert plan.reserved == 4 and plan.num_splits % 4 == 0
    splits = plan.num_splits // 4
    assert plan.kv_chunk == 128 and splits * plan.chunks_per_split >= n_tiles
    assert (splits - 1) * plan.chunks_per_split < n_tiles
    items = 32 * 8 * splits
    assert -(-items // 148) * plan.chunks_per_split <= 1.05 * 32 * 8 * n_tiles / 148 + plan.chunks_per_split
    assert plan.workspace_bytes == 32 * 32 * plan.num_splits * 130 * 4
    # more than 32 query heads per KV head: no replication
    wide = _decode_desc(2, 128, 8192)
    wide.heads_kv = 2
    assert native_lib.tf_decode_plan(C.byref(wide), C.byref(plan)) == 0 and plan.reserved == 1
    d.heads_kv = 5
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == _cabi.TF_ERR_BAD_ARG


def test_decode_plan_honours_requested_splits(native_lib):
    plan = _cabi.TfDecodePlan()
    assert native_lib.tf_decode_plan(C.byref(_decode_desc(4, 8, 4096, splits=3)), C.byref(plan)) == 0
    assert (plan.num_splits, plan.chunks_per_split) == (3, 3)
    assert native_lib.tf_decode_plan(C.byref(_decode_desc(4, 8, 4096, splits=100)), C.byref(plan)) == 0
    assert (plan.num_splits, plan.chunks_per_split) == (8, 1)


def test_decode_plan_for_an_8bit_cache(native_lib):
    plan = _cabi.TfDecodePlan()
    d = _decode_desc(4, 32, 16384)
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == 0 and plan.stages == 3
    for code in (_cabi.TF_FP8_E4M3, _cabi.TF_FP8_E5M2):
        d.kv_dtype = code
        assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == 0
        assert plan.stages == 3 and plan.workspace_bytes == 4 * 32 * plan.num_splits * 130 * 4
    # grouped-query heads over an 8-bit cache: the split kernel's plan (one item per query head and
    # split), not the two-tile kernel's
    d.heads_kv = 8
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == 0
    assert plan.reserved == 0 and plan.workspace_bytes == 4 * 32 * plan.num_splits * 130 * 4
    d.heads_kv = 0
    d.k_stride_h += 8
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == _cabi.TF_ERR_UNSUPPORTED
    assert "multiples of 16" in native_lib.tf_last_error().decode()
    d.k_stride_h -= 8
    d.v_scale = float("inf")
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == _cabi.TF_ERR_BAD_ARG
    d.v_scale, d.kv_dtype = 0.0, 9
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == _cabi.TF_ERR_UNSUPPORTED
    assert "kv_dtype" in native_lib.tf_last_error().decode()


def test_fp8_conversion_argument_checks_need_no_device(native_lib):
    q, dq = native_lib.tf_fp8_quantize, native_lib.tf_fp8_dequantize
    assert q(None, None, 0, _cabi.TF_F16, _cabi.TF_FP8_E4M3, 1.0, None) == 0            # nothing to do
    assert q(None, None, 16, _cabi.TF_F16, _cabi.TF_FP8_E4M3, 1.0, None) == _cabi.TF_ERR_BAD_ARG
    assert q(None, None, -1, _cabi.TF_F16, _cabi.TF_FP8_E4M3, 1.0, None) == _cabi.TF_ERR_BAD_ARG
    assert q(None, None, 0, _cabi.TF_FP8_E4M3, _cabi.TF_FP8_E4M3, 1.0, None) == _cabi.TF_ERR_UNSUPPORTED
    assert dq(None, None, 0, _cabi.TF_BF16, _cabi.TF_BF16, 1.0, None) == _cabi.TF_ERR_UNSUPPORTED
    assert dq(None, None, 0, _cabi.TF_FP8_E5M2, _cabi.TF_BF16, float("nan"), None) == _cabi.TF_ERR_BAD_ARG
    assert dq(8, 32, 16, _cabi.TF_FP8_E5M2, _cabi.TF_BF16, 1.0, None) == _cabi.TF_ERR_UNSUPPORTED   # misaligned src


@pytest.mark.parametrize("kw,needle", [
    (dict(chunk=100), "kv_chunk"), (dict(chunk=2048), "kv_chunk"), (dict(d=96), "head_dim"),
])
def test_decode_validation(native_lib, kw, needle):
    plan = _cabi.TfDecodePlan()
    rc = native_lib.tf_decode_plan(C.byref(_decode_desc(1, 1, 1024, **kw)), C.byref(plan))
    assert rc == _cabi.TF_ERR_UNSUPPORTED and needle in native_lib.tf_last_error().decode()


def test_paged_cache_validation(native_lib):
    plan = _cabi.TfDecodePlan()
    table = (C.c_int32 * 64)()
    d = _decode_desc(2, 4, 4096)
    d.page_size, d.max_pages, d.num_pages = 512, 8, 32
    d.block_table = C.cast(table, C.c_void_p)
    d.k_stride_page = d.v_stride_page = 4 * 512 * 128
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == 0
    d.page_size = 100
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == _cabi.TF_ERR_UNSUPPORTED
    assert "page_size" in native_lib.tf_last_error().decode()
    d.page_size, d.max_pages = 512, 4                        # 4 pages of 512 keys < 4096 keys
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == _cabi.TF_ERR_BAD_ARG
    d.max_pages, d.block_table = 8, None
    assert native_lib.tf_decode_plan(C.byref(d), C.byref(plan)) == _cabi.TF_ERR_BAD_ARG
    assert "block_table" in native_lib.tf_last_error().decode()


def test_fused_two_gemms_validation(native_lib):
    buf = (C.c_char * 64)()
    p = C.addressof(buf)
    p += (-p) % 16
    rc = native_lib.tf_fused_two_gemms(p, p, p, p, 64, 64, 100, 96, _cabi.TF_F16, 104, 104, 64, 96, None)
    assert rc == _cabi.TF_ERR_UNSUPPORTED and "multiples of 8" in native_lib.tf_last_error().decode()
    rc = native_lib.tf_fused_two_gemms(p, p, p, p, 64, 64, 64, 264, _cabi.TF_F16, 64, 64, 64, 264, None)
    assert rc == _cabi.TF_ERR_UNSUPPORTED and "multiples of 8" in native_lib.tf_last_error().decode()
    rc = native_lib.tf_fused_two_gemms(p, p, p, p, 64, 60, 64, 64, _cabi.TF_F16, 64, 64, 64, 64, None)
    assert rc == _cabi.TF_ERR_UNSUPPORTED and "n to be a multiple of 8" in native_lib.tf_last_error().decode()
    rc = native_lib.tf_fused_two_gemms(p, p, p, p, 64, 64, 64, 64, _cabi.TF_F16, 32, 64, 64, 64, None)
    assert rc == _cabi.TF_ERR_BAD_ARG and "leading dimension" in native_lib.tf_last_error().decode()


def test_workspace_too_small_is_reported(native_lib):
    d = _decode_desc(2, 2, 4096)
    buf = (C.c_char * 64)()           # host memory: never dereferenced, the size check comes first
    p = C.addressof(buf)
    p += (-p) % 16
    rc = native_lib.tf_decode(p, p, p, p, None, p, 16, C.byref(d), None)
    assert rc == _cabi.TF_ERR_WORKSPACE and "workspace" in native_lib.tf_last_error().decode()


def test_torch_operator_schema_matches_tilefusion():
    """The schema string of include/kernels/kernel_list.hpp:25-30, verbatim."""
    import torch

    import tilefusion_b200

    tilefusion_b200.load_torch_ops()
    schema = str(torch.ops.tilefusion.flash_attention.default._schema)
    expected = ("tilefusion::flash_attention(Tensor Q, Tensor K, Tensor V, Tensor(a!) O, "
                "int tile_length_q, int tile_length_kv, int tile_hidden_qk, int tile_hidden_v, "
                "float softmax_scale, bool causal) -> ()")
    assert schema == expected
    # include/kernels/kernel_list.hpp:20-23
    assert str(torch.ops.tilefusion.fused_two_gemms.default._schema) == (
        "tilefusion::fused_two_gemms(Tensor A, Tensor B, Tensor C, Tensor(a!) D, "
        "int tm, int tn, int tk, int tp) -> ()")
    for op in ("flash_attention_lse", "flash_attention_bwd", "flash_decoding", "flash_decoding_partial", "flash_decoding_gathered",
               "flash_decoding_partial_scatter", "flash_decoding_gathered_wait"):
        assert hasattr(torch.ops.tilefusion, op)


def test_operator_refuses_cpu_tensors():
    """No CPU fallback: the operators exist for the CUDA dispatch key only."""
    import torch

    import tilefusion_b200 as tilefusion

    q = torch.zeros(64, 128, dtype=torch.float16)
    with pytest.raises((RuntimeError, NotImplementedError)):
        tilefusion.ops.flash_attention(q, q.t(), q, 64, 128, 128, 128, 0.1, False)


# ---- multi-GPU layer: slice arithmetic and argument validation (no GPU, no NCCL) ----
def test_shard_slices_through_the_cabi(native_lib):
    b, e = C.c_int64(), C.c_int64()
    for total, world in [(1024, 8), (1024, 3), (5, 8), (256, 1), (0, 4)]:
        spans = []
        for r in range(world):
            assert native_lib.tf_shard_head_slice(total, r, world, C.byref(b), C.byref(e)) == 0
            spans.append((b.value, e.value))
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(x[1] == y[0] for x, y in zip(spans, spans[1:]))
        sizes = [y - x for x, y in spans]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    for lk, world, align in [(131072, 8, 128), (5000, 4, 128), (100, 8, 128), (129, 2, 128), (1000, 3, 256)]:
        spans = []
        for r in range(world):
            assert native_lib.tf_shard_kv_slice(lk, r, world, align, C.byref(b), C.byref(e)) == 0
            spans.append((b.value, e.value))
        assert spans[0][0] == 0 and spans[-1][1] == lk
        assert all(x[1] == y[0] for x, y in zip(spans, spans[1:]))
        assert all(x % align == 0 for x, y in spans if y > x)
    assert native_lib.tf_shard_head_slice(8, 8, 8, C.byref(b), C.byref(e)) == _cabi.TF_ERR_BAD_ARG
    assert "rank 8" in native_lib.tf_last_error().decode()
    assert native_lib.tf_shard_head_slice(8, 0, 0, C.byref(b), C.byref(e)) == _cabi.TF_ERR_BAD_ARG
    assert native_lib.tf_shard_kv_slice(8, 0, 1, 0, C.byref(b), C.byref(e)) == _cabi.TF_ERR_BAD_ARG
    assert native_lib.tf_shard_head_slice(8, 0, 1, None, None) == _cabi.TF_ERR_BAD_ARG


@pytest.mark.parametrize("args,code,needle", [
    ((2, 2, None, 0, 4, 32, 128, 0), _cabi.TF_ERR_BAD_ARG, "rank 2"),
    ((0, 65, None, 0, 4, 32, 128, 0), _cabi.TF_ERR_BAD_ARG, "world size"),
    ((0, 1, None, 7, 4, 32, 128, 0), _cabi.TF_ERR_BAD_ARG, "transport"),
    ((0, 1, None, 0, 0, 32, 128, 0), _cabi.TF_ERR_BAD_ARG, "positive"),
    ((0, 1, None, 0, 4, 32, 96, 0), _cabi.TF_ERR_UNSUPPORTED, "head_dim"),
    ((0, 1, None, 0, 4, 32, 128, 9), _cabi.TF_ERR_UNSUPPORTED, "dtype"),
    ((1, 2, None, 0, 4, 32, 128, 0), _cabi.TF_ERR_BAD_ARG, "nccl_id is null"),
])
def test_shard_create_validation_precedes_cuda(native_lib, args, code, needle):
    ctx = C.c_void_p()
    rc = native_lib.tf_shard_create(*args, C.byref(ctx))
    assert rc == code and needle in native_lib.tf_last_error().decode()
    assert not ctx.value
    assert native_lib.tf_shard_create(0, 1, None, 0, 4, 32, 128, 0, None) == _cabi.TF_ERR_BAD_ARG


def test_sharded_calls_reject_bad_arguments(native_lib):
    d = _decode_desc(4, 32, 1024)
    assert native_lib.tf_decode_sharded(None, None, None, None, None, None, C.byref(d), None) == _cabi.TF_ERR_BAD_ARG
    assert "ctx is null" in native_lib.tf_last_error().decode()
    assert native_lib.tf_shard_destroy(None) == 0
    assert native_lib.tf_shard_transport(None) == _cabi.TF_ERR_BAD_ARG
    assert native_lib.tf_shard_unique_id(None) == _cabi.TF_ERR_BAD_ARG
    a = _attn_desc()
    assert native_lib.tf_prefill_sharded(3, 2, None, None, None, None, None, C.byref(a), None, None, None) \
        == _cabi.TF_ERR_BAD_ARG
    assert native_lib.tf_prefill_sharded(0, 2, None, None, None, None, None, C.byref(a), None, None, None) \
        == _cabi.TF_ERR_BAD_ARG
    assert "non-null" in native_lib.tf_last_error().decode()
    assert native_lib.tf_prefill_sharded(0, 2, None, None, None, None, None, None, None, None, None) \
        == _cabi.TF_ERR_BAD_ARG


def test_status_peek_and_wait_limit_without_a_device(native_lib):
    code = C.c_int32(5)
    assert native_lib.tf_device_status_peek(C.byref(code)) == 0 and code.value == 0
    assert native_lib.tf_set_wait_limit_ms(0) == _cabi.TF_ERR_BAD_ARG
    assert native_lib.tf_set_wait_limit_ms(2000) == 0


def test_work_item_counter_words_per_stream_and_per_captured_launch(tmp_path):
    """The word a launch of the two-tile kernel draws its work items from must
    never be shared by launches that can overlap.  tests/queue_words_test.cc
    drives tfb::QueueWords (csrc/registry.h) directly."""
    import shutil
    import subprocess

    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("needs g++")
    exe = tmp_path / "queue_words_test"
    subprocess.run([cxx, "-std=c++17", "-O1", f"-I{ROOT / 'include'}", f"-I{ROOT / 'tilefusion_b200' / 'csrc'}",
                    str(ROOT / "tests" / "queue_words_test.cc"), str(ROOT / "tilefusion_b200" / "csrc" / "registry.cc"),
                    "-pthread", "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "ok" in out.stdout
