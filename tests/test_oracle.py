"""The oracle against TileFusion's own FlashAttentionRef outputs (fixtures)."""

import math

import pytest
import torch

from oracle import attention_oracle as orc


def _case(golden, name):
    data, meta = golden
    m = meta[name]
    q = torch.from_numpy(data[f"{name}.q"])
    key_t = torch.from_numpy(data[f"{name}.key_t"])
    v = torch.from_numpy(data[f"{name}.v"])
    ref = torch.from_numpy(data[f"{name}.out_fp32"])
    return m, q, key_t, v, ref


@pytest.mark.parametrize("name", ["ref_case1", "ref_case2", "c1_head", "multi_kv"])
def test_closed_form_matches_reference_class(golden, name):
    m, q, key_t, v, ref = _case(golden, name)
    out, _ = orc.attention_fp32(q, key_t.t(), v, m["softmax_scale"], m["causal"])
    assert orc.max_abs(out, ref) <= 1e-5


@pytest.mark.parametrize("name", ["ref_case1", "ref_case2", "c1_head", "multi_kv"])
@pytest.mark.parametrize("tile_kv", [32, 128])
def test_blocked_matches_reference_class(golden, name, tile_kv):
    m, q, key_t, v, ref = _case(golden, name)
    out, lse = orc.attention_blocked(q, key_t.t(), v, m["softmax_scale"], m["causal"], tile_kv)
    assert orc.max_abs(out, ref) <= 1e-5
    _, lse_ref = orc.attention_fp32(q, key_t.t(), v, m["softmax_scale"], m["causal"])
    assert orc.max_abs(lse, lse_ref) <= 1e-5


def test_reference_fp16_outputs_within_its_own_tolerance(golden):
    # TileFusion's test accepts allclose(atol=1e-2, rtol=1e-2) between its fp16
    # class and its kernel; the fp32 oracle sits inside the same band.
    data, meta = golden
    for name, m in meta.items():
        if not m["has_fp16"]:
            continue
        ref16 = torch.from_numpy(data[f"{name}.out_fp16"]).float()
        ref32 = torch.from_numpy(data[f"{name}.out_fp32"])
        assert torch.allclose(ref16, ref32, atol=1e-2, rtol=1e-2)


def test_causal_blocked_skips_masked_tiles_without_nan():
    q, k, v = orc.seeded_inputs(3, (64, 64), (256, 64), (256, 64), 1.0)
    out, lse = orc.attention_blocked(q, k, v, 0.125, True, 64)
    ref, lse_ref = orc.attention_fp32(q, k, v, 0.125, True)
    assert torch.isfinite(out).all()
    assert orc.max_abs(out, ref) <= 1e-5 and orc.max_abs(lse, lse_ref) <= 1e-5


@pytest.mark.parametrize("len_kv,per_split", [(512, 512), (1000, 256), (4096, 512), (130, 128)])
def test_split_combine_identity(len_kv, per_split):
    q, k, v = orc.seeded_inputs(2, (2, 3, 64), (2, 3, len_kv, 64), (2, 3, len_kv, 64), 1.0)
    scale = 1.0 / math.sqrt(64)
    po, pml = orc.decode_split(q, k, v, scale, per_split)
    out, lse, merged = orc.decode_combine(po, pml)
    ref, lse_ref = orc.decode_fp32(q.unsqueeze(2), k, v, scale)
    assert orc.max_abs(out, ref.squeeze(2)) <= 1e-5
    assert orc.max_abs(lse, lse_ref.squeeze(2)) <= 1e-5
    # merging merged rows again (as after an all-gather of one row per rank) is a no-op
    out2, lse2, _ = orc.decode_combine(merged[..., None, :64], merged[..., None, 64:])
    assert orc.max_abs(out2, out) <= 1e-6 and orc.max_abs(lse2, lse) <= 1e-6


def test_combine_ignores_empty_partials():
    po = torch.randn(4, 3, 16)
    pml = torch.rand(4, 3, 2) + 0.5
    po[:, 1] = 0
    pml[:, 1, 0] = float("-inf")
    pml[:, 1, 1] = 0
    out, lse, _ = orc.decode_combine(po, pml)
    out_ref, lse_ref, _ = orc.decode_combine(po[:, [0, 2]], pml[:, [0, 2]])
    assert orc.max_abs(out, out_ref) <= 1e-6 and orc.max_abs(lse, lse_ref) <= 1e-6
