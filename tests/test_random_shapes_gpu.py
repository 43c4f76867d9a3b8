"""Seeded random shapes through the C-ABI against the oracle: prefill (+ backward
on every other case) and decode (one query head per KV head, grouped-query,
8-bit cache), ragged lengths, both head dims, both dtypes, causal or not.

Tolerances are those of the dedicated test files: max-abs <= 2e-2; relative-L2
<= 1e-3 (fp16) or 1.2 x the computed bf16 bound; |LSE| <= 1e-3; gradients
relative-L2 <= 2e-3 (fp16) / 8e-3 (bf16), an exactly-zero gradient <= 2e-3 absolute.
"""

import math
import random

import pytest
import torch

from oracle import attention_oracle as orc
from oracle import fp8_oracle as f8

pytestmark = pytest.mark.gpu


def _check(failures, name, got, ref, tol_abs, tol_rel):
    g = got.float().cpu()
    if not torch.isfinite(g).all():
        failures.append((name, "non-finite"))
        return
    ma, rl = orc.max_abs(g, ref), orc.rel_l2(g, ref)
    if ma > tol_abs or rl > tol_rel:
        failures.append((name, ma, rl))


@pytest.mark.parametrize("seed", [1, 2])
def test_random_prefill_and_backward_shapes(seed):
    from cabi_helpers import attn_bwd, attn_fwd, device_status

    rng = random.Random(seed)
    failures = []
    for it in range(16):
        d = rng.choice([64, 128])
        dt = rng.choice([torch.float16, torch.bfloat16])
        b, h = rng.choice([1, 2, 3]), rng.choice([1, 2, 5, 37])
        lq = rng.choice([1, 7, 64, 127, 128, 129, 255, 256, 300, 513, 777])
        lk = rng.choice([8, 16, 120, 128, 136, 256, 264, 520, 1000])
        causal = rng.random() < 0.5
        tile_q = rng.choice([0, 0, 256])
        q, k, v = orc.seeded_inputs(1000 * seed + it, (b, h, lq, d), (b, h, lk, d), (b, h, lk, d), 0.7, dt)
        sc = 1 / math.sqrt(d)
        o, lse = attn_fwd(q.cuda(), k.cuda(), v.cuda(), sc, causal, tile_q=tile_q)
        ref, lse_ref = orc.attention_fp32(q, k, v, sc, causal)
        name = f"fwd B{b} H{h} Lq{lq} Lk{lk} D{d} causal={causal} {dt} tile_q={tile_q}"
        _check(failures, name, o, ref, 2e-2, 1e-3 if dt == torch.float16 else 1.2 * orc.rel_l2_bound(ref, dt))
        _check(failures, name + " lse", lse, lse_ref, 1e-3, float("inf"))
        if it % 2 == 0:
            d_o = (torch.randn(b, h, lq, d, generator=torch.Generator().manual_seed(it)) * 0.7).to(dt)
            grads = attn_bwd(q.cuda(), k.cuda(), v.cuda(), o, d_o.cuda(), lse, sc, causal)
            refs = orc.attention_bwd_fp32(q, k, v, d_o, sc, causal)
            for nm, got, want in zip(("dq", "dk", "dv"), grads, refs):
                g = got.float().cpu()
                if not torch.isfinite(g).all():
                    failures.append((name + " " + nm, "non-finite"))
                elif want.abs().max() < 1e-6:
                    if g.abs().max() > 2e-3:
                        failures.append((name + " " + nm, "zero reference", g.abs().max().item()))
                elif orc.rel_l2(g, want) > (2e-3 if dt == torch.float16 else 8e-3):
                    failures.append((name + " " + nm, orc.rel_l2(g, want)))
    assert device_status() == 0
    assert not failures, failures


@pytest.mark.parametrize("seed", [1, 2])
def test_random_decode_shapes(seed):
    from cabi_helpers import decode, device_status

    rng = random.Random(seed)
    failures = []
    for it in range(20):
        d = rng.choice([64, 128])
        dt = rng.choice([torch.float16, torch.bfloat16])
        b, hkv = rng.choice([1, 2, 5]), rng.choice([1, 2, 3])
        g = rng.choice([1, 1, 2, 4, 8, 32, 64])
        lk = rng.choice([1, 31, 33, 127, 128, 129, 640, 1000, 2049, 5000])
        chunk, splits = rng.choice([128, 256, 512, 1024]), rng.choice([0, 0, 1, 3])
        fp8 = g <= 8 and rng.random() < 0.5
        q, k, v = orc.seeded_inputs(2000 * seed + it, (b, hkv * g, 1, d), (b, hkv, lk, d), (b, hkv, lk, d), 1.0, dt)
        name = f"decode B{b} Hkv{hkv} group{g} Lk{lk} D{d} chunk{chunk} splits{splits} fp8={fp8} {dt}"
        if fp8:
            kind = rng.choice([f8.E4M3, f8.E5M2])
            tdt = torch.float8_e4m3fn if kind == f8.E4M3 else torch.float8_e5m2
            k8, v8 = f8.quantize(k, kind, 2.0), f8.quantize(v, kind, 2.0)
            o, lse = decode(q.cuda(), k8.view(tdt).cuda(), v8.view(tdt).cuda(), None, chunk, splits,
                            k_scale=0.5, v_scale=0.5)
            ref, lse_ref = orc.decode_fp32(q, (f8.decode(k8, kind) * 0.5).repeat_interleave(g, dim=1),
                                           (f8.decode(v8, kind) * 0.5).repeat_interleave(g, dim=1))
        else:
            o, lse = decode(q.cuda(), k.cuda(), v.cuda(), None, chunk, splits)
            ref, lse_ref = orc.decode_fp32(q, k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1))
        tol = 1e-3 if dt == torch.float16 else 1.2 * orc.rel_l2_bound(ref, dt, g > 1)
        _check(failures, name, o, ref, 2e-2, tol)
        _check(failures, name + " lse", lse, lse_ref, 1e-3, float("inf"))
    assert device_status() == 0
    assert not failures, failures
