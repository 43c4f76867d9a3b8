"""Generates ``tests/golden/flash_attention_ref.npz``.

Run where TileFusion's source tree is available (its path is the only
argument)::

    python tests/golden/make_golden.py <path-to-TileFusion>

The script imports TileFusion's own test oracle, the ``FlashAttentionRef`` class
of ``tests/python/test_flash_attn.py:21-134`` (a stub stands in for the
``tilefusion`` package that file imports at line 18, because the compiled
library is not needed by the class), runs it on seeded inputs and stores inputs
and outputs.  The fixtures travel with the repository; the TileFusion tree does
not, so tests only ever read the ``.npz``.

Cases:
  ref_case1 / ref_case2 -- the two parameter sets of TileFusion's test-suite
      (``tests/python/test_flash_attn.py:205-230``), seed 1234 as its autouse
      fixture sets (``:137-140``), drawn on the CPU generator.
  c1_head   -- one head of the plumbing config (Lq=Lk=128, D=64, scale 1/8,
      seed 0) with four KV tiles of 32.
  multi_kv  -- Lq=128, Lk=512, D=128, four KV tiles of 128, so the
      renormalisation across tiles is exercised (the reference's own cases
      have a single KV tile).
Each case stores the class's output computed in fp32 on the fp16-rounded
inputs (``out_fp32``) and, where the CPU supports it, computed in fp16 as the
reference test does (``out_fp16``).
"""

from __future__ import annotations

import importlib.util
import json
import math
import sys
import types
from pathlib import Path

import numpy as np
import torch


def load_reference_class(root: Path):
    stub = types.ModuleType("tilefusion")
    stub_ops = types.ModuleType("tilefusion.ops")
    stub_ops.flash_attention = None
    stub.ops = stub_ops
    sys.modules.setdefault("tilefusion", stub)
    sys.modules.setdefault("tilefusion.ops", stub_ops)
    path = root / "tests" / "python" / "test_flash_attn.py"
    spec = importlib.util.spec_from_file_location("tilefusion_ref_test_flash_attn", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.FlashAttentionRef


def run_ref(cls, q, k_t, v, tiles, scale, causal, dtype):
    """Calls the class the way TileFusion's test does: key is [D, Lk].

    The class allocates its output with ``torch.empty`` and multiplies that
    uninitialised buffer by a zero row-sum on the first tile; whatever the
    allocator hands back (inf or NaN bit patterns included) would survive as
    NaN.  ``torch.empty`` is therefore served by ``torch.zeros`` for the duration
    of the call, which leaves the computed values exactly as the class defines
    them."""
    ref = cls(*tiles, scale, causal)
    real_empty = torch.empty
    torch.empty = lambda *a, **kw: torch.zeros(*a, **kw)
    try:
        out = ref(q.to(dtype), k_t.to(dtype), v.to(dtype))
    finally:
        torch.empty = real_empty
    if not torch.isfinite(out).all():
        raise RuntimeError("reference produced non-finite output")
    return out


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path-to-TileFusion-source-tree>")
    root = Path(sys.argv[1])
    cls = load_reference_class(root)
    cases = [
        # name, Lq, Lk, D, Dv, tiles(tq, tkv, thqk, thv), scale, causal, seed, sigma
        ("ref_case1", 64, 128, 128, 128, (64, 128, 128, 128), 1.0 / math.sqrt(128), False, 1234, 1.0),
        ("ref_case2", 128, 128, 128, 128, (64, 128, 128, 128), 1.0 / math.sqrt(128), True, 1234, 1.0),
        ("c1_head", 128, 128, 64, 64, (64, 32, 64, 64), 1.0 / 8.0, False, 0, 1.0),
        ("multi_kv", 128, 512, 128, 128, (64, 128, 128, 128), 1.0 / math.sqrt(128), False, 7, 1.0),
    ]
    arrays = {}
    meta = {}
    for name, lq, lk, d, dv, tiles, scale, causal, seed, sigma in cases:
        torch.manual_seed(seed)
        q = (torch.randn(lq, d) * sigma).half()
        k_t = (torch.randn(d, lk) * sigma).half()   # the reference's key layout
        v = (torch.randn(lk, dv) * sigma).half()
        out32 = run_ref(cls, q, k_t, v, tiles, scale, causal, torch.float32)
        try:
            out16 = run_ref(cls, q, k_t, v, tiles, scale, causal, torch.float16).float()
        except RuntimeError:
            out16 = None
        arrays[f"{name}.q"] = q.numpy()
        arrays[f"{name}.key_t"] = k_t.numpy()
        arrays[f"{name}.v"] = v.numpy()
        arrays[f"{name}.out_fp32"] = out32.numpy()
        if out16 is not None:
            arrays[f"{name}.out_fp16"] = out16.numpy().astype(np.float16)
        meta[name] = dict(len_q=lq, len_kv=lk, head_dim=d, head_dim_v=dv, tiles=list(tiles),
                          softmax_scale=scale, causal=causal, seed=seed, has_fp16=out16 is not None)
    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    out_path = Path(__file__).resolve().parent / "flash_attention_ref.npz"
    np.savez_compressed(out_path, **arrays)
    print("wrote", out_path, {k: v.shape for k, v in arrays.items()})


if __name__ == "__main__":
    main()
