"""CPU restatement of the 8-bit floating-point formats.  TEST INFRASTRUCTURE ONLY.

The product never imports this file: it is the checker used by ``tests/`` and
the CPU arm of ``bench.py``.

TileFusion declares ``__fp8_e4m3`` / ``__fp8_e5m2`` as the CUDA types
``__nv_fp8_e4m3`` / ``__nv_fp8_e5m2`` (``include/types/base.hpp:13-16``) and
converts through their constructors (``from_float`` / ``to_float``,
``include/types/base.hpp:70-107``).  The algorithm is therefore that of a
third-party component, the CUDA toolkit's ``cuda_fp8.hpp`` (not part of
TileFusion's tree); what is restated here is the published OCP "8-bit floating
point specification (OFP8)" both follow:

* e4m3: 1 sign, 4 exponent (bias 7), 3 mantissa bits; no infinities; the only
  NaN is S.1111.111; largest finite value 448; subnormals ``m/8 * 2^-6``.
* e5m2: 1 sign, 5 exponent (bias 15), 2 mantissa bits; IEEE-like: S.11111.00 is
  infinity, S.11111.{01,10,11} NaN; largest finite value 57344; subnormals
  ``m/4 * 2^-14``.
* float -> fp8 rounds to nearest, ties to even, and saturates to the largest
  finite value (the ``__NV_SATFINITE`` mode the CUDA constructors use).

Pinning: ``tests/test_oracle.py`` checks ``decode`` / ``encode`` against every
known answer in TileFusion's ``tests/cpp/types/test_fp8.cu`` (:36-175) and
against torch's own ``float8_e4m3fn`` / ``float8_e5m2`` CPU conversions on all
256 codes and on seeded in-range values.
"""

from __future__ import annotations

import numpy as np
import torch

E4M3, E5M2 = "e4m3", "e5m2"

_FORMATS = {
    # exponent bits, mantissa bits, bias, IEEE-like specials
    E4M3: (4, 3, 7, False),
    E5M2: (5, 2, 15, True),
}


def table(kind: str) -> np.ndarray:
    """The 256 values of a format as float32 (NaN / inf where the format has them)."""
    e_bits, m_bits, bias, ieee = _FORMATS[kind]
    out = np.zeros(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        e = (code >> m_bits) & ((1 << e_bits) - 1)
        m = code & ((1 << m_bits) - 1)
        if ieee and e == (1 << e_bits) - 1:
            val = float("inf") if m == 0 else float("nan")
        elif not ieee and e == (1 << e_bits) - 1 and m == (1 << m_bits) - 1:
            val = float("nan")
        elif e == 0:
            val = m / (1 << m_bits) * 2.0 ** (1 - bias)
        else:
            val = (1.0 + m / (1 << m_bits)) * 2.0 ** (e - bias)
        out[code] = sign * val
    return out


def max_finite(kind: str) -> float:
    t = table(kind)
    return float(np.nanmax(np.where(np.isfinite(t), t, -np.inf)))


def decode(codes: torch.Tensor, kind: str) -> torch.Tensor:
    """uint8 codes -> float32 values."""
    t = torch.from_numpy(table(kind))
    return t[codes.to(torch.int64)]


def encode(x: torch.Tensor, kind: str) -> torch.Tensor:
    """float values -> uint8 codes: nearest, ties to the even code, magnitudes
    beyond the largest finite value saturate to it; NaN gives the format's
    canonical NaN (0x7f for e4m3, 0x7f for e5m2 as the CUDA conversion does)."""
    t = table(kind).astype(np.float64)
    n_finite = int(np.sum(np.isfinite(t[:128])))          # non-negative finite codes 0 .. n_finite-1
    mags = t[:n_finite]
    xv = x.detach().to(torch.float64).cpu().numpy()
    a = np.abs(xv)
    hi = np.clip(np.searchsorted(mags, a, side="left"), 0, n_finite - 1)     # first code with value >= |x|
    lo = np.clip(hi - 1, 0, n_finite - 1)
    d_hi, d_lo = np.abs(mags[hi] - a), np.abs(a - mags[lo])
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo)
    code = np.where(a >= mags[-1], n_finite - 1, code)    # saturation (infinities included)
    code = np.where(np.signbit(xv), code | 0x80, code)
    code = np.where(np.isnan(xv), 0x7F, code)
    return torch.from_numpy(code.astype(np.uint8)).reshape(x.shape)


def quantize(x: torch.Tensor, kind: str, factor: float = 1.0) -> torch.Tensor:
    """What ``tf_fp8_quantize`` computes: the 16-bit input widened to fp32,
    multiplied by ``factor`` in fp32, then encoded."""
    return encode(x.float() * torch.tensor(factor, dtype=torch.float32), kind)


def dequantize(codes: torch.Tensor, kind: str, factor: float, dtype: torch.dtype) -> torch.Tensor:
    """What ``tf_fp8_dequantize`` computes: decode, multiply in fp32, round to ``dtype``."""
    return (decode(codes, kind) * torch.tensor(factor, dtype=torch.float32)).to(dtype)
