"""The 8-bit format oracle against TileFusion's own known answers and torch.

Known answers: tests/cpp/types/test_fp8.cu in TileFusion's tree (:36-175), read
as text -- the values it constructs, and the exact results or tolerances it
expects of from_float / to_float.
"""

import pytest
import torch

from oracle import fp8_oracle as f8

KINDS = [f8.E4M3, f8.E5M2]
TORCH_DTYPE = {f8.E4M3: torch.float8_e4m3fn, f8.E5M2: torch.float8_e5m2}


def _round_trip(value: float, kind: str) -> float:
    return float(f8.decode(f8.encode(torch.tensor([value]), kind), kind)[0])


def test_exactly_representable_values_of_the_reference_suite():
    # test_fp8_construction (test_fp8.cu:36-64)
    assert _round_trip(2.0, f8.E4M3) == 2.0
    assert _round_trip(4.0, f8.E5M2) == 4.0
    for kind in KINDS:
        assert _round_trip(0.0, kind) == 0.0
        assert _round_trip(1.0, kind) == 1.0


@pytest.mark.parametrize("value,tol_e4m3,tol_e5m2", [(0.5, 0.1, 0.1), (3.0, 0.15, 0.25), (9.0, 0.25, 0.5)])
def test_precision_bands_of_the_reference_suite(value, tol_e4m3, tol_e5m2):
    # test_fp8_precision_characteristics (test_fp8.cu:67-106): relative bands
    assert abs(_round_trip(value, f8.E4M3) - value) <= value * tol_e4m3
    assert abs(_round_trip(value, f8.E5M2) - value) <= value * tol_e5m2


def test_conversion_list_of_the_reference_suite_stays_finite():
    # test_fp8_conversion_safety (test_fp8.cu:109-140)
    values = [0.0, 0.0625, 0.125, 0.1875, 0.25, 0.375, 0.5, 0.625, 0.75, 0.875,
              1.0, 1.125, 1.25, 1.375, 1.5, 1.625, 1.75, 1.875,
              2.0, 2.25, 2.5, 2.75, 3.0, 3.25, 3.5, 3.75,
              4.0, 4.5, 5.0, 5.5, 6.0, 6.5, 7.0, 7.5,
              8.0, 9.0, 10.0, 11.0, 12.0, 14.0, 16.0, 20.0, 24.0, 28.0]
    x = torch.tensor(values)
    for kind in KINDS:
        back = f8.decode(f8.encode(x, kind), kind)
        assert torch.isfinite(back).all()


def test_utility_and_arithmetic_cases_of_the_reference_suite():
    # test_fp8_utility_functions (:143-155) and test_fp8_arithmetic (:158-175)
    for kind in KINDS:
        assert abs(_round_trip(1.5, kind) - 1.5) <= 0.01
    a, b = _round_trip(3.0, f8.E4M3), _round_trip(2.0, f8.E5M2)
    assert abs(_round_trip(a + b, f8.E4M3) - 5.0) <= 0.1
    assert abs(_round_trip(a * b, f8.E5M2) - 6.0) <= 0.1


@pytest.mark.parametrize("kind", KINDS)
def test_all_codes_decode_like_torch(kind):
    codes = torch.arange(256, dtype=torch.uint8)
    ours = f8.decode(codes, kind)
    theirs = codes.view(TORCH_DTYPE[kind]).float()
    assert torch.equal(torch.isnan(ours), torch.isnan(theirs))
    ok = ~torch.isnan(ours)
    assert torch.equal(ours[ok], theirs[ok])


@pytest.mark.parametrize("kind", KINDS)
def test_encode_matches_torch_in_range_and_saturates_beyond(kind):
    gen = torch.Generator().manual_seed(11)
    top = f8.max_finite(kind)
    x = torch.cat([
        torch.randn(20000, generator=gen),                       # the bulk of a K/V cache
        torch.randn(20000, generator=gen) * 1e-3,                # subnormal range
        (torch.rand(20000, generator=gen) * 2 - 1) * top,        # up to the largest finite value
        f8.decode(torch.arange(256, dtype=torch.uint8), kind).nan_to_num(0.0, 0.0, 0.0),   # every code is a fixed point
    ])
    # midpoints between neighbouring values: ties go to the even code
    vals = f8.decode(torch.arange(0, 120, dtype=torch.uint8), kind)
    x = torch.cat([x, (vals[:-1] + vals[1:]) / 2, -(vals[:-1] + vals[1:]) / 2])
    ours = f8.encode(x, kind)
    theirs = x.to(TORCH_DTYPE[kind]).view(torch.uint8)
    assert torch.equal(ours, theirs)
    # beyond the range the CUDA constructors saturate (torch's cast does not)
    big = torch.tensor([top * 1.01, top * 4, float("inf"), -top * 2, float("-inf")])
    assert torch.equal(f8.decode(f8.encode(big, kind), kind), torch.tensor([top, top, top, -top, -top]))


@pytest.mark.parametrize("kind", KINDS)
def test_quantize_dequantize_round_trip_with_a_factor(kind):
    gen = torch.Generator().manual_seed(5)
    x = (torch.randn(4096, generator=gen) * 3).to(torch.bfloat16)
    codes = f8.quantize(x, kind, factor=8.0)
    back = f8.dequantize(codes, kind, 1.0 / 8.0, torch.float32)
    # relative error of a normal value is at most half an ulp: 2^-4 (e4m3), 2^-3 (e5m2)
    rel = 2.0 ** -4 if kind == f8.E4M3 else 2.0 ** -3
    big = x.float().abs() > 0.1
    assert ((back - x.float()).abs()[big] <= rel * x.float().abs()[big]).all()
