"""GPU checks of the fast-path arithmetic against the IEEE intrinsics (tests/cuda/math_check.cu):
sqrt on every non-negative normal float, the division sequences on random and structured operands,
both code searches on every float, and the mantissa-trick dequantize on a sweep of scales."""
import ctypes as C
import os
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "cuda"))


@pytest.fixture(scope="module")
def mc():
    import build_mathcheck
    lib = C.CDLL(build_mathcheck.build())
    return lib


def _call(fn, *args):
    bad = (C.c_ulonglong * 1)()
    first = (C.c_uint * 2)()
    assert fn(*args, bad, first) == 0
    return bad[0], (hex(first[0]), hex(first[1]))


def test_sqrt_sequence_is_correctly_rounded_on_every_nonnegative_float(mc):
    # zero, denormals and normals: every finite bit pattern 0 .. 0x7f7fffff
    bad, first = _call(mc.qfc_sqrt, C.c_uint32(0), C.c_uint64(0x7f800000))
    assert bad == 0, first


@pytest.mark.parametrize("mode,a_rng,d_rng", [
    (0, (-40, 10), (-30, 20)),      # update / denominator: den >= eps, numerator small
    (0, (-60, 60), (-60, 60)),      # wide; quotients stay normal (the sequences are not meant for denormal results)
    (1, (-25, 25), (-90, 100)),     # prepared reciprocal, wide
    (2, (-9, -1), (-90, 90)),       # quantize: |a| <= d, down to the smallest midpoint
    (2, (-30, -1), (-60, 90)),
])
@pytest.mark.parametrize("mant_mode", [0, 1, 2])
def test_division_sequences_match_div_rn(mc, mode, a_rng, d_rng, mant_mode):
    per_thread = 4000
    bad, first = _call(mc.qfc_div, C.c_uint64(1234 + 17 * mode + mant_mode), C.c_uint64(per_thread), mode,
                       a_rng[0], a_rng[1], d_rng[0], d_rng[1], mant_mode)
    assert bad == 0, (first, "of", 2 * per_thread * mc.qfc_threads())


@pytest.mark.parametrize("recip_mode", [0, 1], ids=["newton-reciprocal", "rcp.rn"])
@pytest.mark.parametrize("a_exp,d_exp", [(0, 0), (-3, 0), (-7, 5), (10, -20)])
def test_prepared_division_on_every_dividend_mantissa_against_64_divisors(mc, recip_mode, a_exp, d_exp):
    """Structured complement of the random tests: all 2^23 mantissas of the dividend in one binade against 64 divisor
    mantissas (the extremes, their neighbours and a stride in between), 5.4e8 quotients per case, none may differ."""
    bad, first = _call(mc.qfc_div_all_mantissas, a_exp, d_exp, recip_mode)
    assert bad == 0, first


@pytest.mark.parametrize("mode", [0, 1], ids=["prepared", "approx-reciprocal"])
def test_single_correction_division_is_within_one_ulp_and_rarely_off(mc, mode):
    """The one-correction forms used for the requantize divisions and the bf16 parameter update: never more than one
    unit off, and off at all in fewer than one quotient in 10^7 (measured: 0 and 1 of 1.2e9; the rate is printed)."""
    out = (C.c_ulonglong * 4)()
    per_thread = 2000
    assert mc.qfc_div1(C.c_uint64(4321 + mode), C.c_uint64(per_thread), mode, -30, 10, -30, 20, 0, 0, out) == 0
    n = 2 * per_thread * mc.qfc_threads()
    print(f"single-correction division, mode {mode}: {out[0]} of {n} quotients differ from div.rn ({out[0] / n:.2e})")
    assert out[1] == 0
    assert out[0] / n < 1e-7


def test_single_correction_division_changes_no_code(mc):
    """Codes taken from the one-correction quotient against codes from the exact quotient, |a| <= d as in the step:
    no code of either map may differ on 1.2e9 random quotients (a difference needs the quotient to sit on a code
    boundary as well)."""
    out = (C.c_ulonglong * 4)()
    per_thread = 2000
    tot = [0, 0, 0]
    for seed in (7, 8):
        assert mc.qfc_div1(C.c_uint64(seed), C.c_uint64(per_thread), 0, -9, -1, -60, 60, 0, 1, out) == 0
        tot = [tot[0] + out[0], tot[1] + out[2], tot[2] + out[3]]
        assert out[1] == 0
    print(f"single-correction requantize: {tot[0]} quotients differ, {tot[1]} first-moment and {tot[2]} second-moment codes differ")
    assert tot[1] == 0 and tot[2] == 0


def test_product_taken_as_fma_with_zero_then_add_rounds_twice(mc):
    bad, first = _call(mc.qfc_nofuse, C.c_uint64(99), C.c_uint64(2000))
    assert bad == 0, first


def test_searches_match_binary_search_on_every_float(mc):
    bad, first = _call(mc.qfc_search)
    assert bad == 0, first


def test_mantissa_trick_dequantize_matches_table_times_scale(mc):
    bad, first = _call(mc.qfc_dequant_v, C.c_uint32(0x12000000), C.c_uint64(1 << 26))   # scales from 2^-91 up
    assert bad == 0, first
    bad, first = _call(mc.qfc_dequant_v, C.c_uint32(0x2f000000), C.c_uint64(1 << 28))   # around 1e-10 .. 1e-1
    assert bad == 0, first


def test_dispatch_probe_packed_and_integer_instructions_do_not_overlap_for_free(mc):
    """Cycles per warp instruction on one SM sub-partition (four warps), alone and mixed 1 : 1 with packed FMAs: the
    yardstick behind the statement that the step kernels are bound by instruction dispatch.  Printed for the record;
    asserted loosely (a scalar FMA dispatches in about one cycle, a packed one in about two, and an integer
    instruction mixed in costs about a cycle more, never nothing)."""
    import torch
    out = (C.c_double * 12)()
    assert mc.qfc_issue_probe(out) == 0
    try:
        mhz = float(torch.cuda.get_device_properties(0).clock_rate) / 1e3    # maximum SM clock; the probe runs at it
    except Exception:  # noqa: BLE001
        mhz = 1965.0
    per_group = [out[i] * 1e-3 * mhz * 1e6 / (4 * out[11]) for i in range(11)]     # cycles per group of 8 (+8) instructions
    names = ["packed fma", "lop3", "prmt", "funnel shift", "imad", "scalar fma"]
    alone = {n: per_group[i] / 8 for i, n in enumerate(names)}
    mixed = {n: per_group[6 + i] / 8 for i, n in enumerate(names[1:])}
    print(f"SM clock assumed {mhz} MHz; cycles per instruction alone: " + ", ".join(f"{n} {v:.2f}" for n, v in alone.items()))
    print("cycles per (packed fma + one instruction of the class): " + ", ".join(f"{n} {v:.2f}" for n, v in mixed.items()))
    assert 0.8 < alone["scalar fma"] < 1.4
    assert 1.7 < alone["packed fma"] < 2.8
    for n in ("lop3", "prmt", "funnel shift"):
        assert mixed[n] > alone["packed fma"] + 0.5, n          # not hidden behind the packed FMAs
    assert mixed["imad"] > alone["packed fma"] + 1.5             # shares the FMA pipe: fully additive
