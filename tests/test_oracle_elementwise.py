"""The element-wise oracle against outputs of the reference's own reference.py functions.

``tests/golden/elementwise.npz`` was written by ``tests/golden/make_golden_elementwise.py``, which
executes the reference's ``reference_swiglu`` (operators/swiglu/reference.py:7-27),
``reference_residual_rms`` and ``precise_residual_rms`` (operators/residual_rms/reference.py:7-66)
on CPU. Bit-exact wherever the arithmetic is pinned (the 16-bit sum, the quantiser); where the
float32 summation order of the mean of squares or the last bit of exp() can move a value across a
rounding boundary, at most a stated fraction of outputs may differ, by one step.
"""
import os

import numpy as np
import pytest

import elementwise_oracle as ew
from oracle import E4M3FN, E4M3FNUZ, F16, dequantize

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "elementwise.npz"))

MAX_FRACTION_OFF_BY_ONE = 2e-3


def _f16(bits):
    return np.asarray(bits, dtype=np.uint16).view(np.float16)


def _check_bytes(mine, golden):
    distance = ew.fp8_step_distance(mine, golden)
    assert distance.max() <= 1, f"fp8 outputs {distance.max()} codes apart"
    differing = int((distance != 0).sum())
    assert differing <= max(1, MAX_FRACTION_OFF_BY_ONE * distance.size), f"{differing} of {distance.size} bytes differ"


@pytest.mark.parametrize("idx", range(int(GOLDEN["swiglu_count"][0])))
def test_swiglu_matches_the_reference(idx):
    gate_up = _f16(GOLDEN[f"s{idx}_gate_up"])
    scale = float(GOLDEN[f"s{idx}_scale"][0])
    # reference_swiglu(scale) returns the bytes the kernel writes for the doubled scale
    mine = ew.reference_swiglu(gate_up, 2.0 * scale, F16, E4M3FNUZ)
    _check_bytes(mine, GOLDEN[f"s{idx}_bytes"])
    assert not (mine == 0x80).any()
    # the same bytes read as e4m3fn are the e4m3fn encoding for the undoubled scale, up to -0
    fn = ew.reference_swiglu(gate_up, scale, F16, E4M3FN)
    assert np.array_equal(np.where(fn == 0x80, 0, fn), mine)


@pytest.mark.parametrize("idx", range(int(GOLDEN["rms_count"][0])))
def test_residual_rms_matches_the_reference(idx):
    x, res, w = (_f16(GOLDEN[f"r{idx}_{name}"]) for name in ("input", "residual", "weight"))
    eps = float(GOLDEN[f"r{idx}_epsilon"][0])
    scale = float(GOLDEN[f"r{idx}_scale"][0])

    y16, new_res = ew.reference_residual_rms(x, res, w, eps, None, F16, form="torch")
    assert np.array_equal(new_res.view(np.uint16), GOLDEN[f"r{idx}_new_residual"]), "the 16-bit sum is exact"
    distance = ew.ulp16_distance(y16, _f16(GOLDEN[f"r{idx}_out_f16"]), F16)
    assert distance.max() <= 1
    assert (distance != 0).sum() <= max(1, MAX_FRACTION_OFF_BY_ONE * distance.size)

    y8, _ = ew.reference_residual_rms(x, res, w, eps, 2.0 * scale, F16, E4M3FNUZ, form="torch")
    _check_bytes(y8, GOLDEN[f"r{idx}_out_bytes"])

    p8 = ew.precise_residual_rms(x, res, w, eps, 2.0 * scale, F16, E4M3FNUZ)
    _check_bytes(p8, GOLDEN[f"r{idx}_precise_bytes"])
    key = f"r{idx}_precise_f32"
    if key in GOLDEN:
        p64 = ew.precise_residual_rms(x, res, w, eps, None, F16)
        np.testing.assert_allclose(p64.astype(np.float32), GOLDEN[key], rtol=3e-7, atol=1e-30)


@pytest.mark.parametrize("idx", range(int(GOLDEN["rms_count"][0])))
def test_kernel_form_is_no_further_from_precise_than_the_torch_form(idx):
    """The reference's acceptance test for its kernel (tests/test_residual_rms.py:56-87), applied
    to the oracle's statement of that kernel's arithmetic against the golden torch outputs."""
    x, res, w = (_f16(GOLDEN[f"r{idx}_{name}"]) for name in ("input", "residual", "weight"))
    eps = float(GOLDEN[f"r{idx}_epsilon"][0])
    scale = float(GOLDEN[f"r{idx}_scale"][0])
    kernel8, _ = ew.reference_residual_rms(x, res, w, eps, 2.0 * scale, F16, E4M3FNUZ, form="kernel")
    value = lambda q: dequantize(q, E4M3FNUZ).astype(np.float64)
    precise = value(GOLDEN[f"r{idx}_precise_bytes"])
    err_kernel = np.abs(value(kernel8) - precise)
    err_torch = np.abs(value(GOLDEN[f"r{idx}_out_bytes"]) - precise)
    assert err_kernel.max() <= err_torch.max()
    assert err_kernel.mean() <= err_torch.mean() + 1e-6
    assert 100.0 * (err_kernel > err_torch).mean() < 0.1 or err_kernel.size < 1000


def test_16_bit_helpers_round_like_the_hardware():
    rng = np.random.default_rng(5)
    a = rng.standard_normal(4096).astype(np.float16)
    b = (rng.standard_normal(4096) * 37).astype(np.float16)
    assert np.array_equal(ew.add16(a, b, F16), a + b)
    assert np.array_equal(ew.mul16(a, b, F16), a * b)
    assert ew.fp8_step_distance(np.array([0x01, 0x81, 0x7E]), np.array([0x00, 0x01, 0x7D])).tolist() == [1, 2, 1]


def test_quantiser_is_idempotent_on_its_own_grid():
    """Every finite e4m3fn value encodes back to its own byte, for both output kinds (the fnuz
    form drops the sign of zero and halves the value a byte is worth)."""
    from oracle import fp8_table

    codes = np.array([b for b in range(256) if b not in (0x7F, 0xFF)], dtype=np.uint8)
    values = fp8_table(E4M3FN)[codes]
    again = ew.fp8_bytes(values, 1.0, E4M3FN)
    assert np.array_equal(again, codes)
    as_fnuz = ew.fp8_bytes(values / 2, 1.0, E4M3FNUZ)          # a fnuz byte is worth half the fn byte
    assert np.array_equal(as_fnuz, np.where(codes == 0x80, 0, codes))
    # saturation: never the NaN pattern, in either kind
    big = np.array([1e9, -1e9, 449.0, -449.0, 460.0], dtype=np.float32)
    assert set(ew.fp8_bytes(big, 1.0, E4M3FN).tolist()) == {0x7E, 0xFE}
    assert set(ew.fp8_bytes(big, 1.0, E4M3FNUZ).tolist()) == {0x7E, 0xFE}


def test_residual_rms_forms_share_the_sum_and_scale_invariance():
    """Both restatements update the residual identically; doubling the scale with the fnuz kind
    gives the bytes of the e4m3fn kind (up to the sign of zero): the identity the drop-in relies on."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((6, 256)).astype(np.float16)
    res = rng.standard_normal((6, 256)).astype(np.float16)
    w = rng.standard_normal(256).astype(np.float16)
    for form in ("kernel", "torch"):
        out_fn, sum_fn = ew.reference_residual_rms(x, res, w, 1e-5, 0.02, F16, E4M3FN, form=form)
        out_fnuz, sum_fnuz = ew.reference_residual_rms(x, res, w, 1e-5, 0.04, F16, E4M3FNUZ, form=form)
        assert np.array_equal(sum_fn.view(np.uint16), (x + res).view(np.uint16))
        assert np.array_equal(sum_fn.view(np.uint16), sum_fnuz.view(np.uint16))
        assert np.array_equal(np.where(out_fn == 0x80, 0, out_fn), out_fnuz)
    zero = np.zeros((2, 64), dtype=np.float16)
    out, _ = ew.reference_residual_rms(zero, zero, np.ones(64, dtype=np.float16), 1e-5, None, F16)
    assert np.array_equal(out.view(np.uint16), zero.view(np.uint16)), "epsilon keeps an all-zero row finite"
