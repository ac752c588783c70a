"""Parity of the two element-wise CUDA kernels (swiglu, residual + RMS norm) with the CPU oracle and
with the reference's own acceptance criteria. Everything here needs a B200.

Criteria.
* Against the oracle (``oracle/elementwise_oracle.py``, pinned to the reference's outputs): the
  updated residual is bit-exact; fp8 and 16-bit outputs are identical except where the float32
  summation order of the mean of squares, or the last bit of exp(), moves a value across a rounding
  boundary: at most ``MAX_FRACTION_OFF_BY_ONE`` of the outputs, by one step of the output format
  (two for the 16-bit output of residual_rms, which is rounded twice).
* The reference's tests, restated: swiglu within atol 1e-2 / rtol 0.15 of the torch statement with
  fewer than 10 differing elements (tests/test_swiglu.py:23-40); residual_rms no further from the
  high-precision statement than the torch statement is (tests/test_residual_rms.py:56-87).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_FRACTION_OFF_BY_ONE = 2e-3
# A 16-bit output is round16(round16(x * normaliser) * weight): when the inner rounding moves by one
# step just below a power of two and the product lands just above one, the outputs are two steps apart.
MAX_16BIT_STEPS = 2


@pytest.fixture(scope="module")
def capi(native_build):
    from hf_rocm_kernels import _capi

    return _capi


@pytest.fixture(scope="module")
def ew(oracle_mod):
    import elementwise_oracle

    return elementwise_oracle


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _carrier(t: torch.Tensor) -> np.ndarray:
    """16-bit tensor -> the oracle's carrier (float16 array, or uint16 bits for bfloat16)."""
    bits = t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    return bits if t.dtype == torch.bfloat16 else bits.view(np.float16)


def _kinds(oracle_mod, in_dtype, out_dtype):
    dtype = oracle_mod.BF16 if in_dtype == torch.bfloat16 else oracle_mod.F16
    kind = oracle_mod.E4M3FNUZ if out_dtype == torch.float8_e4m3fnuz else oracle_mod.E4M3FN
    return dtype, kind


def _assert_bytes_close(ew, got: torch.Tensor, expect: np.ndarray, label):
    got_np = got.view(torch.uint8).cpu().numpy()
    distance = ew.fp8_step_distance(got_np, expect)
    assert distance.max(initial=0) <= 1, (label, int(distance.max()))
    differing = int((distance != 0).sum())
    assert differing <= max(1, MAX_FRACTION_OFF_BY_ONE * distance.size), (label, differing, distance.size)
    return differing


def _device_ok(capi):
    torch.cuda.synchronize()
    code, word = capi.device_status(clear=True)
    assert code == 0, f"device status word {word:#x}"


# ------------------------------------------------------------------------------------- swiglu
SWIGLU_SHAPES = [(r, h) for r in (1, 3, 16, 256) for h in (8, 24, 512, 4096, 6656)] + [(2048, 6656), (16, 14336)]


@pytest.mark.parametrize("force_scalar", [False, True])
@pytest.mark.parametrize("buffer_cols", [0, 1024])
@pytest.mark.parametrize("rows,hidden", SWIGLU_SHAPES)
def test_swiglu_matches_the_oracle_and_the_reference_criteria(oracle_mod, ew, capi, dev, rows, hidden, buffer_cols,
                                                              force_scalar):
    from hf_rocm_kernels.operators.swiglu import generate_swiglu_data, reference_swiglu, swiglu
    from hf_rocm_kernels.utils.testing import compare_x_with_ref

    gate_up, scale, next_buffer = generate_swiglu_data(rows, hidden, buffer_cols, seed=0, device=dev)
    if next_buffer is not None:
        next_buffer.fill_(3.0)
    out = swiglu(gate_up, scale.mul(2), next_buffer, force_scalar=force_scalar)
    _device_ok(capi)
    assert out.dtype == torch.float8_e4m3fnuz and tuple(out.shape) == (rows, hidden)
    if next_buffer is not None:
        assert int(torch.count_nonzero(next_buffer)) == 0

    expect = ew.reference_swiglu(_carrier(gate_up), 2.0 * float(scale), oracle_mod.F16, oracle_mod.E4M3FNUZ)
    _assert_bytes_close(ew, out, expect, (rows, hidden))

    ref = reference_swiglu(gate_up, scale, None)
    max_error, max_relative_error, changes = compare_x_with_ref(out.float(), ref.float())
    assert max_error < 1e-2 and max_relative_error < 0.15 and changes < 10, (max_error, max_relative_error, changes)


@pytest.mark.parametrize("in_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fnuz, torch.float8_e4m3fn])
def test_swiglu_dtypes_through_the_c_abi(oracle_mod, ew, capi, dev, in_dtype, out_dtype):
    rows, hidden = 16, 14336
    torch.manual_seed(11)
    gate_up = (torch.randn(rows, 2 * hidden, device=dev) * 1.5).to(in_dtype)
    scale = torch.tensor([0.37], device=dev)
    out = torch.empty((rows, hidden), dtype=out_dtype, device=dev)
    next_buffer = torch.full((rows, 4096), -1.0, dtype=in_dtype, device=dev)
    capi.check(capi.swiglu(gate_up, scale, out, next_buffer))
    _device_ok(capi)
    dtype, kind = _kinds(oracle_mod, in_dtype, out_dtype)
    expect = ew.reference_swiglu(_carrier(gate_up), 0.37, dtype, kind)
    _assert_bytes_close(ew, out, expect, (in_dtype, out_dtype))
    assert int(torch.count_nonzero(next_buffer)) == 0


def test_swiglu_saturates_below_the_nan_byte_and_has_no_fnuz_negative_zero(oracle_mod, ew, capi, dev):
    hidden = 64
    gate = torch.tensor([30.0, 30.0, -1e-4, 1e-4, 0.0, -0.0, 8.0, -30.0] * 8, device=dev)
    up = torch.tensor([1000.0, -1000.0, 1e-4, -1e-4, 5.0, 5.0, -0.0, 1000.0] * 8, device=dev)
    gate_up = torch.cat([gate, up]).reshape(1, 2 * hidden).to(torch.float16)
    scale = torch.tensor([1.0], device=dev)
    for out_dtype, scalar in ((torch.float8_e4m3fnuz, False), (torch.float8_e4m3fnuz, True),
                              (torch.float8_e4m3fn, False), (torch.float8_e4m3fn, True)):
        out = torch.empty((1, hidden), dtype=out_dtype, device=dev)
        capi.check(capi.swiglu(gate_up, scale, out, None, force_scalar=scalar))
        _device_ok(capi)
        got = out.view(torch.uint8).cpu().numpy()
        dtype, kind = _kinds(oracle_mod, torch.float16, out_dtype)
        assert np.array_equal(got, ew.reference_swiglu(_carrier(gate_up), 1.0, dtype, kind)), out_dtype
        assert not np.isin(got, (0x7F, 0xFF)).any(), "0x7f/0xff would be NaN to an e4m3fn consumer"
        assert got[0, 0] == 0x7E and got[0, 1] == 0xFE
        if out_dtype == torch.float8_e4m3fnuz:
            assert not (got == 0x80).any(), "0x80 is NaN in e4m3fnuz"
        else:
            assert (got == 0x80).any(), "e4m3fn keeps its negative zero"


def test_swiglu_unaligned_views_take_the_scalar_kernel_and_stay_in_bounds(oracle_mod, ew, capi, dev):
    rows, hidden = 5, 40
    torch.manual_seed(3)
    backing = torch.randn(rows * 2 * hidden + 1, device=dev).to(torch.float16)
    gate_up = backing[1:].view(rows, 2 * hidden)                       # 2-byte aligned only
    out_backing = torch.full((rows * hidden + 6,), 0x55, dtype=torch.uint8, device=dev)
    out = out_backing[3:3 + rows * hidden].view(rows, hidden).view(torch.float8_e4m3fnuz)
    buf_backing = torch.full((rows * 12 + 2,), 9.0, dtype=torch.float16, device=dev)
    next_buffer = buf_backing[1:1 + rows * 12].view(rows, 12)
    scale = torch.tensor([1.3], device=dev)
    capi.check(capi.swiglu(gate_up, scale, out, next_buffer))
    _device_ok(capi)
    expect = ew.reference_swiglu(_carrier(gate_up), 1.3, oracle_mod.F16, oracle_mod.E4M3FNUZ)
    _assert_bytes_close(ew, out, expect, "unaligned")
    assert int(torch.count_nonzero(next_buffer)) == 0
    guard = out_backing.cpu().numpy()
    assert (guard[:3] == 0x55).all() and (guard[-3:] == 0x55).all()
    assert float(buf_backing[0]) == 9.0 and float(buf_backing[-1]) == 9.0


def test_swiglu_empty_and_invalid_inputs(capi, dev):
    scale = torch.tensor([1.0], device=dev)
    empty_in = torch.empty((0, 64), dtype=torch.float16, device=dev)
    empty_out = torch.empty((0, 32), dtype=torch.float8_e4m3fnuz, device=dev)
    assert capi.swiglu(empty_in, scale, empty_out, None) == 0
    gate_up = torch.zeros((2, 64), dtype=torch.float32, device=dev)
    out = torch.empty((2, 32), dtype=torch.float8_e4m3fn, device=dev)
    assert capi.swiglu(gate_up, scale, out, None) == 8      # float32 input: HFRK_BAD_DTYPE
    lib = capi.lib
    g16 = torch.zeros((2, 64), dtype=torch.float16, device=dev)
    assert lib.hfrk_swiglu_fp8(g16.data_ptr(), scale.data_ptr(), out.data_ptr(), 0, 2, 32, 0, capi.F32, capi.E4M3FN,
                               0, 0) == 8
    assert lib.hfrk_swiglu_fp8(g16.data_ptr(), scale.data_ptr(), out.data_ptr(), 0, 2, 32, 0, capi.F16, 5, 0, 0) == 8
    assert lib.hfrk_swiglu_fp8(g16.data_ptr(), scale.data_ptr(), out.data_ptr(), 0, -1, 32, 0, capi.F16, 0, 0, 0) == 6
    assert lib.hfrk_swiglu_fp8(g16.data_ptr(), scale.data_ptr(), out.data_ptr(), 0, 2, 32, 8, capi.F16, 0, 0, 0) == 6
    with pytest.raises(RuntimeError):
        torch.ops._HFRK_C.swiglu(gate_up, scale, out, torch.empty((2, 0), dtype=torch.float16, device=dev), 64, False)


# ----------------------------------------------------------------------------- residual + RMS norm
RMS_SHAPES = [(r, c) for r in (1, 3, 16, 64) for c in (8, 24, 128, 512, 4096, 16384)] + [(256, 4096), (256, 16384)]
RMS_MODES = [(torch.float16, 0), (torch.float8_e4m3fnuz, 0), (torch.float8_e4m3fnuz, 32),
             (torch.float8_e4m3fnuz, 1024)]


def _reference_acceptance(out, ref, precise):
    from hf_rocm_kernels.utils.testing import compare_x_and_ref_to_precise

    (delta_x_max, delta_ref_max, delta_x_mean, delta_ref_mean, regression_percentage, regression_max,
     regression_mean) = compare_x_and_ref_to_precise(out.float(), ref.float(), precise.float())
    assert delta_x_max <= delta_ref_max, (delta_x_max, delta_ref_max)
    assert delta_x_mean <= delta_ref_mean + 1e-6, (delta_x_mean, delta_ref_mean)
    assert regression_percentage < 0.1, regression_percentage
    assert regression_max <= 0.25 and regression_mean < 1e-4, (regression_max, regression_mean)


@pytest.mark.parametrize("force_scalar", [False, True])
@pytest.mark.parametrize("dtype,buffer_cols", RMS_MODES)
@pytest.mark.parametrize("rows,cols", RMS_SHAPES)
def test_residual_rms_matches_the_oracle_and_the_reference_criteria(oracle_mod, ew, capi, dev, rows, cols, dtype,
                                                                    buffer_cols, force_scalar):
    from hf_rocm_kernels.operators.residual_rms import (generate_residual_rms_data, precise_residual_rms,
                                                         reference_residual_rms, residual_rms)

    x, res, weight, epsilon, scale, next_buffer = generate_residual_rms_data(
        rows=rows, cols=cols, buffer_cols=buffer_cols, dtype=dtype, seed=0, device=dev)
    if next_buffer is not None:
        next_buffer.fill_(3.0)
    out, new_res = residual_rms(input=x.clone(), residual=res.clone(), weight=weight, epsilon=epsilon,
                                scale_tensor=scale, next_buffer=next_buffer, force_scalar=force_scalar)
    _device_ok(capi)
    if next_buffer is not None:
        # zeroed with fp8 output only; a 16-bit output leaves the buffer alone, as the reference does
        # (csrc/op_src/residual_rms/residual_rms_dispatch.cu:33-43)
        if scale is None:
            assert bool((next_buffer == 3.0).all())
        else:
            assert int(torch.count_nonzero(next_buffer)) == 0

    scale_f = None if scale is None else float(scale)
    expect, expect_res = ew.reference_residual_rms(_carrier(x), _carrier(res), _carrier(weight), epsilon, scale_f,
                                                   oracle_mod.F16, oracle_mod.E4M3FNUZ, form="kernel")
    assert np.array_equal(_carrier(new_res).view(np.uint16), expect_res.view(np.uint16)), "the 16-bit sum is exact"
    if scale is None:
        assert out.dtype == torch.float16
        distance = ew.ulp16_distance(_carrier(out), expect, oracle_mod.F16)
        assert distance.max() <= MAX_16BIT_STEPS
        assert (distance != 0).sum() <= max(1, MAX_FRACTION_OFF_BY_ONE * distance.size)
    else:
        assert out.dtype == torch.float8_e4m3fnuz
        _assert_bytes_close(ew, out, expect, (rows, cols))

    half_scale = None if scale is None else scale.div(2)
    ref, ref_res, _ = reference_residual_rms(input=x.clone(), residual=res.clone(), weight=weight, epsilon=epsilon,
                                             scale_tensor=half_scale)
    assert torch.equal(new_res, ref_res)
    precise, _ = precise_residual_rms(input=x.clone(), residual=res.clone(), weight=weight, epsilon=epsilon,
                                      scale_tensor=half_scale)
    _reference_acceptance(out, ref, precise)


@pytest.mark.parametrize("out_dtype", [None, torch.float8_e4m3fnuz, torch.float8_e4m3fn])
@pytest.mark.parametrize("in_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols,threads", [(16, 4096, 0), (4, 8192, 256), (2, 32768, 0), (3, 40960, 1024),
                                               (7, 1000, 64), (5, 4104, 0)])
def test_residual_rms_dtypes_long_rows_and_cta_sizes(oracle_mod, ew, capi, dev, rows, cols, threads, in_dtype,
                                                     out_dtype):
    torch.manual_seed(rows * 131 + cols)
    x = torch.randn(rows, cols, device=dev).to(in_dtype)
    res = (torch.randn(rows, cols, device=dev) * 2).to(in_dtype)
    weight = (1 + 0.1 * torch.randn(cols, device=dev)).to(in_dtype)
    scale = None if out_dtype is None else torch.tensor([0.0123], device=dev)
    out = torch.empty((rows, cols), dtype=in_dtype if out_dtype is None else out_dtype, device=dev)
    next_buffer = torch.full((rows, 56), 2.0, dtype=in_dtype, device=dev)
    new_res = res.clone()
    capi.check(capi.residual_rms(x, new_res, weight, scale, 1e-5, out, next_buffer, num_threads=threads))
    _device_ok(capi)
    dtype, kind = _kinds(oracle_mod, in_dtype, out_dtype)
    expect, expect_res = ew.reference_residual_rms(_carrier(x), _carrier(res), _carrier(weight), 1e-5,
                                                   None if scale is None else 0.0123, dtype, kind, form="kernel")
    assert np.array_equal(_carrier(new_res).view(np.uint16), np.asarray(expect_res).view(np.uint16))
    if out_dtype is None:
        distance = ew.ulp16_distance(_carrier(out), expect, dtype)
        assert distance.max() <= MAX_16BIT_STEPS
        assert (distance != 0).sum() <= max(1, MAX_FRACTION_OFF_BY_ONE * distance.size)
    else:
        _assert_bytes_close(ew, out, expect, (rows, cols, in_dtype, out_dtype))
    if out_dtype is None:
        assert bool((next_buffer == 2.0).all())          # 16-bit output: the buffer is not touched
    else:
        assert int(torch.count_nonzero(next_buffer)) == 0


def test_residual_rms_unaligned_views_stay_in_bounds(oracle_mod, ew, capi, dev):
    rows, cols = 3, 72
    torch.manual_seed(8)
    x = torch.randn(rows * cols + 1, device=dev).to(torch.float16)[1:].view(rows, cols)
    res_backing = torch.randn(rows * cols + 2, device=dev).to(torch.float16)
    before = res_backing.clone()
    res = res_backing[1:1 + rows * cols].view(rows, cols)
    weight = torch.randn(cols, device=dev).to(torch.float16)
    out_backing = torch.full((rows * cols + 10,), 0x55, dtype=torch.uint8, device=dev)
    out = out_backing[5:5 + rows * cols].view(rows, cols).view(torch.float8_e4m3fn)
    scale = torch.tensor([0.02], device=dev)
    capi.check(capi.residual_rms(x, res, weight, scale, 1e-5, out, None))
    _device_ok(capi)
    expect, expect_res = ew.reference_residual_rms(_carrier(x), _carrier(before[1:1 + rows * cols].view(rows, cols)),
                                                   _carrier(weight), 1e-5, 0.02, oracle_mod.F16, oracle_mod.E4M3FN)
    _assert_bytes_close(ew, out, expect, "unaligned")
    assert np.array_equal(_carrier(res).view(np.uint16), expect_res.view(np.uint16))
    guard = out_backing.cpu().numpy()
    assert (guard[:5] == 0x55).all() and (guard[-5:] == 0x55).all()
    assert torch.equal(res_backing[:1], before[:1]) and torch.equal(res_backing[-1:], before[-1:])


def test_residual_rms_empty_and_invalid_inputs(capi, dev):
    lib = capi.lib
    x = torch.zeros((2, 64), dtype=torch.float16, device=dev)
    w = torch.ones(64, dtype=torch.float16, device=dev)
    out = torch.empty((2, 64), dtype=torch.float16, device=dev)
    args = (x.data_ptr(), x.data_ptr(), w.data_ptr(), 0)
    assert lib.hfrk_residual_rms(*args, 1e-5, out.data_ptr(), 0, 0, 64, 0, capi.F16, capi.OUT_SAME, 0, 0, 0) == 0
    assert lib.hfrk_residual_rms(*args, 0.0, out.data_ptr(), 0, 2, 64, 0, capi.F16, capi.OUT_SAME, 0, 0, 0) == 6
    assert lib.hfrk_residual_rms(*args, 1e-5, out.data_ptr(), 0, 2, 0, 0, capi.F16, capi.OUT_SAME, 0, 0, 0) == 6
    assert lib.hfrk_residual_rms(*args, 1e-5, out.data_ptr(), 0, 2, 64, 0, capi.F32, capi.OUT_SAME, 0, 0, 0) == 8
    assert lib.hfrk_residual_rms(*args, 1e-5, out.data_ptr(), 0, 2, 64, 0, capi.F16, 7, 0, 0, 0) == 8
    # an fp8 output without a scale
    assert lib.hfrk_residual_rms(*args, 1e-5, out.data_ptr(), 0, 2, 64, 0, capi.F16, capi.OUT_E4M3FN, 0, 0, 0) == 6
    with pytest.raises(RuntimeError):
        torch.ops._HFRK_C.residual_rms(x, x.clone(), w, None, 1e-5,
                                       torch.empty((2, 64), dtype=torch.float8_e4m3fn, device=dev),
                                       torch.empty((2, 0), dtype=torch.float16, device=dev), 0, False)


def test_increment_adds_one_in_place(native_build, dev):
    """The reference's tests/test_increment.py:8-12."""
    from hf_rocm_kernels import increment

    x = torch.rand(size=(128,), device=dev)
    y = x.clone()
    increment(x)
    assert x.eq(y + 1).all()
    with pytest.raises(AssertionError):
        increment(torch.zeros(4))


# ------------------------------------------------------- gate/up GEMM with swiglu in its epilogue
@pytest.mark.parametrize("act_dtype,fp8_dtype", [(torch.float16, torch.float8_e4m3fnuz),
                                                 (torch.bfloat16, torch.float8_e4m3fn)])
@pytest.mark.parametrize("m,inter,k", [(16, 14336, 4096), (1, 14336, 4096), (5, 1040, 256), (16, 64, 128),
                                       (3, 4144, 512), (9, 28672, 8192), (16, 16, 2048),
                                       # K split over a cluster: 5, 5, 8 and 12 CTAs per tile; owners with
                                       # four, one, one-or-none and two-one-or-none token rows
                                       (16, 3584, 8192), (1, 3584, 8192), (7, 2048, 4096), (13, 1024, 8192)])
def test_fused_gemm_swiglu_writes_the_bytes_of_the_two_launches(capi, dev, m, inter, k, act_dtype, fp8_dtype):
    """One launch (GEMM with the activation in its epilogue) against GEMM into a 16-bit buffer
    followed by the swiglu kernel: identical bytes, zeroed buffer, nothing written out of bounds."""
    from hf_rocm_kernels import skinny_gemm, swiglu
    from hf_rocm_kernels.combined_ops import skinny_gemm_swiglu

    torch.manual_seed(m * 7 + inter)
    a = (torch.randn(m, k, device=dev) * 40).clamp(-200, 200).to(torch.float8_e4m3fn).view(torch.uint8)
    w = (torch.randn(2 * inter, k, device=dev) * 40).clamp(-200, 200).to(torch.float8_e4m3fn).view(torch.uint8)
    if fp8_dtype == torch.float8_e4m3fnuz:       # 0x80 is NaN there
        a = torch.where(a == 0x80, torch.zeros_like(a), a)
        w = torch.where(w == 0x80, torch.zeros_like(w), w)
    a, w = a.view(fp8_dtype), w.view(fp8_dtype)
    scale = torch.tensor([2.5 / (40.0 * 40.0 * k ** 0.5)], device=dev)
    act_scale = torch.tensor([0.021], device=dev)

    gate_up = torch.zeros((m, 2 * inter), dtype=act_dtype, device=dev)
    skinny_gemm(a, w.t(), scale, gate_up)
    buf_two = torch.full((m, 264), 3.0, dtype=act_dtype, device=dev)
    expect = swiglu(gate_up, act_scale, buf_two, out_dtype=fp8_dtype)

    buf_one = torch.full((m, 264), 3.0, dtype=act_dtype, device=dev)
    got = skinny_gemm_swiglu(a, w.t(), scale, act_scale, buf_one, mid_dtype=act_dtype, out_dtype=fp8_dtype)
    _device_ok(capi)
    assert got.dtype == fp8_dtype and tuple(got.shape) == (m, inter)
    assert torch.equal(got.view(torch.uint8), expect.view(torch.uint8))
    assert int(torch.count_nonzero(buf_one)) == 0
    spread = expect.view(torch.uint8).unique().numel()
    assert spread > 8 or inter * m < 64, "degenerate test data"

    # guard bytes either side of the output
    backing = torch.full((m * inter + 64,), 0x55, dtype=torch.uint8, device=dev)
    out = backing[32:32 + m * inter].view(m, inter).view(fp8_dtype)
    capi.check(capi.skinny_gemm_swiglu(a, w, out, scale, act_scale, None, act_dtype))
    _device_ok(capi)
    assert torch.equal(out.view(torch.uint8), expect.view(torch.uint8))
    guard = backing.cpu().numpy()
    assert (guard[:32] == 0x55).all() and (guard[-32:] == 0x55).all()


def test_fused_gemm_swiglu_rejects_what_it_cannot_do(capi, dev):
    a = torch.zeros((17, 256), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    w = torch.zeros((256, 256), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    out = torch.empty((17, 128), dtype=torch.float8_e4m3fn, device=dev)
    s = torch.ones(1, device=dev)
    assert capi.skinny_gemm_swiglu(a, w, out, s, s) == 12                       # more than 16 tokens
    w2 = torch.zeros((2 * 24, 256), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    assert capi.skinny_gemm_swiglu(a[:4], w2, out.flatten()[:4 * 24].view(4, 24), s, s) == 6   # inter % 16
    assert capi.skinny_gemm_swiglu(a[:4], w, out[:4], s, s, mid_dtype=torch.float32) == 8


# ------------------------------------------------------------------------------------ the MLP chain
def _mlp_inputs(dev, tokens, hidden, inter, act_dtype, fp8_dtype):
    from hf_rocm_kernels.utils.fp8 import fp8_quantize, fp8_quantize_e4m3fn

    torch.manual_seed(21)
    attn = torch.randn(tokens, hidden, device=dev).to(act_dtype)
    residual = torch.randn(tokens, hidden, device=dev).to(act_dtype)
    rms_w = (1 + 0.1 * torch.randn(hidden, device=dev)).to(act_dtype)
    w_gu = torch.randn(2 * inter, hidden, device=dev) * 0.02
    w_dn = torch.randn(hidden, inter, device=dev) * 0.02
    if fp8_dtype == torch.float8_e4m3fnuz:
        s_gu, s_dn = [(w.abs().amax().float() / 448).reshape(1) for w in (w_gu, w_dn)]
        q_gu, s_gu2 = fp8_quantize(w_gu, s_gu)
        q_dn, s_dn2 = fp8_quantize(w_dn, s_dn)
    else:
        q_gu, s_gu2 = fp8_quantize_e4m3fn(w_gu)
        q_dn, s_dn2 = fp8_quantize_e4m3fn(w_dn)
    in_scale_gu = torch.tensor([4.0 / 448 * (2 if fp8_dtype == torch.float8_e4m3fnuz else 1)], device=dev)
    in_scale_dn = torch.tensor([16.0 / 448 * (2 if fp8_dtype == torch.float8_e4m3fnuz else 1)], device=dev)
    return dict(attn=attn, residual=residual, rms_w=rms_w, q_gu=q_gu, q_dn=q_dn,
                in_scale_gu=in_scale_gu, out_scale_gu=(in_scale_gu * s_gu2), in_scale_dn=in_scale_dn,
                out_scale_dn=(in_scale_dn * s_dn2), w_gu=w_gu, w_dn=w_dn)


@pytest.mark.parametrize("act_dtype,fp8_dtype", [(torch.float16, torch.float8_e4m3fnuz),
                                                 (torch.bfloat16, torch.float8_e4m3fn)])
@pytest.mark.parametrize("tokens", [1, 16])
def test_llama_mlp_chain_equals_its_parts_and_tracks_the_unquantised_block(capi, dev, tokens, act_dtype, fp8_dtype):
    """The four-launch chain must equal the same four operators run one by one with a
    synchronisation in between (programmatic dependent launch must not change a bit), replay
    identically from a CUDA graph, and stay close to the block computed without quantisation."""
    from hf_rocm_kernels import residual_rms, skinny_gemm, swiglu
    from hf_rocm_kernels.combined_ops import llama_mlp_combined_ops

    hidden, inter = 4096, 14336
    p = _mlp_inputs(dev, tokens, hidden, inter, act_dtype, fp8_dtype)

    def chain(residual):
        return llama_mlp_combined_ops(p["attn"], residual, p["rms_w"], 1e-5, p["q_gu"].t(), p["in_scale_gu"],
                                      p["out_scale_gu"], p["q_dn"].t(), p["in_scale_dn"], p["out_scale_dn"])

    out, new_res = chain(p["residual"].clone())
    _device_ok(capi)
    from hf_rocm_kernels.combined_ops import can_fuse_swiglu

    assert can_fuse_swiglu(tokens, hidden, inter)          # so `chain` ran the three-launch form
    assert not can_fuse_swiglu(17, hidden, inter) and not can_fuse_swiglu(4, hidden, 1000)
    for fuse in (False, True):
        out_f, res_f = llama_mlp_combined_ops(p["attn"], p["residual"].clone(), p["rms_w"], 1e-5, p["q_gu"].t(),
                                              p["in_scale_gu"], p["out_scale_gu"], p["q_dn"].t(), p["in_scale_dn"],
                                              p["out_scale_dn"], fuse_swiglu=fuse)
        assert torch.equal(out_f, out) and torch.equal(res_f, new_res)

    # step by step
    res2 = p["residual"].clone()
    gate_up = torch.full((tokens, 2 * inter), 5.0, dtype=act_dtype, device=dev)
    normed, _ = residual_rms(p["attn"], res2, p["rms_w"], 1e-5, p["in_scale_gu"], gate_up, out_dtype=fp8_dtype)
    torch.cuda.synchronize()
    skinny_gemm(normed, p["q_gu"].t(), p["out_scale_gu"], gate_up)
    torch.cuda.synchronize()
    mlp = torch.full((tokens, hidden), 5.0, dtype=act_dtype, device=dev)
    act = swiglu(gate_up, p["in_scale_dn"], mlp, out_dtype=fp8_dtype)
    torch.cuda.synchronize()
    skinny_gemm(act, p["q_dn"].t(), p["out_scale_dn"], mlp)
    torch.cuda.synchronize()
    assert torch.equal(out, mlp) and torch.equal(new_res, res2)

    # graph replay
    static_res = p["residual"].clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        chain(static_res.clone())            # warm-up outside capture
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            g_out, g_res = chain(static_res)
    for _ in range(3):
        static_res.copy_(p["residual"])
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(g_out, out) and torch.equal(g_res, new_res)
    _device_ok(capi)

    # the unquantised block in float32
    summed = (p["attn"] + p["residual"]).float()
    normal = summed * torch.rsqrt(summed.pow(2).mean(-1, keepdim=True) + 1e-5) * p["rms_w"].float()
    gu = normal @ p["w_gu"].t()
    expect = (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]) @ p["w_dn"].t()
    error = (out.float() - expect).norm() / expect.norm()
    assert float(error) < 0.15, float(error)      # fp8 on both operands of both GEMMs: ~5 % each
