"""CPU oracle for the two element-wise operators of the decode path -- TEST INFRASTRUCTURE ONLY.

Only the test-suite and the smoke check import this module; the shipped package never does.

It restates, in numpy, what the reference (huggingface/hf-rocm-kernels) defines for

* swiglu        -- ``hf_rocm_kernels/operators/swiglu/reference.py:7-27``: silu(gate) * up in
  float32, then ``fp8_quantize`` (``utils/fp8.py:17-33``); the kernel does the same arithmetic
  (``csrc/op_src/swiglu/swiglu_scalar.cu:52-60``).
* residual_rms  -- two forms. ``form="torch"`` follows
  ``hf_rocm_kernels/operators/residual_rms/reference.py:7-37`` (sum in 16 bits, norm in float32,
  rounded to 16 bits, 16-bit product with the weight, then ``fp8_quantize``). ``form="kernel"``
  follows the vectorised kernel ``csrc/op_src/residual_rms/residual_rms_vectorized.cu:96-146``:
  the same for a 16-bit output, but for an fp8 output ``float(sum) * float(weight) *
  (normaliser / scale)`` with one rounding, to fp8. ``precise_residual_rms`` follows
  ``reference.py:40-66``.

16-bit values travel as numpy ``float16`` arrays or, for bfloat16, as ``uint16`` bit patterns
(``dtype=BF16``). fp8 results are returned as bytes.

Parity pin: ``tests/golden/elementwise.npz`` holds outputs of the reference's own
``reference_swiglu``, ``reference_residual_rms`` and ``precise_residual_rms`` executed on CPU
(``tests/golden/make_golden_elementwise.py``); ``tests/test_oracle_elementwise.py`` checks this
module against them. The mean of squares is accumulated in float64 here and in float32, in another
order, by torch and by the kernel, so the normaliser can differ in its last bit and a small
fraction of outputs by one step of the output format; the tests bound both.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np

from oracle import BF16, E4M3FN, E4M3FNUZ, F16, bf16_bits_to_f32, quantize_e4m3fn, to_bf16_bits


# ----------------------------------------------------------------------------- 16-bit helpers
def to_f32(x16: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == BF16:
        return bf16_bits_to_f32(x16)
    return np.asarray(x16, dtype=np.float16).astype(np.float32)


def round16(x32: np.ndarray, dtype: int) -> np.ndarray:
    """float32 -> the 16-bit carrier (float16 array, or uint16 bits for bfloat16), nearest even."""
    if dtype == BF16:
        return to_bf16_bits(x32)
    with np.errstate(over="ignore"):
        return np.asarray(x32, dtype=np.float32).astype(np.float16)


def add16(a16: np.ndarray, b16: np.ndarray, dtype: int) -> np.ndarray:
    """Correctly rounded 16-bit sum (the float32 sum of two 16-bit values rounds the same way)."""
    return round16(to_f32(a16, dtype) + to_f32(b16, dtype), dtype)


def mul16(a16: np.ndarray, b16: np.ndarray, dtype: int) -> np.ndarray:
    """Correctly rounded 16-bit product (the float32 product of two 16-bit values is exact)."""
    return round16(to_f32(a16, dtype) * to_f32(b16, dtype), dtype)


def fp8_bytes(x32: np.ndarray, scale: float, kind: int) -> np.ndarray:
    """``x / scale`` as fp8 bytes. E4M3FNUZ: the bytes the reference emits when it is handed
    ``scale`` as the doubled scale of ``utils/fp8.py:31-33`` (e4m3fn bytes of ``x / (scale / 2)``
    with 0x80 cleared); E4M3FN: plain e4m3fn bytes of ``x / scale``."""
    if kind == E4M3FNUZ:
        return quantize_e4m3fn(x32, np.float32(scale) / np.float32(2.0), zero_negative_zero=True)
    return quantize_e4m3fn(x32, np.float32(scale), zero_negative_zero=False)


# ----------------------------------------------------------------------------- swiglu
def silu_mul(gate_up16: np.ndarray, dtype: int = F16) -> np.ndarray:
    """silu(gate) * up in float32 steps; gate is the left half of the columns, up the right."""
    x = to_f32(gate_up16, dtype)
    hidden = x.shape[1] // 2
    gate, up = x[:, :hidden], x[:, hidden:]
    with np.errstate(over="ignore"):
        e = np.exp(-gate.astype(np.float64)).astype(np.float32)   # correctly rounded float32 exp
    denom = (np.float32(1.0) + e).astype(np.float32)
    silu = (gate / denom).astype(np.float32)
    return (silu * up).astype(np.float32)


def reference_swiglu(gate_up16: np.ndarray, scale: float, dtype: int = F16, kind: int = E4M3FNUZ) -> np.ndarray:
    """Bytes of ``fp8(silu(gate) * up / scale)``; see :func:`fp8_bytes` for what ``scale`` means per kind."""
    return fp8_bytes(silu_mul(gate_up16, dtype), scale, kind)


# ----------------------------------------------------------------------------- residual + RMS norm
def _normaliser(sum16: np.ndarray, epsilon: float, dtype: int) -> Tuple[np.ndarray, np.ndarray]:
    x = to_f32(sum16, dtype)
    variance = (np.sum(x.astype(np.float64) ** 2, axis=-1, keepdims=True) / x.shape[-1]).astype(np.float32)
    normaliser = (np.float32(1.0) / np.sqrt(variance + np.float32(epsilon), dtype=np.float32)).astype(np.float32)
    return x, normaliser


def reference_residual_rms(input16: np.ndarray, residual16: np.ndarray, weight16: np.ndarray, epsilon: float,
                           scale: Optional[float] = None, dtype: int = F16, kind: int = E4M3FNUZ,
                           form: str = "kernel") -> Tuple[np.ndarray, np.ndarray]:
    """Returns ``(output, new residual)``: the residual in the 16-bit carrier; the output in the
    16-bit carrier when ``scale`` is None, else fp8 bytes (``scale`` as in :func:`fp8_bytes`)."""
    assert form in ("kernel", "torch")
    sum16 = add16(residual16, input16, dtype)
    x, normaliser = _normaliser(sum16, epsilon, dtype)
    if scale is None or form == "torch":
        y16 = mul16(round16((x * normaliser).astype(np.float32), dtype), np.broadcast_to(weight16, sum16.shape), dtype)
        if scale is None:
            return y16, sum16
        return fp8_bytes(to_f32(y16, dtype), scale, kind), sum16
    factor = (normaliser / np.float32(scale)).astype(np.float32)
    if kind == E4M3FNUZ:
        factor = (factor * np.float32(2.0)).astype(np.float32)
    v = ((x * to_f32(weight16, dtype)).astype(np.float32) * factor).astype(np.float32)
    # v is already divided by the scale: encode it as it stands.
    return quantize_e4m3fn(v, np.float32(1.0), zero_negative_zero=(kind == E4M3FNUZ)), sum16


def precise_residual_rms(input16: np.ndarray, residual16: np.ndarray, weight16: np.ndarray, epsilon: float,
                         scale: Optional[float] = None, dtype: int = F16, kind: int = E4M3FNUZ) -> np.ndarray:
    """The reference's high-precision form: float64 sum (not rounded to 16 bits) and product with
    the weight, float32 norm. float64 values when ``scale`` is None, else fp8 bytes."""
    summed = to_f32(input16, dtype).astype(np.float64) + to_f32(residual16, dtype).astype(np.float64)
    x32 = summed.astype(np.float32)
    variance = (np.sum(x32.astype(np.float64) ** 2, axis=-1, keepdims=True) / x32.shape[-1]).astype(np.float32)
    normalised = (x32 * (np.float32(1.0) / np.sqrt(variance + np.float32(epsilon), dtype=np.float32))).astype(np.float32)
    y = to_f32(weight16, dtype).astype(np.float64) * normalised.astype(np.float64)
    if scale is None:
        return y
    inv = np.float32(1.0) / (np.float32(scale) / np.float32(2.0) if kind == E4M3FNUZ else np.float32(scale))
    return quantize_f64_e4m3fn(y * np.float64(inv), zero_negative_zero=(kind == E4M3FNUZ))


def quantize_f64_e4m3fn(v: np.ndarray, zero_negative_zero: bool) -> np.ndarray:
    """float64 values -> e4m3fn bytes, clamp to +-448, one rounding to nearest even (what a cast of
    a float64 tensor to ``float8_e4m3fn`` does)."""
    v = np.clip(np.asarray(v, dtype=np.float64), -448.0, 448.0)
    sign = np.signbit(v)
    a = np.abs(v)
    _, e = np.frexp(a)
    ue = np.maximum(e.astype(np.int64) - 1, -6)
    ue = np.where(a == 0, -6, ue)
    steps = np.rint(a / np.ldexp(1.0, ue - 3))
    carry = steps >= 16
    steps = np.where(carry, 8.0, steps)
    ue = np.where(carry, ue + 1, ue)
    steps_i = steps.astype(np.int64)
    bits = np.where(steps_i < 8, steps_i, ((ue + 7) << 3) | (steps_i - 8)).astype(np.uint8)
    bits = bits | np.where(sign, 0x80, 0).astype(np.uint8)
    if zero_negative_zero:
        bits = np.where(bits == 0x80, 0, bits).astype(np.uint8)
    return bits


# ----------------------------------------------------------------------------- comparison
def fp8_step_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """How many codes apart two e4m3 byte arrays are on the number line (sign-magnitude order)."""
    def order(q):
        q = np.asarray(q, dtype=np.uint8).astype(np.int32)
        return np.where(q & 0x80, -(q & 0x7F), q & 0x7F)
    return np.abs(order(a) - order(b))


def ulp16_distance(a16: np.ndarray, b16: np.ndarray, dtype: int) -> np.ndarray:
    """How many representable values apart two 16-bit arrays are."""
    def order(x):
        bits = (np.asarray(x, dtype=np.float16).view(np.uint16) if dtype != BF16 else np.asarray(x, np.uint16))
        bits = bits.astype(np.int32)
        return np.where(bits & 0x8000, -(bits & 0x7FFF), bits & 0x7FFF)
    return np.abs(order(a16) - order(b16))
