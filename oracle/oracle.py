"""CPU oracle for the FP8 skinny GEMM -- TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA path. Only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark import it; the shipped package never does.

It restates the arithmetic that the reference (huggingface/hf-rocm-kernels) defines for the path:

* quantisation     -- ``hf_rocm_kernels/utils/fp8.py:17-29``: ``clamp(x * (1/scale), +-448)`` cast
  to e4m3fn with round-to-nearest-even, byte ``0x80`` rewritten to ``0x00``; the same byte read as
  e4m3fnuz is worth exactly half.
* expected result  -- ``hf_rocm_kernels/operators/skinny_gemm/reference.py:18-25``:
  ``out = cast(scale_a * scale_b * (A @ B))``.
* in-place contract -- ``hf_rocm_kernels/operators/skinny_gemm/wrapped.py:115``:
  ``D <- D_in + scale * (A @ W.T)`` with ``D_in`` zeros or the broadcast bias.

Parity pin: the reference has no golden vectors for this path (``tests/test_skinny_gemm.py:21-36``
is a differential test against ``torch._scaled_mm`` on an AMD GPU). The quantiser is pinned
bit-for-bit to outputs of the reference's own ``fp8.py`` executed on CPU, and the GEMM to
``torch._scaled_mm`` -- the function the reference calls -- executed on CPU on the same bytes; the
vectors are in ``tests/golden/``.

Everything is numpy; a C twin (``skinny_gemm_oracle.c``) is loaded through ctypes by
:func:`load_c_oracle`. The two agree bit-for-bit on the quantiser and on the GEMM without
``d_in``; with ``d_in`` the numpy form rounds the final multiply-add twice where C's ``fmaf``
rounds once, so they may differ by one float32 ulp.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from typing import Optional

import numpy as np

E4M3FN = 0
E4M3FNUZ = 1
F16 = 0
BF16 = 1

_HERE = os.path.dirname(os.path.abspath(__file__))


# ----------------------------------------------------------------------------- fp8 decode
def fp8_table(kind: int = E4M3FN) -> np.ndarray:
    """float32 value of each of the 256 bit patterns (NaN where the format has one).

    e4m3fn: bias 7, 0x7f/0xff are NaN, no infinities, max 448.
    e4m3fnuz: bias 8, 0x80 is NaN, no negative zero, max 240.
    """
    bias = 8 if kind == E4M3FNUZ else 7
    out = np.empty(256, dtype=np.float32)
    for bits in range(256):
        sign = -1.0 if bits & 0x80 else 1.0
        exp = (bits >> 3) & 0xF
        man = bits & 0x7
        if kind == E4M3FNUZ and bits == 0x80:
            out[bits] = np.nan
        elif kind == E4M3FN and exp == 15 and man == 7:
            out[bits] = np.nan
        elif exp == 0:
            out[bits] = sign * math.ldexp(man, 1 - bias - 3)
        else:
            out[bits] = sign * math.ldexp(8 + man, exp - bias - 3)
    return out


def dequantize(q: np.ndarray, kind: int = E4M3FN) -> np.ndarray:
    """uint8 bit patterns -> float32 values."""
    return fp8_table(kind)[np.asarray(q, dtype=np.uint8)]


# ----------------------------------------------------------------------------- fp8 encode
def quantize_e4m3fn(x: np.ndarray, scale: float, zero_negative_zero: bool = False) -> np.ndarray:
    """Bytes of ``clamp(x * (1/scale), -448, 448)`` rounded to nearest-even e4m3fn.

    Follows ``hf_rocm_kernels/utils/fp8.py:17-25``; ``zero_negative_zero`` is the reference's
    ``0x80 -> 0x00`` step (needed when the bytes will be read as e4m3fnuz).
    """
    x = np.asarray(x, dtype=np.float32)
    inv = np.float32(1.0) / np.float32(scale)
    v = np.clip(x * inv, np.float32(-448.0), np.float32(448.0)).astype(np.float32)
    sign = np.signbit(v)
    a = np.abs(v)
    _, e = np.frexp(a)                      # a = f * 2**e with f in [0.5, 1)
    ue = np.maximum(e.astype(np.int32) - 1, -6)
    ue = np.where(a == 0, -6, ue)
    quantum = np.ldexp(np.float32(1.0), ue - 3).astype(np.float32)
    steps = np.rint(a / quantum)            # exact division by a power of two; rint = half-to-even
    carry = steps >= 16
    steps = np.where(carry, 8.0, steps)
    ue = np.where(carry, ue + 1, ue)
    steps_i = steps.astype(np.int32)
    normal = ((ue + 7) << 3) | (steps_i - 8)
    bits = np.where(steps_i < 8, steps_i, normal).astype(np.uint8)
    bits = bits | np.where(sign, 0x80, 0).astype(np.uint8)
    if zero_negative_zero:
        bits = np.where(bits == 0x80, 0, bits).astype(np.uint8)
    return bits


def per_tensor_scale(x: np.ndarray) -> np.float32:
    """amax / 448 in float32: the per-tensor scale of the benchmark configurations."""
    return np.float32(np.max(np.abs(np.asarray(x, dtype=np.float32)))) / np.float32(448.0)


# ----------------------------------------------------------------------------- the GEMM
def kind_factor(a_kind: int, w_kind: int) -> np.float32:
    """0.5 per e4m3fnuz operand: its bytes are evaluated as e4m3fn and the result halved."""
    f = np.float32(1.0)
    if a_kind == E4M3FNUZ:
        f = f * np.float32(0.5)
    if w_kind == E4M3FNUZ:
        f = f * np.float32(0.5)
    return f


def reference_skinny_gemm(a_q: np.ndarray, w_q: np.ndarray, scale: float, d_in: Optional[np.ndarray] = None,
                          a_kind: int = E4M3FN, w_kind: int = E4M3FN, exact: bool = True) -> np.ndarray:
    """float32 ``D_in + scale * (A @ W.T)`` for byte matrices ``a_q [M,K]`` and ``w_q [N,K]``.

    ``exact=True`` sums in float64: products of two e4m3 values are multiples of 2**-18 below
    2**18, and up to 2**15 of them add without rounding in 53 bits, so this is the mathematical
    dot product rounded once to float32. ``exact=False`` is a float32 matmul of the dequantised
    operands (numpy/BLAS summation order). The scale and ``d_in`` are then applied in float32 with
    a single rounding, like the fused multiply-add of the CUDA epilogue.
    """
    a_q = np.asarray(a_q, dtype=np.uint8)
    w_q = np.asarray(w_q, dtype=np.uint8)
    table = fp8_table(E4M3FN)
    eff_scale = np.float32(scale) * kind_factor(a_kind, w_kind)
    if exact:
        dot = (table[a_q].astype(np.float64) @ table[w_q].astype(np.float64).T)
        dot32 = dot.astype(np.float32)
    else:
        dot32 = table[a_q] @ table[w_q].T
    base = np.zeros_like(dot32) if d_in is None else np.asarray(d_in, dtype=np.float32)
    # fused multiply-add in float32 == the float64 expression rounded once (both products and the
    # sum are exact in float64: 24+24 bit product, then one rounding).
    return (dot32.astype(np.float64) * np.float64(eff_scale) + base.astype(np.float64)).astype(np.float32)


# ----------------------------------------------------------------------------- output casts
def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even, NaN kept quiet."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)
    nan = np.isnan(np.asarray(x, dtype=np.float32))
    return np.where(nan, np.uint32(0x7FC0), rounded).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def cast_out(ref32: np.ndarray, d_dtype: int) -> np.ndarray:
    """The oracle's output as float32 values after rounding to the output dtype."""
    if d_dtype == BF16:
        return bf16_bits_to_f32(to_bf16_bits(ref32))
    with np.errstate(over="ignore"):
        return np.asarray(ref32, dtype=np.float32).astype(np.float16).astype(np.float32)


# ----------------------------------------------------------------------------- tolerance
def ulp(ref32: np.ndarray, d_dtype: int = BF16) -> np.ndarray:
    """Spacing of the output format at |ref32| (bf16: 8 significant bits, fp16: 11)."""
    a = np.abs(np.asarray(ref32, dtype=np.float64))
    if d_dtype == BF16:
        min_exp, frac_bits = -126, 7
    else:
        min_exp, frac_bits = -14, 10
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.where(a > 0, np.maximum(e, min_exp), min_exp)
    return np.ldexp(1.0, (e - frac_bits).astype(np.int64))


def tolerance(ref32: np.ndarray, k: int, scale: float, d_dtype: int = BF16) -> np.ndarray:
    """The stated bound, per element: one output ulp of the reference value + 1e-3*sqrt(K)*|scale|."""
    return ulp(ref32, d_dtype) + 1e-3 * math.sqrt(k) * abs(float(scale))


def accumulation_floor(a_q: np.ndarray, w_q: np.ndarray, scale: float, a_kind: int = E4M3FN,
                       w_kind: int = E4M3FN) -> np.ndarray:
    """Rounding noise no fp32 accumulation of these dot products can avoid, per element.

    An fp32 accumulator that absorbs K/32 block results rounds K/32 times at 2**-24 relative to the
    running sum; the running sum of a dot product of signed terms wanders with magnitude
    sqrt(sum_k (a_k w_k)**2), and independent roundings add in quadrature. Two units of that:
        floor = 2**-23 * sqrt(K / 32) * sqrt(sum_k (a_k w_k)**2) * |scale|.
    For K = 4096 it is about a quarter of the absolute term of :func:`tolerance`; from K ~ 14k on
    it exceeds it, which is where any fp32 matmul (a host BLAS included) starts to disagree with the
    exact product on outputs that happen to land within ~1e-3 of zero. It only ever matters there:
    against a typical output it is a relative 1e-6.
    """
    table = fp8_table(E4M3FN).astype(np.float64)
    a2 = table[np.asarray(a_q, dtype=np.uint8)] ** 2
    w2 = table[np.asarray(w_q, dtype=np.uint8)] ** 2
    walk = np.sqrt(a2 @ w2.T)
    k = a_q.shape[1]
    eff = abs(float(np.float32(scale) * kind_factor(a_kind, w_kind)))
    return (2.0 ** -23) * math.sqrt(k / 32.0) * walk * eff


# How many elements of one case may exceed the stated bound itself while staying inside bound + floor.
# Observed over every parity case (126 cases, 0 to 459k outputs each): none in any case of up to 262,144
# outputs at K <= 5120; 1 of 458,752 outputs at K = 4096 (ratio 1.6); 3 of 229,376 at K = 8192 (ratio
# 1.4), 6 of 917,504 at K = 8192 (ratio 2.2); at most 4 per case at K >= 14336 (outputs that cancel to
# within ~1e-6 of zero). The cap is a count per 262,144 outputs (3e-5 of them), not a loose share.
MAX_STRICT_EXCEPTIONS = 8


def strict_exception_cap(k: int, count: int = 0) -> int:
    """Elements of a case of ``count`` outputs that may lie beyond :func:`tolerance` (never beyond
    tolerance + floor): none for short reductions and moderate output counts, otherwise a handful
    per 262,144 outputs (the largest case, 917,504 outputs at K = 8192, showed 6: which elements
    nearly cancel depends on the summation order, that is on the K split the planner picks for the
    chip, so the cap leaves room beside what one chip showed)."""
    if k <= 5120 and count <= 262144:
        return 0
    return MAX_STRICT_EXCEPTIONS * max(1, -(-count // 262144))


def compare(out32: np.ndarray, ref32: np.ndarray, k: int, scale: float, d_dtype: int = BF16,
            floor: Optional[np.ndarray] = None) -> dict:
    """Error of ``out32`` (the kernel's output as float32) against ``ref32``.

    ``violations`` counts elements beyond :func:`tolerance`; ``hard_violations`` those beyond
    tolerance + ``floor`` (see :func:`accumulation_floor`; zero when no floor is given).
    """
    out32 = np.asarray(out32, dtype=np.float64)
    ref = np.asarray(ref32, dtype=np.float64)
    err = np.abs(out32 - ref)
    tol = tolerance(ref32, k, scale, d_dtype)
    ratio = err / tol
    bad = ~(err <= tol)
    hard = bad if floor is None else ~(err <= tol + floor)
    worst = int(np.argmax(np.where(np.isnan(ratio), np.inf, ratio))) if err.size else 0
    return {
        "max_abs_err": float(np.nanmax(err)) if err.size else 0.0,
        "max_err_over_tol": float(np.nanmax(ratio)) if err.size else 0.0,
        "violations": int(bad.sum()),
        "hard_violations": int(hard.sum()),
        "count": int(err.size),
        "worst_index": worst,
        "worst_out": float(out32.flat[worst]) if err.size else 0.0,
        "worst_ref": float(ref.flat[worst]) if err.size else 0.0,
        "nan_out": int(np.isnan(out32).sum()),
    }


# ----------------------------------------------------------------------------- C twin
class COracle:
    """ctypes view of ``libhfrk_oracle.so`` (built from ``skinny_gemm_oracle.c`` by the Makefile)."""

    def __init__(self, path: str):
        lib = ctypes.CDLL(path)
        lib.hfrk_oracle_fp8_to_f32.restype = ctypes.c_float
        lib.hfrk_oracle_fp8_to_f32.argtypes = [ctypes.c_uint8, ctypes.c_int]
        lib.hfrk_oracle_quantize.restype = None
        lib.hfrk_oracle_quantize.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_int,
                                             ctypes.c_void_p]
        lib.hfrk_oracle_skinny_gemm.restype = None
        lib.hfrk_oracle_skinny_gemm.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                                ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64,
                                                ctypes.c_int, ctypes.c_void_p]
        lib.hfrk_oracle_set_num_threads.restype = None
        lib.hfrk_oracle_set_num_threads.argtypes = [ctypes.c_int]
        lib.hfrk_oracle_num_threads.restype = ctypes.c_int
        self.lib = lib

    def set_threads(self, threads: int) -> None:
        self.lib.hfrk_oracle_set_num_threads(int(threads))

    def fp8_to_f32(self, bits: int, kind: int) -> float:
        return float(self.lib.hfrk_oracle_fp8_to_f32(bits, kind))

    def quantize(self, x: np.ndarray, scale: float, zero_negative_zero: bool = False) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.uint8)
        self.lib.hfrk_oracle_quantize(x.ctypes.data, x.size, float(scale), int(zero_negative_zero), out.ctypes.data)
        return out

    def skinny_gemm(self, a_q: np.ndarray, w_q: np.ndarray, scale: float, d_in: Optional[np.ndarray] = None,
                    a_kind: int = E4M3FN, w_kind: int = E4M3FN, exact: bool = True) -> np.ndarray:
        a_q = np.ascontiguousarray(a_q, dtype=np.uint8)
        w_q = np.ascontiguousarray(w_q, dtype=np.uint8)
        m, k = a_q.shape
        n = w_q.shape[0]
        ref = np.empty((m, n), dtype=np.float32)
        d_ptr = None
        if d_in is not None:
            d_in = np.ascontiguousarray(d_in, dtype=np.float32)
            d_ptr = d_in.ctypes.data
        eff = float(np.float32(scale) * kind_factor(a_kind, w_kind))
        self.lib.hfrk_oracle_skinny_gemm(a_q.ctypes.data, w_q.ctypes.data, d_ptr, eff, m, n, k, k, int(exact),
                                         ref.ctypes.data)
        return ref


def c_oracle_path() -> str:
    return os.path.join(_HERE, "libhfrk_oracle.so")


def build_c_oracle(force: bool = False) -> str:
    """Runs the Makefile beside this file (gcc only) and returns the library path."""
    path = c_oracle_path()
    src = os.path.join(_HERE, "skinny_gemm_oracle.c")
    if force or not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libhfrk_oracle.so"], check=True, capture_output=True)
    return path


def load_c_oracle() -> COracle:
    return COracle(build_c_oracle())
