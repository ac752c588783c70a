"""Error metrics for comparing an operator's output with a reference.

Same entry points and return values as the reference's ``hf_rocm_kernels/utils/testing.py``
(``compare_x_with_ref`` :5-51, ``compare_x_and_ref_to_precise`` :54-80), plus the tolerance this
library is held to for the skinny GEMM.
"""
import math
from typing import Optional, Tuple

import torch
from torch import Tensor


def _same_shape(a: Tensor, b: Tensor, what: str) -> None:
    if a.shape != b.shape:
        raise ValueError(f"Cannot compare tensor of shape {tuple(a.shape)} with {what} of shape {tuple(b.shape)}.")


def compare_x_with_ref(x: Tensor, ref: Tensor, name: Optional[str] = None) -> Tuple[float, float, float]:
    """Returns (max |ref - x|, max |ref - x| / ref over non-zero ref, number of differing elements).

    With a ``name`` it also prints a short report (heads and tails of both tensors, the three
    metrics, the mean error and NaN counts).
    """
    _same_shape(x, ref, "reference")
    x32, ref32 = x.float(), ref.float()
    delta = (ref32 - x32).abs()
    max_abs = delta.max().item()
    nonzero = ref32 != 0
    max_rel = (delta[nonzero] / ref32[nonzero]).max().item() if bool(nonzero.any()) else float("inf")
    changed = int((delta != 0).sum().item())
    if name is not None:
        if max_abs == 0:
            print(f"All good for {name}")
        else:
            flat_x, flat_ref = x32.flatten().tolist(), ref32.flatten().tolist()
            print(f"Not good for {name}")
            print("  reference:", flat_ref[:4], "...", flat_ref[-4:])
            print("  computed: ", flat_x[:4], "...", flat_x[-4:])
            print(f"  max abs diff {max_abs}, max rel diff {max_rel}, mean abs diff {delta.mean().item()}")
            print(f"  {changed} of {delta.numel()} elements differ ({100.0 * changed / delta.numel():.5f} %)")
            print(f"  NaNs: reference {int(ref32.isnan().sum())}, computed {int(x32.isnan().sum())}")
    return max_abs, max_rel, changed


def compare_x_and_ref_to_precise(x: Tensor, ref: Tensor, precise: Tensor) -> Tuple[float, ...]:
    """Errors of ``x`` and of ``ref`` against a higher-precision result.

    Returns (max err x, max err ref, mean err x, mean err ref, % of elements where x is worse than
    ref, max and mean of x's error over those elements).
    """
    _same_shape(x, ref, "reference")
    _same_shape(x, precise, "precise")
    err_x = (precise.float() - x.float()).abs()
    err_ref = (precise.float() - ref.float()).abs()
    worse = err_x > err_ref
    masked = err_x * worse
    return (
        err_x.max().item(), err_ref.max().item(),
        err_x.mean().item(), err_ref.mean().item(),
        worse.float().mean().item() * 100.0, masked.max().item(), masked.mean().item(),
    )


def skinny_gemm_tolerance(ref32: Tensor, k: int, scale: float, out_dtype: torch.dtype) -> Tensor:
    """Per-element bound: one ulp of ``out_dtype`` at ``|ref32|`` plus ``1e-3 * sqrt(k) * |scale|``."""
    frac_bits, min_exp = (7, -126) if out_dtype == torch.bfloat16 else (10, -14)
    mag = ref32.double().abs()
    exponent = torch.floor(torch.log2(torch.where(mag > 0, mag, torch.ones_like(mag)))).clamp(min=min_exp)
    exponent = torch.where(mag > 0, exponent, torch.full_like(exponent, min_exp))
    return torch.pow(2.0, exponent - frac_bits) + 1e-3 * math.sqrt(k) * abs(scale)
