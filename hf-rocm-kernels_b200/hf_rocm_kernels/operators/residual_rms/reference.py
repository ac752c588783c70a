"""Torch statements of the residual_rms operator (working precision and fp64) and its input
generator, with the names and argument order of the reference's
``hf_rocm_kernels/operators/residual_rms/reference.py`` (``reference_residual_rms`` :7-37,
``precise_residual_rms`` :40-66, ``reference_rms`` :69-72, ``generate_residual_rms_data`` :75-92)."""
from typing import Optional, Tuple

import torch
from torch import Tensor

from hf_rocm_kernels.utils.fp8 import fp8_quantize


def reference_rms(x: Tensor, eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension, in fp32 whatever the dtype of ``x``."""
    x = x.to(torch.float32)
    variance = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(variance + eps)


def _finish(normalised: Tensor, scale_tensor: Optional[Tensor], next_buffer: Optional[Tensor]):
    if scale_tensor is None:
        return normalised, None
    quantised, doubled_scale = fp8_quantize(normalised, scale_tensor)
    if next_buffer is not None:
        next_buffer.fill_(0)
    return quantised, doubled_scale


def reference_residual_rms(
    input: Tensor,
    residual: Tensor,
    weight: Tensor,
    epsilon: float,
    scale_tensor: Optional[Tensor],
    next_buffer: Optional[Tensor] = None,
) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
    """The operator as a model would write it: the sum in 16 bits (``input`` is overwritten by it),
    the norm in fp32, the product with the weight in the weight's dtype, then ``fp8_quantize``.
    Returns ``(output, residual, doubled scale or None)``."""
    assert input.dtype in (torch.float16, torch.bfloat16), f"Expected a 16-bit input but got {input.dtype = }"
    assert residual.dtype == input.dtype, f"Expected {input.dtype} but got {residual.dtype = }"
    input += residual
    residual = input
    normalised = reference_rms(input, epsilon)
    if weight.dtype in (torch.float16, torch.bfloat16):
        normalised = normalised.to(weight.dtype)
    normalised = weight * normalised
    output, doubled_scale = _finish(normalised, scale_tensor, next_buffer)
    return output, residual, doubled_scale


def precise_residual_rms(
    input: Tensor,
    residual: Tensor,
    weight: Tensor,
    epsilon: float,
    scale_tensor: Optional[Tensor],
    next_buffer: Optional[Tensor] = None,
) -> Tuple[Tensor, Tensor]:
    """The yardstick both the kernel and ``reference_residual_rms`` are measured against: the sum
    and the product with the weight in fp64 (so the sum is not rounded to 16 bits), the norm itself
    in fp32 as ``reference_rms`` computes it. Returns ``(output, residual)``."""
    summed = input.to(torch.float64) + residual.to(torch.float64)
    normalised = weight.to(torch.float64) * reference_rms(summed, epsilon)
    output, _ = _finish(normalised, scale_tensor, next_buffer)
    return output, summed


def generate_residual_rms_data(
    rows: int, cols: int, buffer_cols: int = 0, dtype: torch.dtype = torch.float16, seed: Optional[int] = None,
    device: str = "cuda", input_dtype: torch.dtype = torch.float16,
) -> Tuple[Tensor, Tensor, Tensor, float, Optional[Tensor], Optional[Tensor]]:
    """N(0, 1) input, residual and weight, an epsilon in [1e-5, 2e-5) and, when ``dtype`` is an fp8
    type, a scale in [1, 3) (``None`` otherwise); a (rows, buffer_cols) buffer when asked for.
    Returns ``(input, residual, weight, epsilon, scale_tensor, next_buffer)``."""
    if seed is not None:
        torch.manual_seed(seed)
    input = torch.normal(0, 1, size=(rows, cols), device=device, dtype=input_dtype)
    residual = torch.normal(0, 1, size=(rows, cols), device=device, dtype=input_dtype)
    weights = torch.normal(0, 1, size=(cols, ), device=device, dtype=input_dtype)
    epsilon = torch.rand(size=(1,)).add(1).mul(1e-5).item()
    if dtype in (torch.float8_e4m3fnuz, torch.float8_e4m3fn):
        scale_tensor = torch.rand(size=(1,), device=device, dtype=torch.float32).mul(2).add(1)
    else:
        scale_tensor = None
    next_buffer = None if buffer_cols == 0 else torch.empty((rows, buffer_cols), device=device, dtype=input_dtype)
    return input, residual, weights, epsilon, scale_tensor, next_buffer
