"""Keyword bridge to the registered torch op, as in the reference's
``hf_rocm_kernels/operators/residual_rms/binding.py:7-21``: same function name and argument names."""
from typing import Optional

import torch
from torch import Tensor

import hf_rocm_kernels._HFRK_C  # noqa: F401  (loads the extension that registers torch.ops._HFRK_C)


def _residual_rms(
    input: Tensor,
    residual: Tensor,
    weight: Tensor,
    scale_tensor: Optional[Tensor],
    epsilon: float,
    output: Tensor,
    next_buffer: Tensor,
    num_threads: int,
    force_scalar: bool,
) -> None:
    """``residual += input``; ``output`` <- RMS-normalised ``residual`` times ``weight`` (divided by
    the scale and rounded to fp8 when ``output`` is an fp8 tensor); ``next_buffer`` <- 0. A ``None``
    scale reaches the op as an undefined tensor, which it accepts for a 16-bit output."""
    torch.ops._HFRK_C.residual_rms(
        input, residual, weight, scale_tensor, epsilon, output, next_buffer, num_threads, force_scalar
    )
