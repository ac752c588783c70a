"""Per-tensor FP8 quantisers used to prepare inputs of the skinny GEMM.

``fp8_quantize`` keeps the name, arguments and return value of the reference's helper
(``hf_rocm_kernels/utils/fp8.py:6-29`` in huggingface/hf-rocm-kernels): it returns an
``float8_e4m3fnuz`` tensor and the scale doubled, because a byte read as e4m3fnuz is worth half of
the same byte read as e4m3fn. ``fp8_quantize_e4m3fn`` is the form native to B200, whose tensor
cores consume OCP e4m3fn directly: same rounding, no reinterpretation, scale unchanged.
"""
from typing import Optional, Tuple

import torch
from torch import Tensor

E4M3FN_MAX = 448.0
_NEGATIVE_ZERO_BYTE = -128  # 0x80: -0.0 in e4m3fn, NaN in e4m3fnuz


def _to_e4m3fn(x_full_precision: Tensor, scale: Tensor) -> Tensor:
    scaled = x_full_precision * scale.reciprocal()
    return scaled.clamp(min=-E4M3FN_MAX, max=E4M3FN_MAX).to(torch.float8_e4m3fn)


def fp8_quantize(x_full_precision: Tensor, scale: Tensor) -> Tuple[Tensor, Tensor]:
    """Quantises with a tensor-wise ``scale`` and returns ``(x as float8_e4m3fnuz, 2 * scale)``.

    The values are rounded on the e4m3fn grid; the one byte that means NaN in e4m3fnuz (0x80, the
    negative zero of e4m3fn) is replaced by +0 before the bits are relabelled as e4m3fnuz.
    """
    as_bytes = _to_e4m3fn(x_full_precision, scale).view(torch.int8)
    as_bytes = torch.where(as_bytes == _NEGATIVE_ZERO_BYTE, torch.zeros_like(as_bytes), as_bytes)
    return as_bytes.view(torch.float8_e4m3fnuz), scale * 2.0


def fp8_quantize_e4m3fn(x_full_precision: Tensor, scale: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """Quantises to ``float8_e4m3fn``; ``scale`` defaults to ``amax(|x|) / 448`` (float32, one element).

    Returns ``(x as float8_e4m3fn, scale)`` with ``x ~= q.float() * scale``.
    """
    if scale is None:
        scale = (x_full_precision.abs().amax().to(torch.float32) / E4M3FN_MAX).reshape(1)
    return _to_e4m3fn(x_full_precision, scale), scale
