"""``residual_rms`` with the signature of the reference's wrapper
(``hf_rocm_kernels/operators/residual_rms/wrapped.py:78-126``): checks, output allocation, one launch."""
from typing import Optional, Tuple

import torch
from torch import Tensor

from .binding import _residual_rms

_FP8_DTYPES = (torch.float8_e4m3fnuz, torch.float8_e4m3fn)


def residual_rms_checks(
    input: Tensor,
    residual: Tensor,
    weight: Tensor,
    scale_tensor: Optional[Tensor],
    epsilon: float,
    next_buffer: Tensor,
) -> None:
    """The argument checks of the reference (``wrapped.py:11-37``), with bf16 admitted next to fp16."""
    assert input.dim() == 2, f"Expected input to have 2 dimensions but got {input.dim() = } instead."
    assert residual.shape == input.shape, \
        f"Expected input and residual to have same shape but got {input.shape = } and {residual.shape = }"
    assert weight.shape == (input.size(1), ), \
        f"Expected weight to have shape {(input.size(1), ) = } but got {weight.shape = }"
    assert input.dtype in (torch.float16, torch.bfloat16), f"Expected fp16 or bf16 but got {input.dtype = }"
    assert residual.dtype == input.dtype and weight.dtype == input.dtype, \
        f"Expected one dtype but got {input.dtype = }, {residual.dtype = }, {weight.dtype = }"
    device = input.device
    assert device.type == "cuda", f"Expected input.device to be of type cuda, but got {device.type = } instead."
    assert residual.device == device, f"Expected {residual.device = } to be the same as {input.device = }"
    assert weight.device == device, f"Expected {weight.device = } to be the same as {input.device = }"
    if scale_tensor is not None:
        assert scale_tensor.device == device, f"Expected {scale_tensor.device = } to be the same as {input.device = }"
        assert scale_tensor.numel() == 1, f"Expected {scale_tensor.numel() = } to be 1."
    assert next_buffer.device == device, f"Expected {next_buffer.device = } to be the same as {input.device = }"
    assert next_buffer.size(0) == input.size(0), \
        f"Expected same number of rows: {next_buffer.shape = } but {input.shape = }."
    assert input.is_contiguous(), f"Expected input to be contiguous but got {input.stride() = }"
    assert residual.is_contiguous(), f"Expected residual to be contiguous but got {residual.stride() = }"
    assert next_buffer.is_contiguous(), f"Expected next_buffer to be contiguous but got {next_buffer.stride() = }"
    assert epsilon > 0, f"Expected RMS epsilon to be > 0 to avoid division by zero, but got {epsilon = }"


def infer_num_threads(rows: int, num_threads: int) -> int:
    """0 lets the library size the CTA from the row length (one 16-byte vector per thread, up to
    1024 threads); any other value in [1, 1024] is passed on (reference ``wrapped.py:60-76``)."""
    if num_threads < 0 or num_threads > 1024:
        raise ValueError(f"{num_threads = } is not between 0 and 1024")
    return num_threads


def residual_rms(
    input: Tensor,
    residual: Tensor,
    weight: Tensor,
    epsilon: float,
    scale_tensor: Optional[Tensor] = None,
    next_buffer: Optional[Tensor] = None,
    num_threads: int = 0,
    force_scalar: bool = False,
    out_dtype: torch.dtype = torch.float8_e4m3fnuz,
) -> Tuple[Tensor, Tensor]:
    """Residual connection, RMS norm and conversion to fp8 in one kernel. ``residual`` is modified
    in place (``residual <- input + residual``).

    Args:
        input, residual: (rows, cols) fp16 or bf16, row-major
        weight: (cols,) weight of the RMS norm, same dtype
        epsilon: added to the mean of squares
        scale_tensor: one fp32 on the device that divides the result before the conversion to fp8;
            ``None`` keeps the result in the input's dtype
        next_buffer: optional 16-bit tensor of shape (rows, .) to fill with zeros
        num_threads: CTA size (a multiple of 32); 0 lets the library choose
        out_dtype: fp8 format used when ``scale_tensor`` is given: ``float8_e4m3fnuz`` (the
            reference's, the default) or ``float8_e4m3fn``
    Returns ``(output, residual)``.
    """
    assert out_dtype in _FP8_DTYPES, f"Expected an e4m3 output dtype but got {out_dtype = }"
    if next_buffer is None:
        next_buffer = torch.empty(size=(input.size(0), 0), device=input.device, dtype=torch.float16)
    residual_rms_checks(input, residual, weight, scale_tensor, epsilon, next_buffer)
    num_threads = infer_num_threads(input.size(0), num_threads)
    output = torch.empty(
        size=input.shape, dtype=(out_dtype if scale_tensor is not None else input.dtype), device=input.device
    )
    _residual_rms(
        input=input,
        residual=residual,
        weight=weight,
        scale_tensor=scale_tensor,
        epsilon=epsilon,
        output=output,
        next_buffer=next_buffer,
        num_threads=num_threads,
        force_scalar=force_scalar,
    )
    return output, residual
