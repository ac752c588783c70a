"""``swiglu`` with the signature of the reference's wrapper
(``hf_rocm_kernels/operators/swiglu/wrapped.py:49-84``): checks, output allocation, one launch."""
from typing import Optional

import torch
from torch import Tensor

from .binding import _swiglu

MAX_THREADS_PER_SM = 1024
_FP8_DTYPES = (torch.float8_e4m3fnuz, torch.float8_e4m3fn)


def swiglu_checks(gate_up_proj: Tensor, scale_tensor: Tensor, next_buffer: Tensor) -> None:
    """The argument checks of the reference (``wrapped.py:11-29``), with bf16 admitted next to fp16."""
    assert gate_up_proj.dim() == 2, f"Expected gate_up_proj to have 2 dims but got {gate_up_proj.dim() = } instead."
    assert gate_up_proj.size(1) % 2 == 0, f"Expected gate_up_proj an even number of columns: {gate_up_proj.shape}."
    assert gate_up_proj.dtype in (torch.float16, torch.bfloat16), f"Expected fp16 or bf16, got {gate_up_proj.dtype = }"
    assert next_buffer.size(0) == gate_up_proj.size(0), \
        f"Expected same number of rows: {next_buffer.shape = } but {gate_up_proj.shape = }."
    assert next_buffer.element_size() == 2, f"Expected a 16-bit next_buffer but got {next_buffer.dtype = }"
    assert scale_tensor.numel() == 1, f"Expected {scale_tensor.numel() = } to be 1."
    device = gate_up_proj.device
    assert device.type == "cuda", f"Expected gate_up_proj.device to be of type cuda, but got {device.type = } instead."
    assert scale_tensor.device == device, f"Expected {scale_tensor.device = } to be the same as {device = }"
    assert next_buffer.device == device, f"Expected {next_buffer.device = } to be the same as {device = }"
    assert gate_up_proj.is_contiguous(), f"Expected gate_up_proj to be contiguous but got {gate_up_proj.stride() = }"
    assert next_buffer.is_contiguous(), f"Expected next_buffer to be contiguous but got {next_buffer.stride() = }"


def infer_num_threads(rows: int, force_scalar: bool, num_threads: int) -> int:
    """Kept for callers that pass the result on (reference ``wrapped.py:31-47``). The B200 kernel
    strides a fixed-size grid over the matrix, so the value does not reach the launch."""
    if 0 < num_threads <= MAX_THREADS_PER_SM:
        return num_threads
    return 256


def swiglu(
    gate_up_proj: Tensor,
    scale_tensor: Tensor,
    next_buffer: Optional[Tensor] = None,
    force_scalar: bool = False,
    num_threads: int = -1,
    out_dtype: torch.dtype = torch.float8_e4m3fnuz,
) -> Tensor:
    """SwiGLU fused with the conversion to fp8; can also zero a buffer with as many rows.

    Args:
        gate_up_proj: (rows, 2 * hidden) fp16 or bf16, row-major; gate in the left half, up in the right
        scale_tensor: one fp32 on the device; the activation is divided by it before the conversion
        next_buffer: optional 16-bit tensor of shape (rows, .) to fill with zeros
        force_scalar: take the element-by-element kernel even when 16-byte loads are possible
        num_threads: accepted for compatibility, not used
        out_dtype: ``float8_e4m3fnuz`` (the reference's format, the default) or ``float8_e4m3fn``
    Returns the (rows, hidden) fp8 tensor.
    """
    assert out_dtype in _FP8_DTYPES, f"Expected an e4m3 output dtype but got {out_dtype = }"
    if next_buffer is None:
        next_buffer = torch.empty(size=(gate_up_proj.size(0), 0), device=gate_up_proj.device, dtype=torch.float16)
    swiglu_checks(gate_up_proj, scale_tensor, next_buffer)
    swiglu_out = torch.empty(
        size=(gate_up_proj.size(0), gate_up_proj.size(1) // 2), dtype=out_dtype, device=gate_up_proj.device
    )
    _swiglu(
        gate_up_proj=gate_up_proj,
        scale_tensor=scale_tensor,
        swiglu_out=swiglu_out,
        next_buffer=next_buffer,
        force_scalar=force_scalar,
        num_threads=infer_num_threads(gate_up_proj.size(0), force_scalar, num_threads),
    )
    return swiglu_out
