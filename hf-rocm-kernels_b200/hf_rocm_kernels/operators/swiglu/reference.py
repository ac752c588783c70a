"""Torch statement of the swiglu operator and its input generator, with the names and argument
order of the reference's ``hf_rocm_kernels/operators/swiglu/reference.py`` (``reference_swiglu``
:7-27, ``generate_swiglu_data`` :30-42)."""
from typing import Optional, Tuple

import torch
from torch import Tensor

from hf_rocm_kernels.utils.fp8 import fp8_quantize


def reference_swiglu(gate_up_proj: Tensor, scale_tensor: Tensor, next_buffer: Optional[Tensor]) -> Tensor:
    """silu(gate) * up in fp32, then ``fp8_quantize`` with ``scale_tensor``; zeroes ``next_buffer``.

    Returns e4m3fnuz bytes worth ``x / (2 * scale_tensor)``: the kernel reproduces them when it is
    given the doubled scale, as ``fp8_quantize`` hands it on.
    """
    assert gate_up_proj.dtype in (torch.float16, torch.bfloat16), f"Expected a 16-bit input, got {gate_up_proj.dtype = }"
    if next_buffer is not None:
        assert next_buffer.element_size() == 2, f"Expected a 16-bit next_buffer, got {next_buffer.dtype = }"
    halves = gate_up_proj.view(-1, 2, gate_up_proj.size(1) // 2).float()
    activated = torch.nn.functional.silu(halves[:, 0]) * halves[:, 1]
    quantised, _ = fp8_quantize(activated, scale_tensor)
    if next_buffer is not None:
        next_buffer.fill_(0)
    return quantised


def generate_swiglu_data(
    rows: int, hidden_dim: int, buffer_cols: int = 0, seed: Optional[int] = None,
    dtype: torch.dtype = torch.float16, device: str = "cuda",
) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
    """N(0, 1) gate_up of shape (rows, 2 * hidden_dim), a scale in [1, 3) and, when ``buffer_cols``
    is non-zero, an uninitialised (rows, buffer_cols) buffer."""
    if seed is not None:
        torch.manual_seed(seed)
    gate_up_proj = torch.normal(0, 1, size=(rows, 2 * hidden_dim), device=device, dtype=dtype)
    scale_tensor = torch.rand(size=(1,), device=device, dtype=torch.float32).mul(2).add(1)
    next_buffer = None if buffer_cols == 0 else torch.empty((rows, buffer_cols), device=device, dtype=dtype)
    return gate_up_proj, scale_tensor, next_buffer
