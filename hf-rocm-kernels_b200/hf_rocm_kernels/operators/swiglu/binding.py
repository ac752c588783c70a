"""Keyword bridge to the registered torch op, as in the reference's
``hf_rocm_kernels/operators/swiglu/binding.py:7-18``: same function name and argument names."""
import torch
from torch import Tensor

import hf_rocm_kernels._HFRK_C  # noqa: F401  (loads the extension that registers torch.ops._HFRK_C)


def _swiglu(
    gate_up_proj: Tensor,
    scale_tensor: Tensor,
    swiglu_out: Tensor,
    next_buffer: Tensor,
    num_threads: int,
    force_scalar: bool,
) -> None:
    """Fills ``swiglu_out`` with ``fp8(silu(gate) * up / scale)`` and ``next_buffer`` with zeros."""
    torch.ops._HFRK_C.swiglu(gate_up_proj, scale_tensor, swiglu_out, next_buffer, num_threads, force_scalar)
