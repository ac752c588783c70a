"""User-facing ``skinny_gemm``: argument checks, output allocation, launch parameters.

Mirrors the reference's ``hf_rocm_kernels/operators/skinny_gemm/wrapped.py`` (checks :9-35,
parameter inference :42-102, entry point :104-128) with the differences B200 brings:

* inputs may be ``float8_e4m3fn`` (native to the tcgen05 tensor cores) as well as the reference's
  ``float8_e4m3fnuz``; the output may be ``bfloat16`` as well as ``float16``;
* the nine tuning integers no longer select a kernel; they are still produced so that code which
  prints or forwards them keeps working;
* a non-zero status from the launcher raises instead of being dropped (the reference ignores it,
  ``wrapped.py:124-127``).
"""
from typing import Dict, Optional

import torch
from torch import Tensor

from .binding import _skinny_gemm
from .tuning import load_from_environment

load_from_environment()  # HFRK_TUNING_FILE: per-shape launch shapes from the grid search

_FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e4m3fnuz)
_OUT_DTYPES = (torch.float16, torch.bfloat16)

_STATUS_TEXT = {
    3: "k must be a multiple of 16",
    6: "invalid shape or tuning value",
    7: "tensors must be 16-byte aligned and b.stride(1) a multiple of 16",
    8: "unsupported dtype",
    9: "CUDA error during launch",
    10: "device-side wait timed out",
}


def skinny_gemm_checks(
    skinny_a: Tensor,
    b: Tensor,
    scale_tensor: Tensor,
    output: Tensor,
) -> None:
    """Raises AssertionError unless the four tensors form a valid call (shapes, layouts, dtypes, device)."""
    m, k = skinny_a.size(0), skinny_a.size(1)
    assert skinny_a.dim() == 2, f"Expected skinny_a to have 2 dimensions but got {skinny_a.dim() = } instead."
    assert b.dim() == 2 and k == b.size(0), f"Expected {skinny_a.size(1) = } and {b.size(0) = } to be the same."
    assert scale_tensor.numel() == 1, f"Expected {scale_tensor.numel() = } to be 1."
    assert tuple(output.shape) == (m, b.size(1)), (
        f"{tuple(output.shape)} does not match with {tuple(skinny_a.shape) = } and {tuple(b.shape) = }")
    assert skinny_a.is_contiguous(), f"Expected skinny_a to be contiguous but got {skinny_a.stride() = }"
    assert b.stride(0) == 1, f"Expected b to be column-major but got {b.stride() = }"
    assert output.is_contiguous(), f"Expected output to be contiguous but got {output.stride() = }"
    assert skinny_a.dtype in _FP8_DTYPES, f"Expected {skinny_a.dtype = } to be one of {_FP8_DTYPES}"
    assert b.dtype in _FP8_DTYPES, f"Expected {b.dtype = } to be one of {_FP8_DTYPES}"
    assert scale_tensor.dtype == torch.float32, f"Expected {scale_tensor.dtype = } to be torch.float32"
    assert output.dtype in _OUT_DTYPES, f"Expected {output.dtype = } to be one of {_OUT_DTYPES}"
    device = skinny_a.device
    assert device.type == "cuda", f"Expected input.device to be of type cuda, but got {device.type = } instead."
    for name, tensor in (("b", b), ("scale_tensor", scale_tensor), ("output", output)):
        assert tensor.device == device, f"Expected {name}.device = {tensor.device} to be the same as {device = }"


def infer_skinny_gemm_params(skinny_a: Tensor, b: Tensor) -> Dict[str, int]:
    """The nine integers of the op schema for this call.

    On B200 the launch shape (K split, pipeline depth) is derived inside the library from
    (M, N, K) and the SM count, so ``split_k`` is 0 = "choose for me". The remaining values
    describe the kernel that actually runs, in the reference's vocabulary, for logs: one TMA
    producer warp feeds both operands, one warp issues the MMAs, the tile is 128 weight rows
    (``b_lanes`` x 16 x 8) by ``op_m`` padded tokens.
    """
    m = skinny_a.size(0)
    return {
        "split_k": 0, "A_producers": 1, "B_producers": 1, "consumers": 1,
        "a_lanes": 1, "b_lanes": 1, "qsize": 12, "op_m": 16 * ((min(m, 64) + 15) // 16), "ops": 4,
    }


def skinny_gemm(
    skinny_a: Tensor,
    b: Tensor,
    scale_tensor: Tensor,
    output: Optional[Tensor] = None,
) -> Tensor:
    """FP8 skinny GEMM ``output += scale_tensor * (skinny_a @ b)``.

    Args:
        skinny_a: fp8 (m, k) row-major activations.
        b: fp8 (k, n) column-major weights, i.e. ``weight_nk.t()`` of a row-major (n, k) matrix.
        scale_tensor: one float32 on the same device, the product of both quantisation scales.
        output: optional (m, n) float16/bfloat16 buffer that already holds zeros or the bias; the
            result is accumulated into it. Allocated as float16 zeros when omitted.
    Returns:
        ``output``.
    """
    if output is None:
        output = torch.zeros((skinny_a.size(0), b.size(1)), dtype=torch.float16, device=skinny_a.device)
    skinny_gemm_checks(skinny_a, b, scale_tensor, output)
    if torch.compiler.is_compiling():
        # a traced graph cannot hold an op that returns an int: same kernel, raises on a bad status
        torch.ops._HFRK_C.skinny_gemm_inplace(skinny_a, b, output, scale_tensor, 0)
        return output
    status = _skinny_gemm(A=skinny_a, B=b, scale_tensor=scale_tensor, D=output, **infer_skinny_gemm_params(skinny_a, b))
    if status != 0:
        raise RuntimeError(f"skinny_gemm failed with status {status}: {_STATUS_TEXT.get(status, 'see hfrk_b200.h')}")
    return output
