"""On-device comparator and input generator for ``skinny_gemm``.

Same names and signatures as the reference's
``hf_rocm_kernels/operators/skinny_gemm/reference.py`` (:8-26 and :29-46). The comparator is
``torch._scaled_mm`` (cuBLASLt on B200), which wants ``float8_e4m3fn``: e4m3fnuz inputs are
relabelled and their scale halved, which is exact for every byte the quantiser emits.
"""
from typing import Optional, Tuple

import torch
from torch import Tensor

from hf_rocm_kernels.utils.fp8 import fp8_quantize, fp8_quantize_e4m3fn


def _as_e4m3fn(x: Tensor, scale: Tensor) -> Tuple[Tensor, Tensor]:
    if x.dtype == torch.float8_e4m3fnuz:
        return x.view(torch.float8_e4m3fn), scale * 0.5
    return x, scale


def reference_skinny_gemm(
    skinny_a: Tensor,
    b: Tensor,
    scale_a: Tensor,
    scale_b: Tensor,
    output: Optional[Tensor] = None,
) -> Tensor:
    """``cast(scale_a * scale_b * (skinny_a @ b))`` through ``torch._scaled_mm``, written to ``output``."""
    out_dtype = torch.float16 if output is None else output.dtype
    a_fn, sa = _as_e4m3fn(skinny_a, scale_a.reshape(()).float())
    b_fn, sb = _as_e4m3fn(b, scale_b.reshape(()).float())
    result = torch._scaled_mm(a_fn, b_fn, scale_a=sa, scale_b=sb, out_dtype=out_dtype)
    if output is None:
        return result
    output.copy_(result)
    return output


def generate_skinny_gemm_data(
    m: int, n: int, k: int, seed: Optional[int] = None, fp8_dtype: torch.dtype = torch.float8_e4m3fnuz,
    out_dtype: torch.dtype = torch.float16, device: str = "cuda",
) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """Random (skinny_a, b, scale_tensor, zeroed output) as the reference's tests draw them:
    one scale ~ U(1, 3) used to quantise N(0,1) activations (m, k) and weights (n, k); ``b`` is
    the transposed view of the weights. ``fp8_dtype`` picks the reference's e4m3fnuz or e4m3fn."""
    if seed is not None:
        torch.manual_seed(seed)
    scale_tensor = torch.rand((1,), device=device, dtype=torch.float32) * 2 + 1
    a_full = torch.normal(0, 1, size=(m, k), device=device, dtype=torch.float32)
    w_full = torch.normal(0, 1, size=(n, k), device=device, dtype=torch.float32)
    if fp8_dtype == torch.float8_e4m3fnuz:
        skinny_a = fp8_quantize(a_full, scale_tensor)[0]
        weights = fp8_quantize(w_full, scale_tensor)[0]
    else:
        skinny_a = fp8_quantize_e4m3fn(a_full, scale_tensor)[0]
        weights = fp8_quantize_e4m3fn(w_full, scale_tensor)[0]
    output = torch.zeros((m, n), dtype=out_dtype, device=device)
    return skinny_a, weights.t(), scale_tensor, output
