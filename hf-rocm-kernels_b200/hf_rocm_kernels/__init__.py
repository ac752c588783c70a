"""B200 (sm_100a) drop-in for the FP8 skinny GEMM of huggingface/hf-rocm-kernels.

``from hf_rocm_kernels import skinny_gemm`` works as it does with the reference
(``hf_rocm_kernels/__init__.py:4``); the other three operators of the reference (increment,
residual_rms, swiglu) are not part of this package.
"""
from .operators.skinny_gemm import skinny_gemm

__all__ = ["skinny_gemm"]
