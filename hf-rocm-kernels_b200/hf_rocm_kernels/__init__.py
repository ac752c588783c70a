"""B200 (sm_100a) drop-in for the decode-path operators of huggingface/hf-rocm-kernels.

``from hf_rocm_kernels import skinny_gemm, residual_rms, swiglu`` works as it does with the
reference (``hf_rocm_kernels/__init__.py:1-6``). The reference's fourth operator, ``increment``
(a build smoke test that adds one to a tensor), is not part of this package.
"""
from .operators.residual_rms import residual_rms
from .operators.swiglu import swiglu
from .operators.skinny_gemm import skinny_gemm

__all__ = ["residual_rms", "swiglu", "skinny_gemm"]
