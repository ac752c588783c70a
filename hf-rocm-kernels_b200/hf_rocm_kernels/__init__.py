"""B200 (sm_100a) drop-in for the operators of huggingface/hf-rocm-kernels.

``from hf_rocm_kernels import skinny_gemm, residual_rms, swiglu, increment`` works as it does with
the reference (``hf_rocm_kernels/__init__.py:1-6``).
"""
from .operators.increment import increment
from .operators.residual_rms import residual_rms
from .operators.swiglu import swiglu
from .operators.skinny_gemm import skinny_gemm

__all__ = ["increment", "residual_rms", "swiglu", "skinny_gemm"]
