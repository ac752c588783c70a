"""skinny_gemm: the operator, its torch statement and its input generator."""
from . import reference as _reference
from . import wrapped as _wrapped

skinny_gemm = _wrapped.skinny_gemm
reference_skinny_gemm = _reference.reference_skinny_gemm
generate_skinny_gemm_data = _reference.generate_skinny_gemm_data

__all__ = ("skinny_gemm", "reference_skinny_gemm", "generate_skinny_gemm_data")
