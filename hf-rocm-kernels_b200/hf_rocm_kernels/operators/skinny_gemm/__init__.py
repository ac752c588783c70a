from .wrapped import skinny_gemm
from .reference import reference_skinny_gemm, generate_skinny_gemm_data

__all__ = ["skinny_gemm", "reference_skinny_gemm", "generate_skinny_gemm_data"]
