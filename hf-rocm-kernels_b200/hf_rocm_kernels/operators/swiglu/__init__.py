from .wrapped import swiglu
from .reference import reference_swiglu, generate_swiglu_data

__all__ = ["swiglu", "reference_swiglu", "generate_swiglu_data"]
