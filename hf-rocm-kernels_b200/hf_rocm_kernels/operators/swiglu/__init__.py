"""swiglu: the operator, its torch statement and its input generator."""
from . import reference as _reference
from . import wrapped as _wrapped

swiglu = _wrapped.swiglu
reference_swiglu = _reference.reference_swiglu
generate_swiglu_data = _reference.generate_swiglu_data

__all__ = ("swiglu", "reference_swiglu", "generate_swiglu_data")
