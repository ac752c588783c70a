"""residual_rms: the operator, its two torch statements and its input generator."""
from . import reference as _reference
from . import wrapped as _wrapped

residual_rms = _wrapped.residual_rms
reference_residual_rms = _reference.reference_residual_rms
precise_residual_rms = _reference.precise_residual_rms
generate_residual_rms_data = _reference.generate_residual_rms_data

__all__ = ("residual_rms", "reference_residual_rms", "generate_residual_rms_data", "precise_residual_rms")
