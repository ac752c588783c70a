from .wrapped import residual_rms
from .reference import reference_residual_rms, generate_residual_rms_data, precise_residual_rms

__all__ = ["residual_rms", "reference_residual_rms", "generate_residual_rms_data", "precise_residual_rms"]
