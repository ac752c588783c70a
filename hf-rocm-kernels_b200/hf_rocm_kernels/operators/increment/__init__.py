from .wrapped import increment

__all__ = ["increment"]
