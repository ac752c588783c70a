"""increment: the registration smoke test of the extension."""
from . import wrapped as _wrapped

increment = _wrapped.increment

__all__ = ("increment",)
