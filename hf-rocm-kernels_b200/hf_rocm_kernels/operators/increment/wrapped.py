"""``increment``: one ATen ``add_`` behind the same registration path as the real operators. The
reference ships it as its build smoke test (``operators/increment/wrapped.py``)."""
from torch import Tensor

from . import binding


def increment(x: Tensor) -> None:
    """x <- x + 1, in place; ``x`` must live on a CUDA device."""
    if x.device.type != "cuda":
        raise AssertionError(f"increment works on CUDA tensors, got one on {x.device}")
    binding._increment(x)
