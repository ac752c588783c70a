"""``increment``: the reference's build smoke test (``operators/increment/wrapped.py:6-9``), a
one-line ATen op behind the same registration path as the real operators."""
import torch

from .binding import _increment


def increment(x: torch.Tensor) -> None:
    """Adds 1 to the given GPU-resident tensor in place."""
    assert x.device.type == "cuda", f"Expected x.device to be of type cuda but got {x.device.type = }"
    _increment(x)
