"""Hands the tensor to ``torch.ops._HFRK_C.increment`` (the reference does the same in
``operators/increment/binding.py``); importing the extension module registers the op."""
from torch import Tensor, ops

from hf_rocm_kernels import _HFRK_C as _extension  # noqa: F401


def _increment(x: Tensor) -> None:
    ops._HFRK_C.increment(x)
