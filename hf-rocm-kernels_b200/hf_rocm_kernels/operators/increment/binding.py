"""Bridge to the registered torch op, as in the reference's
``hf_rocm_kernels/operators/increment/binding.py:6-7``."""
import torch

import hf_rocm_kernels._HFRK_C  # noqa: F401  (loads the extension that registers torch.ops._HFRK_C)


def _increment(x: torch.Tensor) -> None:
    torch.ops._HFRK_C.increment(x)
