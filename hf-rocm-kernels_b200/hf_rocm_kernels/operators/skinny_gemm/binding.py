"""Positional bridge to the registered torch op, as in the reference's
``hf_rocm_kernels/operators/skinny_gemm/binding.py:7-28``: same function name, same argument
names and order, same integer return value."""
import torch
from torch import Tensor

import hf_rocm_kernels._HFRK_C  # noqa: F401  (loads the extension that registers torch.ops._HFRK_C)


def _skinny_gemm(
    A: Tensor,
    B: Tensor,
    scale_tensor: Tensor,
    D: Tensor,
    split_k: int,
    A_producers: int,
    B_producers: int,
    consumers: int,
    a_lanes: int,
    b_lanes: int,
    qsize: int,
    op_m: int,
    ops: int,
) -> int:
    """``D += scale_tensor[0] * (A @ B)`` in place; returns the launcher's status code (0 = success).

    ``split_k`` is honoured as a request (0 lets the library choose); the other eight integers
    steered the reference's MI300X producer/consumer kernel and are accepted and ignored.
    """
    return torch.ops._HFRK_C.skinny_gemm_tb(
        A, B, D, scale_tensor, split_k, A_producers, B_producers, consumers, a_lanes, b_lanes, qsize, op_m, ops
    )
