"""The oracle as a timed CPU implementation -- TEST/BENCHMARK INFRASTRUCTURE ONLY.

What the reference defines as the expected result of the skinny GEMM is a dequantised matmul
(``hf_rocm_kernels/operators/skinny_gemm/reference.py:18-25`` calls ``torch._scaled_mm``; the
in-place ``D += ...`` contract is ``wrapped.py:115``). The reference has no CPU implementation of
its own, so the CPU baseline is this port of those semantics on the host cores: dequantise A and W
to float32, ``A32 @ W32.T`` with torch's CPU BLAS on all threads, apply the scale, add ``D_in``,
round to the output dtype. It is imported by the CPU-baseline leg of ``bench.py`` and by nothing
that ships.
"""
import os
import time
from typing import Dict, List, Optional

import torch


def host_threads() -> int:
    return len(os.sched_getaffinity(0))


def skinny_gemm_cpu(a_q: torch.Tensor, w_q: torch.Tensor, scale: torch.Tensor, d_in: Optional[torch.Tensor],
                    out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``cast(D_in + scale * (A @ W.T))`` for float8 CPU tensors ``a_q [M,K]``, ``w_q [N,K]``."""
    acc = a_q.float() @ w_q.float().t()
    acc = acc * scale.float()
    if d_in is not None:
        acc = acc + d_in.float()
    return acc.to(out_dtype)


def time_cases_predequantised(inputs: List[Dict[str, torch.Tensor]], repeats: int = 1,
                              threads: Optional[int] = None) -> float:
    """As :func:`time_cases` with the weights converted to float32 once, outside the timed region:
    the matmul, the scale, the bias and the cast only. The weight matrix is then 4 bytes per
    element in host memory, which no deployment of an fp8 model would keep; the figure separates
    the cost of the dequantisation from the cost of the product."""
    torch.set_num_threads(threads or host_threads())
    wide = [inp["w"].float() for inp in inputs]
    best = float("inf")
    for rep in range(repeats + 1):
        start = time.perf_counter()
        for inp, w32 in zip(inputs, wide):
            acc = (inp["a"].float() @ w32.t()) * inp["scale"].float()
            if inp["d_in"] is not None:
                acc = acc + inp["d_in"].float()
            acc.to(torch.bfloat16)
        elapsed = time.perf_counter() - start
        if rep > 0:
            best = min(best, elapsed)
    return best


def time_cases(inputs: List[Dict[str, torch.Tensor]], repeats: int = 1, threads: Optional[int] = None) -> float:
    """Seconds for one pass over ``inputs`` (dicts from ``workloads.make_inputs`` on CPU), best of
    ``repeats`` after one untimed pass."""
    torch.set_num_threads(threads or host_threads())
    best = float("inf")
    for rep in range(repeats + 1):
        start = time.perf_counter()
        for inp in inputs:
            skinny_gemm_cpu(inp["a"], inp["w"], inp["scale"], inp["d_in"])
        elapsed = time.perf_counter() - start
        if rep > 0:
            best = min(best, elapsed)
    return best
