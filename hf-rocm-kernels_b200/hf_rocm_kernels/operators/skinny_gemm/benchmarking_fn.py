"""CUDA-graph timing of ``skinny_gemm`` on rotating weights.

Same entry point and method as the reference's
``hf_rocm_kernels/operators/skinny_gemm/benchmarking_fn.py:8-101``: ``graph_size`` different weight
matrices, one graph of ``graph_size`` back-to-back calls captured on a side stream, replayed
``warmups + iterations`` times between CUDA events, microseconds per call = replay time /
``graph_size``. Differences: the pool is sized from the L2 (at least twice its capacity, so that no
call finds its weights cached), inputs are ``float8_e4m3fn`` with bf16 output by default, and
``skg_kwargs`` may carry the pins of ``_capi.skinny_gemm_ex`` instead of the reference's nine knobs.
"""
from typing import Any, Dict, Optional, Tuple

import torch

from hf_rocm_kernels import _capi
from hf_rocm_kernels.operators.skinny_gemm.wrapped import skinny_gemm
from hf_rocm_kernels.utils.fp8 import fp8_quantize_e4m3fn

from hf_rocm_kernels.operators.skinny_gemm.binding import _skinny_gemm


def l2_bytes(device: str = "cuda") -> int:
    """The L2 capacity of the device the benchmark runs on (126 MiB on B200), asked of the driver."""
    return int(torch.cuda.get_device_properties(device).L2_cache_size)


def benchmark_skinny_gemm(
    m: int,
    n: int,
    k: int,
    skg_kwargs: Optional[Dict[str, Any]] = None,
    graph_size: int = 8,
    warmups: int = 32,
    iterations: int = 128,
    device: str = "cuda",
    mode: str = "mean",
    out_dtype: torch.dtype = torch.bfloat16,
) -> Tuple[float, float]:
    """Returns (mean or median microseconds per call, standard deviation).

    ``skg_kwargs=None`` times ``torch._scaled_mm`` (the vendor GEMM), ``{}`` the wrapped operator,
    anything else is forwarded to ``_capi.skinny_gemm_ex`` (variant, split_k, num_stages, ...).
    """
    graph_size = max(graph_size, -(-2 * l2_bytes(device) // (n * k)))
    activations, scale_a = fp8_quantize_e4m3fn(torch.randn((m, k), device=device))
    weights = [fp8_quantize_e4m3fn(torch.randn((n, k), device=device)) for _ in range(graph_size)]
    scales = [(scale_a * scale_w).float() for _w, scale_w in weights]
    output = torch.zeros((m, n), device=device, dtype=out_dtype)

    if skg_kwargs is None:
        def fn(i: int) -> None:
            torch._scaled_mm(activations, weights[i][0].t(), scale_a=scale_a.reshape(()),
                             scale_b=weights[i][1].reshape(()), out_dtype=out_dtype, out=output)
    elif not skg_kwargs:
        def fn(i: int) -> None:
            skinny_gemm(activations, weights[i][0].t(), scales[i], output)
    else:
        def fn(i: int) -> None:
            _capi.check(_capi.skinny_gemm_ex(activations, weights[i][0], output, scales[i], **skg_kwargs))

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        fn(0)  # first call outside the capture (library scratch, cuBLASLt heuristics)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(graph_size):
                fn(i)
        torch.cuda.synchronize()
        samples = []
        for i in range(warmups + iterations):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            if i >= warmups:
                samples.append(1000.0 * start.elapsed_time(end) / graph_size)
    stats = torch.tensor(samples)
    if mode == "mean":
        return stats.mean().item(), stats.std().item()
    if mode == "median":
        return stats.median().item(), stats.std().item()
    raise ValueError(f"Invalid mode: {mode}")


def benchmark_skinny_gemm_general(
    m: int,
    n: int,
    k: int,
    split_k: int,
    A_producers: int = 0,
    B_producers: int = 0,
    consumers: int = 0,
    a_lanes: int = 0,
    b_lanes: int = 0,
    qsize: int = 0,
    op_m: int = 0,
    ops: int = 0,
    graph_size: int = 8,
    warmups: int = 32,
    iterations: int = 128,
    device: str = "cuda",
) -> Tuple[float, float]:
    """The reference's second timing entry point (``benchmarking_fn.py:103-197``), same signature:
    times the raw binding ``_skinny_gemm`` with the nine knobs given by hand, or ``torch._scaled_mm``
    when ``split_k == 0``; fp16 output as in the reference. Of the knobs only ``split_k`` steers
    this library (as a hint); the others are accepted so that existing sweep scripts run. Returns
    (mean, standard deviation) in microseconds per call."""
    graph_size = max(graph_size, -(-2 * l2_bytes(device) // (n * k)))
    activations, scale_a = fp8_quantize_e4m3fn(torch.randn((m, k), device=device))
    weights = [fp8_quantize_e4m3fn(torch.randn((n, k), device=device)) for _ in range(graph_size)]
    scales = [(scale_a * scale_w).float() for _w, scale_w in weights]
    output = torch.zeros((m, n), device=device, dtype=torch.float16)

    if split_k == 0:
        def fn(i: int) -> None:
            torch._scaled_mm(activations, weights[i][0].t(), scale_a=scale_a.reshape(()),
                             scale_b=weights[i][1].reshape(()), out_dtype=torch.float16, out=output)
    else:
        def fn(i: int) -> None:
            _skinny_gemm(A=activations, B=weights[i][0].t(), scale_tensor=scales[i], D=output, split_k=split_k,
                         A_producers=A_producers, B_producers=B_producers, consumers=consumers, a_lanes=a_lanes,
                         b_lanes=b_lanes, qsize=qsize, op_m=op_m, ops=ops)

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        fn(0)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(graph_size):
                fn(i)
        torch.cuda.synchronize()
        samples = []
        for i in range(warmups + iterations):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            if i >= warmups:
                samples.append(1000.0 * start.elapsed_time(end) / graph_size)
    stats = torch.tensor(samples)
    return stats.mean().item(), stats.std().item()
