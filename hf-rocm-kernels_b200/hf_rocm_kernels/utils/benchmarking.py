"""Latency measurement for single operators: a CUDA graph of back-to-back calls timed with CUDA
events on the stream that replays it, and a small table builder.

Same role and entry points as the reference's ``hf_rocm_kernels/utils/benchmarking.py``
(``benchmark_cuda_graph_no_cache`` :14-67, ``Bench`` :70-146); the timing is done here with torch
alone. A graph holds ``graph_size`` calls, each on its own set of tensors so that no call finds its
inputs in L1, and the figure returned is the median replay time divided by ``graph_size``.
"""
import itertools
import warnings
from typing import Callable, Dict, Sequence

import torch


def randomize_tensors(x):
    """A fresh N(0, 1) tensor of the same shape and dtype; anything that is not a tensor is kept."""
    if isinstance(x, torch.Tensor) and x.numel() > 0 and x.is_floating_point() and x.element_size() > 1:
        return torch.randn(x.shape, device=x.device, dtype=torch.float32).to(x.dtype)
    return x


def time_graph_us(call: Callable[[int], None], graph_size: int = 16, warmups: int = 10, iterations: int = 50,
                  device: str = "cuda") -> float:
    """``call(i)`` for i in range(graph_size) captured once, replayed ``warmups + iterations``
    times; returns the median microseconds per call."""
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        call(0)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(graph_size):
                call(i)
        samples = []
        for it in range(warmups + iterations):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            if it >= warmups:
                samples.append(start.elapsed_time(end) * 1000.0 / graph_size)
    samples.sort()
    return samples[len(samples) // 2]


def benchmark_cuda_graph_no_cache(fn, args: Sequence, kwargs: Dict, graph_size: int = 8, warmups: int = 32,
                                  iterations: int = 128, device: str = "cuda") -> float:
    """Microseconds per call of ``fn(*args, **kwargs)`` with the tensor arguments re-drawn for
    every slot of the graph."""
    arg_sets = [tuple(randomize_tensors(a) for a in args) for _ in range(graph_size)]
    kwarg_sets = [{k: randomize_tensors(v) for k, v in kwargs.items()} for _ in range(graph_size)]
    return time_graph_us(lambda i: fn(*arg_sets[i], **kwarg_sets[i]), graph_size, warmups, iterations, device)


class Bench:
    """Collects (column, row) -> microseconds and prints them as one table."""

    def __init__(self) -> None:
        torch.set_grad_enabled(False)
        self.check_device_is_free(warn_if_not=True)
        self._measures: Dict[str, Dict[int, float]] = {}

    @staticmethod
    def check_device_is_free(warn_if_not: bool = False) -> Dict[str, int]:
        """Utilisation and memory use of the current GPU as NVML reports them (read-only queries); on a
        shared machine a busy GPU explains a bad number. Same role as the reference's
        ``Bench.check_device_is_free`` (``utils/benchmarking.py:83-95``). Returns -1 where NVML is
        not available."""
        metrics = {"utilization": -1, "memory_usage": -1}
        try:
            metrics["utilization"] = int(torch.cuda.utilization())
            metrics["memory_usage"] = int(torch.cuda.memory_usage())
        except Exception:
            pass
        if warn_if_not and (metrics["utilization"] > 0 or metrics["memory_usage"] > 0):
            warnings.warn(f"Device {torch.cuda.current_device()} is not fully free: {metrics = }")
        return metrics

    @staticmethod
    def benchmark_fn(fn: Callable[[], None], graph_size: int = 16, iterations: int = 50) -> float:
        """Microseconds per call of ``fn()``, from a graph of ``graph_size`` calls."""
        t = time_graph_us(lambda i: fn(), graph_size=graph_size, iterations=iterations)
        torch.cuda.synchronize()
        return t

    def add_measure(self, header: str, label: int, fn: Callable[[], None]) -> float:
        t = self.benchmark_fn(fn)
        self.add_raw_measure(header, label, t)
        return t

    def add_raw_measure(self, header: str, label: int, measure: float) -> None:
        self._measures.setdefault(header, {})[label] = measure

    def add_speedup_column(self, ref_header: str, our_header: str) -> None:
        if ref_header not in self._measures or our_header not in self._measures:
            raise ValueError(f"Headers {ref_header} and {our_header} must be present in the benchmark table.")
        for label, ref in self._measures[ref_header].items():
            if label in self._measures[our_header]:
                self.add_raw_measure("Speedup", label, ref / self._measures[our_header][label])

    def display_table(self, row_header: str) -> None:
        rows = sorted(set(itertools.chain(*[m.keys() for m in self._measures.values()])))
        headers = [row_header] + list(self._measures)
        table = [[str(r)] + [f"{self._measures[h][r]:.3f}" if r in self._measures[h] else "-"
                             for h in self._measures] for r in rows]
        widths = [max(len(h), *(len(line[i]) for line in table)) if table else len(h) for i, h in enumerate(headers)]
        print("  ".join(h.rjust(w) for h, w in zip(headers, widths)))
        print("  ".join("-" * w for w in widths))
        for line in table:
            print("  ".join(c.rjust(w) for c, w in zip(line, widths)))
