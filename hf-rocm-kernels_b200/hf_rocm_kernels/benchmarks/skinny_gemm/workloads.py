"""Seeded synthetic inputs for the five benchmark configurations of the FP8 skinny GEMM.

No dataset or checkpoint is involved: the Llama-3 8B/70B projection *dimensions* stand in for the
models, values are N(0, 1) drawn from a seeded generator and quantised per tensor to e4m3fn with
``scale = amax / 448`` (``utils/fp8.py``). The reference draws its benchmark inputs the same way
(``hf_rocm_kernels/operators/skinny_gemm/benchmarking_fn.py:20-28`` of the reference), with its
own shapes.

Configurations (index = position in the benchmark specification):
  0  single call M=1, N=K=4096, no bias
  1  Llama-3-8B decode projections, M in {1,2,4,8,16}; bias (bf16 N(0, 0.02)) on qkv only
  2  Llama-3-70B decode projections, M in {1,4,16}; weights N-split over 1/2/4/8 GPUs
  3  row-parallel down_proj A[M,28672] x W[8192,28672], M in {1,2,8,16}; K-split over 2/4/8 GPUs
  4  edge sweep: M in {3,5,7,13,16} x N in {1000,4104,11008} x K in {1040,4096,5120}, bias on every
     other case, 1 % of the entries replaced by +-1e6 AFTER the scale is taken (they saturate to +-448)
Seed of a case = 1000 * configuration + case index.

This module imports torch only (nothing else of the package), so that a CPU-only arm of a benchmark
can load it by file path without loading the CUDA libraries.
"""
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor

E4M3FN_MAX = 448.0   # largest finite e4m3fn value; the same constant as utils/fp8.py

LLAMA3_8B = {"qkv": (6144, 4096), "o_proj": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336)}
LLAMA3_70B = {"qkv": (10240, 8192), "o_proj": (8192, 8192), "gate_up": (57344, 8192), "down": (8192, 28672)}


@dataclass(frozen=True)
class Case:
    config: int
    index: int
    name: str
    m: int
    n: int
    k: int
    bias: bool = False
    outliers: bool = False

    @property
    def seed(self) -> int:
        return 1000 * self.config + self.index

    @property
    def weight_bytes(self) -> int:
        return self.n * self.k

    def algorithmic_bytes(self, out_bytes: int = 2) -> int:
        """W + A + D written (+ D read when a bias is accumulated) + the scale."""
        d = self.m * self.n * out_bytes
        return self.n * self.k + self.m * self.k + d + (d if self.bias else 0) + 4


def cases(config: int) -> List[Case]:
    out: List[Case] = []
    if config == 0:
        out.append(Case(0, 0, "single", 1, 4096, 4096))
    elif config == 1:
        for m in (1, 2, 4, 8, 16):
            for name, (n, k) in LLAMA3_8B.items():
                out.append(Case(1, len(out), f"8b_{name}_m{m}", m, n, k, bias=(name == "qkv")))
    elif config == 2:
        for m in (1, 4, 16):
            for name, (n, k) in LLAMA3_70B.items():
                out.append(Case(2, len(out), f"70b_{name}_m{m}", m, n, k))
    elif config == 3:
        for m in (1, 2, 8, 16):
            out.append(Case(3, len(out), f"70b_down_rowpar_m{m}", m, 8192, 28672))
    elif config == 4:
        for m in (3, 5, 7, 13, 16):
            for n in (1000, 4104, 11008):
                for k in (1040, 4096, 5120):
                    idx = len(out)
                    out.append(Case(4, idx, f"edge_m{m}_n{n}_k{k}", m, n, k, bias=(idx % 2 == 0), outliers=True))
    else:
        raise ValueError(f"unknown configuration {config}")
    return out


def _quantize(x: Tensor, outlier_mask: Optional[Tensor], outlier_sign: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    scale = (x.abs().amax().to(torch.float32) / E4M3FN_MAX).reshape(1)
    if outlier_mask is not None:
        x = torch.where(outlier_mask, outlier_sign * 1e6, x)
    q = (x * scale.reciprocal()).clamp(-E4M3FN_MAX, E4M3FN_MAX).to(torch.float8_e4m3fn)
    return q, scale


def make_inputs(case: Case, device: str = "cpu", out_dtype: torch.dtype = torch.bfloat16) -> Dict[str, Optional[Tensor]]:
    """Draws one case. Returns ``a`` [M,K] and ``w`` [N,K] as float8_e4m3fn, ``scale`` = scale_a *
    scale_w (float32, one element), ``scale_a``/``scale_w`` and ``d_in`` (the bias broadcast over
    M in ``out_dtype``, or None). The generator lives on ``device``; CPU and CUDA streams of
    random numbers differ, so parity tests draw on CPU and move the tensors."""
    gen = torch.Generator(device=device).manual_seed(case.seed)
    a_full = torch.randn((case.m, case.k), generator=gen, device=device, dtype=torch.float32)
    w_full = torch.randn((case.n, case.k), generator=gen, device=device, dtype=torch.float32)
    masks = [None, None, None, None]
    if case.outliers:
        for i, t in enumerate((a_full, w_full)):
            masks[2 * i] = torch.rand(t.shape, generator=gen, device=device) < 0.01
            masks[2 * i + 1] = torch.where(torch.rand(t.shape, generator=gen, device=device) < 0.5, -1.0, 1.0)
    a_q, scale_a = _quantize(a_full, masks[0], masks[1])
    w_q, scale_w = _quantize(w_full, masks[2], masks[3])
    d_in = None
    if case.bias:
        bias = (torch.randn((case.n,), generator=gen, device=device, dtype=torch.float32) * 0.02).to(out_dtype)
        d_in = bias.unsqueeze(0).repeat(case.m, 1).contiguous()
    return {"a": a_q, "w": w_q, "scale": (scale_a * scale_w).to(torch.float32), "scale_a": scale_a,
            "scale_w": scale_w, "d_in": d_in}


# ------------------------------------------------------------------------------- sharding
def n_split_rows(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows [begin, end) of W (= columns of the output) held by ``rank`` under column-parallel
    sharding. N must divide evenly, as it does for every benchmark shape and world size."""
    if n % world != 0:
        raise ValueError(f"N={n} does not divide over {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def k_split_cols(k: int, world: int, rank: int, align: int = 16) -> Tuple[int, int]:
    """Columns [begin, end) of A and W held by ``rank`` under row-parallel sharding; shard
    boundaries stay multiples of ``align`` so that every shard is a valid GEMM on its own."""
    if k % (world * align) != 0:
        raise ValueError(f"K={k} does not divide over {world} ranks in multiples of {align}")
    per = k // world
    return rank * per, (rank + 1) * per
