"""residual_rms against vLLM's ``fused_add_rms_norm`` (16-bit output) and the same followed by its
static fp8 quantiser, when a vLLM build with CUDA custom ops is importable. Counterpart of the
reference's ``hf_rocm_kernels/benchmarks/residual_rms/vs_vllm.py``.

    python -m hf_rocm_kernels.benchmarks.residual_rms.vs_vllm -r 1 16 256 -c 4096
"""
import argparse

import torch

from hf_rocm_kernels.benchmarks.swiglu.vs_vllm import load_vllm_ops
from hf_rocm_kernels.operators.residual_rms import generate_residual_rms_data, residual_rms
from hf_rocm_kernels.utils.benchmarking import Bench


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--rows", "-r", nargs="+", type=int, default=[1, 2, 4, 8, 16, 32, 64, 128, 256])
    parser.add_argument("--cols", "-c", type=int, default=4096)
    parser.add_argument("--fp16-output", action="store_true")
    args = parser.parse_args()

    ops = load_vllm_ops()
    dtype = torch.float16 if args.fp16_output else torch.float8_e4m3fn
    bench = Bench()
    for rows in args.rows:
        x, res, w, eps, scale, _ = generate_residual_rms_data(rows, args.cols, 0, dtype, seed=0)
        if ops is not None:
            def vllm_residual_rms():
                ops.fused_add_rms_norm(x, res, w, eps)
                return x if scale is None else ops.scaled_fp8_quant(x, scale)

            bench.add_measure("vLLM (us)", rows, vllm_residual_rms)
        bench.add_measure("Ours (us)", rows,
                          lambda: residual_rms(x, res, w, eps, scale, None, out_dtype=torch.float8_e4m3fn))
    if ops is not None:
        bench.add_speedup_column("vLLM (us)", "Ours (us)")
    bench.display_table(row_header="rows")


if __name__ == "__main__":
    main()
