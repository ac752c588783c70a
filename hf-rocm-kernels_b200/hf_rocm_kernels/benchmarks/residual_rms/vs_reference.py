"""residual_rms: the kernel (16-byte loads and element by element) against the torch statement, per
row count. Counterpart of the reference's ``hf_rocm_kernels/benchmarks/residual_rms/vs_reference.py``.

    python -m hf_rocm_kernels.benchmarks.residual_rms.vs_reference -r 1 16 256 -c 4096 -b 28672
"""
import argparse

import torch

from hf_rocm_kernels.operators.residual_rms import generate_residual_rms_data, reference_residual_rms, residual_rms
from hf_rocm_kernels.utils.benchmarking import Bench


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--rows", "-r", nargs="+", type=int, default=[1, 2, 4, 8, 16, 32, 64, 128, 256])
    parser.add_argument("--cols", "-c", type=int, default=4096)
    parser.add_argument("--buffer-cols", "-b", type=int, default=0)
    parser.add_argument("--fp16-output", action="store_true", help="no scale: keep the output in 16 bits")
    args = parser.parse_args()

    dtype = torch.float16 if args.fp16_output else torch.float8_e4m3fnuz
    bench = Bench()
    for rows in args.rows:
        x, res, w, eps, scale, next_buffer = generate_residual_rms_data(rows, args.cols, args.buffer_cols, dtype, seed=0)
        bench.add_measure("Torch (us)", rows, lambda: reference_residual_rms(x.clone(), res, w, eps, scale, next_buffer))
        bench.add_measure("Scalar (us)", rows,
                          lambda: residual_rms(x, res, w, eps, scale, next_buffer, force_scalar=True))
        t = bench.add_measure("Vectorized (us)", rows, lambda: residual_rms(x, res, w, eps, scale, next_buffer))
        moved = rows * args.cols * (6 + (2 if args.fp16_output else 1)) + args.cols * 2 + rows * args.buffer_cols * 2
        bench.add_raw_measure("GB/s", rows, moved / t / 1e3)
    bench.add_speedup_column("Torch (us)", "Vectorized (us)")
    print(f"cols {args.cols}, buffer cols {args.buffer_cols}, output {dtype}")
    bench.display_table(row_header="rows")


if __name__ == "__main__":
    main()
