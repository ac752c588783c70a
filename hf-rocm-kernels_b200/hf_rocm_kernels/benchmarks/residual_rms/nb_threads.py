"""residual_rms latency against the CTA size, per row count: the sweep behind the library's
choice of one 16-byte vector per thread. Counterpart of the reference's
``hf_rocm_kernels/benchmarks/residual_rms/nb_threads.py``; prints a table instead of drawing a plot.

    python -m hf_rocm_kernels.benchmarks.residual_rms.nb_threads -r 1 16 64 -c 8192
"""
import argparse

import torch

from hf_rocm_kernels.operators.residual_rms import generate_residual_rms_data, residual_rms
from hf_rocm_kernels.utils.benchmarking import Bench


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--rows", "-r", nargs="+", type=int, default=[1, 4, 16, 64, 256])
    parser.add_argument("--cols", "-c", type=int, default=4096)
    parser.add_argument("--buffer-cols", "-b", type=int, default=0)
    parser.add_argument("--threads", "-t", nargs="+", type=int, default=[0] + [128 * i for i in range(1, 9)],
                        help="0 = the library's own choice")
    args = parser.parse_args()

    bench = Bench()
    for rows in args.rows:
        x, res, w, eps, scale, next_buffer = generate_residual_rms_data(
            rows, args.cols, args.buffer_cols, torch.float8_e4m3fnuz, seed=0)
        for threads in args.threads:
            bench.add_measure(f"rows={rows} (us)", threads,
                              lambda: residual_rms(x, res, w, eps, scale, next_buffer, num_threads=threads))
    print(f"cols {args.cols}, buffer cols {args.buffer_cols}")
    bench.display_table(row_header="threads")


if __name__ == "__main__":
    main()
