"""swiglu: the kernel (16-byte loads and element by element) against the torch statement, per row
count. Counterpart of the reference's ``hf_rocm_kernels/benchmarks/swiglu/vs_reference.py``.

    python -m hf_rocm_kernels.benchmarks.swiglu.vs_reference -r 1 16 256 -i 14336 -b 4096
"""
import argparse

from hf_rocm_kernels.operators.swiglu import generate_swiglu_data, reference_swiglu, swiglu
from hf_rocm_kernels.utils.benchmarking import Bench


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--rows", "-r", nargs="+", type=int, default=[1, 2, 4, 8, 16, 32, 64, 128, 256, 2048])
    parser.add_argument("--intermediate-size", "-i", type=int, default=14336)
    parser.add_argument("--buffer-cols", "-b", type=int, default=0)
    args = parser.parse_args()

    bench = Bench()
    for rows in args.rows:
        gate_up, scale, next_buffer = generate_swiglu_data(rows, args.intermediate_size, args.buffer_cols, seed=0)
        bench.add_measure("Torch (us)", rows, lambda: reference_swiglu(gate_up, scale, next_buffer))
        bench.add_measure("Scalar (us)", rows, lambda: swiglu(gate_up, scale, next_buffer, force_scalar=True))
        t = bench.add_measure("Vectorized (us)", rows, lambda: swiglu(gate_up, scale, next_buffer))
        moved = rows * args.intermediate_size * 5 + rows * args.buffer_cols * 2
        bench.add_raw_measure("GB/s", rows, moved / t / 1e3)
    bench.add_speedup_column("Torch (us)", "Vectorized (us)")
    print(f"intermediate size {args.intermediate_size}, buffer cols {args.buffer_cols}")
    bench.display_table(row_header="rows")


if __name__ == "__main__":
    main()
