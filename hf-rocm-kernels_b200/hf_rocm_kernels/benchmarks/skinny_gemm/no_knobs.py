"""Times one (M, N, K) with the library's own launch shape, against ``torch._scaled_mm``.

The counterpart of the reference's ``hf_rocm_kernels/benchmarks/skinny_gemm/no_knobs.py``: same
question ("how fast is the op with no manual tuning, and how does it compare with the vendor
GEMM"), same method (CUDA graph of back-to-back calls on different weight matrices, see
``operators/skinny_gemm/benchmarking_fn.py``). Also the small, self-contained command used for
profiler captures:

    python -m hf_rocm_kernels.benchmarks.skinny_gemm.no_knobs --m 16 --n 28672 --k 4096 --plain-calls 3
"""
import argparse
import json

import torch

from hf_rocm_kernels import skinny_gemm
from hf_rocm_kernels.operators.skinny_gemm.benchmarking_fn import benchmark_skinny_gemm


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--m", type=int, default=16)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--k", type=int, default=4096)
    parser.add_argument("--plain-calls", type=int, default=0,
                        help="only issue this many plain (non-graph) calls on different weights and exit")
    parser.add_argument("--iterations", type=int, default=64)
    args = parser.parse_args()
    if args.plain_calls > 0:
        dev = torch.device("cuda")
        a = torch.randint(0, 120, (args.m, args.k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        ws = [torch.randint(0, 120, (args.n, args.k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
              for _ in range(args.plain_calls)]
        scale = torch.full((1,), 1e-4, device=dev)
        out = torch.zeros((args.m, args.n), dtype=torch.bfloat16, device=dev)
        for w in ws:
            skinny_gemm(a, w.t(), scale, out)
        torch.cuda.synchronize()
        print(json.dumps({"calls": args.plain_calls, "checksum": float(out.float().abs().sum())}))
        return
    ours, ours_std = benchmark_skinny_gemm(args.m, args.n, args.k, skg_kwargs={}, iterations=args.iterations)
    ref, ref_std = benchmark_skinny_gemm(args.m, args.n, args.k, skg_kwargs=None, iterations=args.iterations)
    bytes_moved = args.n * args.k + args.m * args.k + 4 * args.m * args.n + 4
    print(json.dumps({
        "m": args.m, "n": args.n, "k": args.k, "us_per_call": round(ours, 3), "std": round(ours_std, 3),
        "hbm_tbps": round(bytes_moved / ours / 1e6, 3), "scaled_mm_us_per_call": round(ref, 3),
        "percent_of_scaled_mm_speed": round(100.0 * ref / ours, 2)}))


if __name__ == "__main__":
    main()
