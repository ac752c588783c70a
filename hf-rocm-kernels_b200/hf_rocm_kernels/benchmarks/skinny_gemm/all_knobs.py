"""Times one (M, N, K) with every launch knob set by hand, against ``torch._scaled_mm``.

Counterpart of the reference's ``hf_rocm_kernels/benchmarks/skinny_gemm/all_knobs.py`` (manual
producers/consumers/lanes/queue/ops there; kernel variant, K split, CTAs per SM, stages and
programmatic dependent launch here); prints the same "% of the reference's speed" figure
(``100 * t(_scaled_mm) / t(ours)``, ``all_knobs.py:99`` of the reference).
"""
import argparse

from hf_rocm_kernels import _capi
from hf_rocm_kernels.operators.skinny_gemm.benchmarking_fn import benchmark_skinny_gemm


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--m", type=int, default=16)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--k", type=int, default=4096)
    parser.add_argument("--variant", type=int, default=_capi.VARIANT_CLUSTER, help="1 cluster split-K, 2 stream-K")
    parser.add_argument("--split-k", type=int, default=0)
    parser.add_argument("--ctas-per-sm", type=int, default=0)
    parser.add_argument("--stages", type=int, default=0)
    parser.add_argument("--no-pdl", action="store_true")
    parser.add_argument("--iterations", type=int, default=128)
    args = parser.parse_args()
    knobs = dict(variant=args.variant, split_k=args.split_k, ctas_per_sm=args.ctas_per_sm, num_stages=args.stages,
                 use_pdl=not args.no_pdl)
    ours, std = benchmark_skinny_gemm(args.m, args.n, args.k, skg_kwargs=knobs, iterations=args.iterations)
    ref, ref_std = benchmark_skinny_gemm(args.m, args.n, args.k, skg_kwargs=None, iterations=args.iterations)
    print(f"skinny_gemm {knobs}: {ours:.3f} +- {std:.3f} us   torch._scaled_mm: {ref:.3f} +- {ref_std:.3f} us   "
          f"-> {100.0 * ref / ours:.2f} % of its speed")


if __name__ == "__main__":
    main()
