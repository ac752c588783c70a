"""Grid search over the launch shape of ``skinny_gemm`` (K split x pipeline stages) per problem size.

Counterpart of the reference's ``hf_rocm_kernels/benchmarks/skinny_gemm/grid_search.py`` (which
sweeps producers/consumers/lanes/queue size of its MI300X kernel and dumps a JSON per shape): same
timing function, results written incrementally, best entry per shape. The output is the tuning
file ``operators/skinny_gemm/tuning.py`` loads.

    python -m hf_rocm_kernels.benchmarks.skinny_gemm.grid_search --out tuning.json            # Llama-3 8B/70B + shards
    python -m hf_rocm_kernels.benchmarks.skinny_gemm.grid_search --shapes 4096x4096 --m 1 16
"""
import argparse
import json
from typing import List, Tuple

from hf_rocm_kernels import _capi
from hf_rocm_kernels.benchmarks.skinny_gemm.workloads import LLAMA3_8B, LLAMA3_70B
from hf_rocm_kernels.operators.skinny_gemm.benchmarking_fn import benchmark_skinny_gemm

SPLITS = (1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 16)
STAGES = (2, 3, 4, 6)


def default_shapes() -> List[Tuple[int, int]]:
    shapes = list(LLAMA3_8B.values()) + list(LLAMA3_70B.values())
    for n, k in LLAMA3_70B.values():
        for g in (2, 4, 8):
            shapes.append((n // g, k))           # column-parallel shard
    for g in (2, 4, 8):
        shapes.append((8192, 28672 // g))        # row-parallel shard of the down projection
    return sorted(set(shapes))


def candidates(m: int, n: int, k: int):
    tiles, k_blocks = (n + 127) // 128, (k + 127) // 128
    for split in SPLITS:
        if split > 1 and split > k_blocks // 2:
            continue
        for stages in STAGES:
            try:
                plan = _capi.plan(m, n, k, _capi.VARIANT_CLUSTER, split)
            except _capi.HfrkError:
                continue
            if plan["split_k"] != split:
                continue
            # a clustered grid must be resident at once; plain CTAs may queue
            smem = plan["smem_bytes"] - plan["num_stages"] * (16384 + 128 * plan["m_pad"]) + stages * (16384 + 128 * plan["m_pad"])
            per_sm = (228 * 1024) // (smem + 1024)
            if per_sm < 1 or (split > 1 and tiles * split > 148 * per_sm):
                continue
            yield split, stages


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--shapes", nargs="*", default=None, help="NxK pairs, e.g. 4096x4096 28672x4096")
    parser.add_argument("--m", nargs="*", type=int, default=[16])
    parser.add_argument("--iterations", type=int, default=24)
    parser.add_argument("--warmups", type=int, default=8)
    parser.add_argument("--out", default="skinny_gemm_tuning.json")
    args = parser.parse_args()
    shapes = default_shapes() if not args.shapes else [tuple(int(v) for v in s.split("x")) for s in args.shapes]
    entries, log = [], []
    for n, k in shapes:
        for m in args.m:
            default_us, _ = benchmark_skinny_gemm(m, n, k, skg_kwargs={}, warmups=args.warmups,
                                                  iterations=args.iterations, mode="median")
            best = None
            for split, stages in candidates(m, n, k):
                us, _ = benchmark_skinny_gemm(
                    m, n, k, skg_kwargs=dict(variant=_capi.VARIANT_CLUSTER, split_k=split, num_stages=stages, use_pdl=True),
                    warmups=args.warmups, iterations=args.iterations, mode="median")
                log.append({"m": m, "n": n, "k": k, "split_k": split, "num_stages": stages, "us": round(us, 3)})
                if best is None or us < best[0]:
                    best = (us, split, stages)
            if best is None:
                continue
            entries.append({"m": m, "n": n, "k": k, "split_k": best[1], "num_stages": best[2],
                            "us": round(best[0], 3), "default_us": round(default_us, 3)})
            print(f"m={m:3d} n={n:6d} k={k:6d}: best split {best[1]:2d} stages {best[2]} -> {best[0]:7.2f} us "
                  f"(built-in rule {default_us:7.2f} us)", flush=True)
            with open(args.out, "w") as fh:      # incremental, like the reference's search
                json.dump({"entries": entries, "all": log}, fh, indent=1)
    print(f"wrote {args.out}: {len(entries)} entries")


if __name__ == "__main__":
    main()
