"""Row-parallel (K split over GPUs) GEMM with the all-reduce in its epilogue, against the same GEMM
followed by an NCCL all-reduce, and against the local GEMM alone.

    torchrun --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29555 \\
        -m hf_rocm_kernels.benchmarks.skinny_gemm.row_parallel --tokens 1 16 -n 8192 -k 28672
    python -m hf_rocm_kernels.benchmarks.skinny_gemm.row_parallel --tokens 16 --plain-calls 3      # one GPU, for a profiler

(Under torchrun give the sizes as -n / -k: its own parser takes --n for an abbreviation of its options.)
Each rank holds K / world columns. Times are microseconds per call from a CUDA graph of 16 calls on 16
different weight shards, the maximum over ranks. Without torchrun the script runs as a group of one.
"""
import argparse
import os

import torch
import torch.distributed as dist

from hf_rocm_kernels import _capi
from hf_rocm_kernels.combined_ops import RowParallelSkinnyGemm, skinny_gemm_then_allreduce


def _graph_time_us(calls, device, world: int, reps: int = 20, warm: int = 5) -> float:
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for call in calls:
            call()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for call in calls:
                call()
        samples = []
        for i in range(warm + reps):
            if world > 1:
                dist.barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            graph.replay()
            end.record(stream)
            end.synchronize()
            if i >= warm:
                samples.append(start.elapsed_time(end) * 1000.0 / len(calls))
    samples.sort()
    value = torch.tensor([samples[len(samples) // 2]], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(value, op=dist.ReduceOp.MAX)
    return float(value)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--tokens", nargs="+", type=int, default=[1, 16])
    parser.add_argument("-n", "--n", type=int, default=8192)
    parser.add_argument("-k", "--k", type=int, default=28672, help="the whole K; every rank takes K / world of it")
    parser.add_argument("--plain-calls", type=int, default=0,
                        help="only issue this many plain (non-graph) fused calls per token count and exit")
    args = parser.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    k_shard = args.k // world
    group = RowParallelSkinnyGemm(max_m=16, max_n=args.n, device=device)
    scale = torch.full((1,), 1e-4, device=device)

    def fp8(rows, cols):
        return torch.randint(0, 120, (rows, cols), dtype=torch.uint8, device=device).view(torch.float8_e4m3fn)

    weights = [fp8(args.n, k_shard) for _ in range(max(16, args.plain_calls))]
    for m in args.tokens:
        a = fp8(m, k_shard)
        out = torch.zeros((m, args.n), dtype=torch.bfloat16, device=device)
        if args.plain_calls:
            for w in weights[:args.plain_calls]:
                group(a, w, scale, out)
            torch.cuda.synchronize()
            if rank == 0:
                print(f"{args.plain_calls} fused calls of m={m} run on {world} GPU(s)")
            continue
        partial = torch.empty((m, args.n), dtype=torch.float32, device=device)
        row = {}
        for mode in ("one_shot", "two_shot", "auto"):
            group.set_mode(mode)
            row[mode] = _graph_time_us([lambda w=w: group(a, w, scale, out) for w in weights[:16]], device, world)
        local_us = _graph_time_us([lambda w=w: _capi.check(_capi.skinny_gemm(a, w, out, scale)) for w in weights[:16]],
                                  device, world)
        unfused = _graph_time_us([lambda w=w: skinny_gemm_then_allreduce(a, w, scale, out, partial)
                                  for w in weights[:16]], device, world)
        if rank == 0:
            print(f"world={world} m={m} n={args.n} k/gpu={k_shard}: fused one-shot {row['one_shot']:.2f} "
                  f"two-shot {row['two_shot']:.2f} auto {row['auto']:.2f} | local GEMM {local_us:.2f} | "
                  f"GEMM + NCCL all-reduce {unfused:.2f} us", flush=True)
    code, word = _capi.device_status(clear=True)
    if code != 0:
        raise RuntimeError(f"device status word {word:#x}")
    if world > 1:
        dist.barrier()
    group.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
