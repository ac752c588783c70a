"""The MLP block of a decoder layer through ``llama_mlp_combined_ops``: three launches (swiglu in
the gate/up GEMM's epilogue) against the reference's four, with the weights of every call coming
from HBM (several weight sets rotate through a CUDA graph).

    python -m hf_rocm_kernels.benchmarks.llama_mlp.block --tokens 1 16 --hidden 4096 --intermediate 14336
    python -m hf_rocm_kernels.benchmarks.llama_mlp.block --tokens 16 --plain-calls 3      # for a profiler
"""
import argparse

import torch

from hf_rocm_kernels.combined_ops import can_fuse_swiglu, llama_mlp_combined_ops
from hf_rocm_kernels.utils.benchmarking import time_graph_us
from hf_rocm_kernels.utils.fp8 import fp8_quantize_e4m3fn


def make_block(tokens: int, hidden: int, inter: int, sets: int, device: str = "cuda"):
    """Inputs of ``sets`` MLP blocks that share activations and differ in their weights."""
    gen = torch.Generator(device=device).manual_seed(7)
    attn = torch.randn(tokens, hidden, device=device, generator=gen).bfloat16()
    residual = torch.randn(tokens, hidden, device=device, generator=gen).bfloat16()
    rms_weight = torch.ones(hidden, device=device).bfloat16()
    gate_up = [fp8_quantize_e4m3fn(torch.randn(2 * inter, hidden, device=device, generator=gen) * 0.02)
               for _ in range(sets)]
    down = [fp8_quantize_e4m3fn(torch.randn(hidden, inter, device=device, generator=gen) * 0.02)
            for _ in range(sets)]
    s_in = torch.tensor([4.0 / 448], device=device)
    s_act = torch.tensor([16.0 / 448], device=device)

    def run(i: int, fuse=None):
        j = i % sets
        return llama_mlp_combined_ops(attn, residual, rms_weight, 1e-5, gate_up[j][0].t(), s_in, s_in * gate_up[j][1],
                                      down[j][0].t(), s_act, s_act * down[j][1], fuse_swiglu=fuse)

    return run


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--tokens", "-t", nargs="+", type=int, default=[1, 16])
    parser.add_argument("--hidden", type=int, default=4096)
    parser.add_argument("--intermediate", type=int, default=14336)
    parser.add_argument("--plain-calls", type=int, default=0,
                        help="run this many blocks with plain launches and exit (no graph, no timing)")
    args = parser.parse_args()
    weight_bytes = 3 * args.intermediate * args.hidden
    sets = max(2, int(2 * 126e6 / weight_bytes) + 2)

    for tokens in args.tokens:
        run = make_block(tokens, args.hidden, args.intermediate, sets)
        if args.plain_calls:
            for i in range(args.plain_calls):
                run(i)
            torch.cuda.synchronize()
            print(f"{args.plain_calls} blocks of {tokens} tokens run")
            continue
        fusable = can_fuse_swiglu(tokens, args.hidden, args.intermediate)
        four = time_graph_us(lambda i: run(i, False), graph_size=2 * sets, warmups=5, iterations=20)
        line = f"tokens {tokens:3d}: four launches {four:7.2f} us ({weight_bytes / four / 1e6:.2f} TB/s of weights)"
        if fusable:
            three = time_graph_us(lambda i: run(i, True), graph_size=2 * sets, warmups=5, iterations=20)
            line += f" | three launches {three:7.2f} us ({weight_bytes / three / 1e6:.2f} TB/s)"
        else:
            line += " | the library splits K for this gate/up shape: swiglu stays a kernel of its own"
        print(line, flush=True)


if __name__ == "__main__":
    main()
