"""swiglu against vLLM's ``silu_and_mul`` followed by its static fp8 quantiser, when a vLLM build
with CUDA custom ops is importable. Counterpart of the reference's
``hf_rocm_kernels/benchmarks/swiglu/vs_vllm.py``.

    python -m hf_rocm_kernels.benchmarks.swiglu.vs_vllm -r 1 16 256 -i 14336
"""
import argparse

import torch

from hf_rocm_kernels.operators.swiglu import generate_swiglu_data, swiglu
from hf_rocm_kernels.utils.benchmarking import Bench


def load_vllm_ops():
    """The three vLLM kernels the comparisons need (``silu_and_mul``, ``scaled_fp8_quant``,
    ``fused_add_rms_norm``) as attributes of one object, or None with the reason printed. vLLM has
    moved ``silu_and_mul`` between its Python wrapper module and ``torch.ops._C`` over time."""
    try:
        import types

        import vllm._custom_ops as ops

        silu = getattr(ops, "silu_and_mul", None) or torch.ops._C.silu_and_mul
        return types.SimpleNamespace(silu_and_mul=silu, scaled_fp8_quant=ops.scaled_fp8_quant,
                                     fused_add_rms_norm=ops.fused_add_rms_norm)
    except BaseException as error:   # vLLM raises more than ImportError when its extension is absent
        print(f"vLLM custom ops unavailable ({type(error).__name__}: {error}); only this library is timed.")
        return None


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--rows", "-r", nargs="+", type=int, default=[1, 2, 4, 8, 16, 32, 64, 128, 256])
    parser.add_argument("--intermediate-size", "-i", type=int, default=14336)
    args = parser.parse_args()

    ops = load_vllm_ops()
    bench = Bench()
    for rows in args.rows:
        gate_up, scale, _ = generate_swiglu_data(rows, args.intermediate_size, 0, seed=0)
        if ops is not None:
            activated = torch.empty((rows, args.intermediate_size), dtype=gate_up.dtype, device=gate_up.device)

            def vllm_swiglu():
                ops.silu_and_mul(activated, gate_up)
                return ops.scaled_fp8_quant(activated, scale)

            bench.add_measure("vLLM (us)", rows, vllm_swiglu)
        bench.add_measure("Ours (us)", rows, lambda: swiglu(gate_up, scale, None, out_dtype=torch.float8_e4m3fn))
    if ops is not None:
        bench.add_speedup_column("vLLM (us)", "Ours (us)")
    bench.display_table(row_header="rows")


if __name__ == "__main__":
    main()
