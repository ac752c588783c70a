"""Generates the golden vectors in this folder from the reference itself.

Run once, in a container where the reference checkout is present (it is not needed afterwards):

    python tests/golden/make_golden.py /path/to/hf-rocm-kernels

What is taken from the reference:

* ``hf_rocm_kernels/utils/fp8.py`` is loaded from the checkout and its ``fp8_quantize`` is EXECUTED
  on CPU: ``quantiser.npz`` holds its inputs (values, scales) and the bytes it returned.
* The expected GEMM results come from ``torch._scaled_mm``, the function the reference's
  ``reference_skinny_gemm`` calls (``operators/skinny_gemm/reference.py:18-25``), with the same
  arguments as the reference's test (``tests/test_skinny_gemm.py:13-17``: ``scale_a = scale``,
  ``scale_b = 1``, fp16 output). The CPU build of that function does not take ``float8_e4m3fnuz``,
  so the bytes are relabelled ``float8_e4m3fn`` and the scale is multiplied by 0.25 (each fnuz
  operand is worth exactly half of the same byte read as e4m3fn). ``gemm_cases.npz`` holds the
  bytes, the scale, the optional ``D_in`` and the fp16/bf16 bit patterns returned.

The reference's own inputs cannot be regenerated bit-for-bit (it draws them with the GPU
generator), so the cases here are drawn with a CPU generator seeded per case, with the
distribution of ``generate_skinny_gemm_data`` (``reference.py:29-46``): scale ~ U(1, 3) shared by
both operands, N(0, 1) values.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

GEMM_SHAPES = [  # (m, n, k, with_d_in)
    (1, 128, 256, False), (2, 136, 256, False), (3, 40, 1040, True), (8, 64, 512, False),
    (11, 96, 256, True), (16, 128, 256, False), (17, 66, 256, False), (32, 64, 256, True),
]


def load_reference_fp8(reference_root: str):
    path = os.path.join(reference_root, "hf_rocm_kernels", "utils", "fp8.py")
    spec = importlib.util.spec_from_file_location("reference_fp8", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.fp8_quantize


def main(reference_root: str) -> None:
    fp8_quantize = load_reference_fp8(reference_root)

    # ---- quantiser vectors
    gen = torch.Generator().manual_seed(20240)
    values = torch.cat([
        torch.randn(4096, generator=gen) * 3.0,
        torch.linspace(-500.0, 500.0, 4001),
        torch.tensor([0.0, -0.0, 1e-9, -1e-9, 2.0 ** -10, 1.5 * 2.0 ** -9, 0.5 * 2.0 ** -9, 2.5 * 2.0 ** -9,
                      447.9, 448.0, 448.1, -448.1, 464.0, 1e6, -1e6, 0.0019531251]),
    ]).float()
    scales = torch.tensor([1.0, 0.5, 2.3, 0.0107421875, 1.7], dtype=torch.float32)
    q_bytes = []
    doubled = []
    for s in scales:
        q, s2 = fp8_quantize(values.clone(), s.reshape(1))
        assert q.dtype == torch.float8_e4m3fnuz
        q_bytes.append(q.view(torch.uint8).numpy().copy())
        doubled.append(float(s2))
    np.savez_compressed(os.path.join(HERE, "quantiser.npz"), values=values.numpy(), scales=scales.numpy(),
                        bytes=np.stack(q_bytes), returned_scales=np.array(doubled, dtype=np.float32))

    # ---- GEMM cases
    out = {}
    for idx, (m, n, k, with_d) in enumerate(GEMM_SHAPES):
        gen = torch.Generator().manual_seed(1000 + idx)
        scale = torch.rand(1, generator=gen) * 2 + 1
        a = fp8_quantize(torch.randn(m, k, generator=gen), scale)[0]
        w = fp8_quantize(torch.randn(n, k, generator=gen), scale)[0]
        a_fn = a.view(torch.uint8).view(torch.float8_e4m3fn)
        w_fn = w.view(torch.uint8).view(torch.float8_e4m3fn)
        scale_fn = (scale * 0.25).reshape(())
        one = torch.ones(())
        res16 = torch._scaled_mm(a_fn, w_fn.t(), scale_a=scale_fn, scale_b=one, out_dtype=torch.float16)
        resbf = torch._scaled_mm(a_fn, w_fn.t(), scale_a=scale_fn, scale_b=one, out_dtype=torch.bfloat16)
        res32 = torch._scaled_mm(a_fn, w_fn.t(), scale_a=scale_fn, scale_b=one, out_dtype=torch.float32)
        out[f"c{idx}_shape"] = np.array([m, n, k], dtype=np.int64)
        out[f"c{idx}_a"] = a.view(torch.uint8).numpy().copy()
        out[f"c{idx}_w"] = w.view(torch.uint8).numpy().copy()
        out[f"c{idx}_scale"] = scale.numpy().astype(np.float32)
        out[f"c{idx}_f16"] = res16.view(torch.int16).numpy().view(np.uint16).copy()
        out[f"c{idx}_bf16"] = resbf.view(torch.int16).numpy().view(np.uint16).copy()
        out[f"c{idx}_f32"] = res32.numpy().copy()
        if with_d:
            bias = (torch.randn(n, generator=gen) * 0.02).to(torch.float16)
            out[f"c{idx}_d_in_f16"] = bias.repeat(m, 1).view(torch.int16).numpy().view(np.uint16).copy()
    out["count"] = np.array([len(GEMM_SHAPES)], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "gemm_cases.npz"), **out)
    print("wrote", os.path.join(HERE, "quantiser.npz"), os.path.join(HERE, "gemm_cases.npz"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/hf-rocm-kernels")
    main(sys.argv[1])
