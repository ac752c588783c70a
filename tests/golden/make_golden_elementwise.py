"""Generates ``elementwise.npz`` in this folder from the reference itself.

Run once, in a container where the reference checkout is present (it is not needed afterwards):

    python tests/golden/make_golden_elementwise.py /path/to/hf-rocm-kernels

What is taken from the reference: ``hf_rocm_kernels/utils/fp8.py``,
``hf_rocm_kernels/operators/swiglu/reference.py`` and
``hf_rocm_kernels/operators/residual_rms/reference.py`` are loaded from the checkout by file path
(the package itself cannot be imported without its compiled extension) and their
``reference_swiglu``, ``reference_residual_rms`` and ``precise_residual_rms`` are EXECUTED on CPU.
The file holds their inputs and what they returned.

The reference draws its test inputs with the GPU generator (``generate_swiglu_data``,
``generate_residual_rms_data``), which cannot be reproduced here; the cases below use a CPU
generator seeded per case with the same distributions: N(0, 1) fp16 values, scale ~ U(1, 3),
epsilon ~ U(1e-5, 2e-5).
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

SWIGLU_SHAPES = [(1, 8), (3, 24), (4, 128), (8, 512), (1, 4096), (1, 6656)]          # (rows, hidden)
RMS_SHAPES = [(1, 8), (3, 24), (4, 128), (8, 512), (1, 4096), (1, 16384)]           # (rows, cols)


def _load(name: str, path: str):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def load_reference(reference_root: str):
    """fp8.py under its real dotted name (the two reference.py files import it that way), inside
    empty stand-ins for the parent packages."""
    pkg = os.path.join(reference_root, "hf_rocm_kernels")
    for name in ("hf_rocm_kernels", "hf_rocm_kernels.utils"):
        stub = types.ModuleType(name)
        stub.__path__ = []
        sys.modules[name] = stub
    _load("hf_rocm_kernels.utils.fp8", os.path.join(pkg, "utils", "fp8.py"))
    swiglu = _load("reference_swiglu_module", os.path.join(pkg, "operators", "swiglu", "reference.py"))
    rms = _load("reference_rms_module", os.path.join(pkg, "operators", "residual_rms", "reference.py"))
    return swiglu.reference_swiglu, rms.reference_residual_rms, rms.precise_residual_rms


def f16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main(reference_root: str) -> None:
    reference_swiglu, reference_residual_rms, precise_residual_rms = load_reference(reference_root)
    out = {}

    for idx, (rows, hidden) in enumerate(SWIGLU_SHAPES):
        gen = torch.Generator().manual_seed(3000 + idx)
        gate_up = torch.randn(rows, 2 * hidden, generator=gen).to(torch.float16)
        scale = torch.rand(1, generator=gen) * 2 + 1
        buffer = torch.full((rows, 16), 7.0, dtype=torch.float16)
        q = reference_swiglu(gate_up.clone(), scale, buffer)
        assert q.dtype == torch.float8_e4m3fnuz and float(buffer.abs().sum()) == 0.0
        out[f"s{idx}_gate_up"] = f16_bits(gate_up)
        out[f"s{idx}_scale"] = scale.numpy().astype(np.float32)
        out[f"s{idx}_bytes"] = q.view(torch.uint8).numpy().copy()
    out["swiglu_count"] = np.array([len(SWIGLU_SHAPES)], dtype=np.int64)

    for idx, (rows, cols) in enumerate(RMS_SHAPES):
        gen = torch.Generator().manual_seed(4000 + idx)
        x = torch.randn(rows, cols, generator=gen).to(torch.float16)
        res = torch.randn(rows, cols, generator=gen).to(torch.float16)
        weight = torch.randn(cols, generator=gen).to(torch.float16)
        epsilon = float((torch.rand(1, generator=gen) + 1) * 1e-5)
        scale = torch.rand(1, generator=gen) * 2 + 1
        y16, new_res, _ = reference_residual_rms(x.clone(), res.clone(), weight, epsilon, None)
        y8, new_res8, doubled = reference_residual_rms(x.clone(), res.clone(), weight, epsilon, scale)
        assert torch.equal(new_res, new_res8) and float(doubled) == float(scale * 2)
        p64, _ = precise_residual_rms(x.clone(), res.clone(), weight, epsilon, None)
        p8, _ = precise_residual_rms(x.clone(), res.clone(), weight, epsilon, scale)
        out[f"r{idx}_input"] = f16_bits(x)
        out[f"r{idx}_residual"] = f16_bits(res)
        out[f"r{idx}_weight"] = f16_bits(weight)
        out[f"r{idx}_epsilon"] = np.array([epsilon], dtype=np.float64)
        out[f"r{idx}_scale"] = scale.numpy().astype(np.float32)
        out[f"r{idx}_new_residual"] = f16_bits(new_res)
        out[f"r{idx}_out_f16"] = f16_bits(y16)
        out[f"r{idx}_out_bytes"] = y8.view(torch.uint8).numpy().copy()
        if cols <= 512:   # the reference's test reads it as float32; kept for the small cases only
            out[f"r{idx}_precise_f32"] = p64.float().numpy().copy()
        out[f"r{idx}_precise_bytes"] = p8.view(torch.uint8).numpy().copy()
    out["rms_count"] = np.array([len(RMS_SHAPES)], dtype=np.int64)

    path = os.path.join(HERE, "elementwise.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/hf-rocm-kernels")
    main(sys.argv[1])
