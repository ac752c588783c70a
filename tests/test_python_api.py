"""The Python surface the reference exposes for this path, checked without a GPU: names,
signatures, the op schema, argument checks."""
import inspect

import pytest
import torch


@pytest.fixture(scope="module")
def pkg(native_build):
    import hf_rocm_kernels

    return hf_rocm_kernels


def test_public_names(pkg):
    from hf_rocm_kernels.operators.skinny_gemm import generate_skinny_gemm_data, reference_skinny_gemm, skinny_gemm
    from hf_rocm_kernels.operators.skinny_gemm.binding import _skinny_gemm
    from hf_rocm_kernels.utils.fp8 import fp8_quantize
    from hf_rocm_kernels.utils.testing import compare_x_and_ref_to_precise, compare_x_with_ref

    assert pkg.skinny_gemm is skinny_gemm
    assert list(inspect.signature(skinny_gemm).parameters) == ["skinny_a", "b", "scale_tensor", "output"]
    assert list(inspect.signature(_skinny_gemm).parameters) == [
        "A", "B", "scale_tensor", "D", "split_k", "A_producers", "B_producers", "consumers",
        "a_lanes", "b_lanes", "qsize", "op_m", "ops"]
    assert list(inspect.signature(reference_skinny_gemm).parameters) == [
        "skinny_a", "b", "scale_a", "scale_b", "output"]
    assert list(inspect.signature(generate_skinny_gemm_data).parameters)[:4] == ["m", "n", "k", "seed"]
    assert callable(fp8_quantize) and callable(compare_x_with_ref) and callable(compare_x_and_ref_to_precise)


def test_op_schema_is_the_reference_schema(pkg):
    schema = torch.ops._HFRK_C.skinny_gemm_tb.default._schema
    # the reference's definition string (csrc/torch_bindings.cpp:38-41), parsed by torch itself
    want = torch._C.parse_schema(
        "_HFRK_C::skinny_gemm_tb(Tensor A, Tensor B, Tensor! D, Tensor scale_tensor, int split_k, int A_producers, "
        "int B_producers, int consumers, int a_lanes, int b_lanes, int qsize, int op_m, int ops) -> int")
    assert str(schema) == str(want)
    assert [a.name for a in schema.arguments] == [a.name for a in want.arguments]
    assert schema.arguments[2].alias_info is not None and schema.arguments[2].alias_info.is_write


def test_elementwise_operators_keep_the_reference_surface(pkg):
    """Names, argument order and op schemas of swiglu and residual_rms
    (reference: hf_rocm_kernels/__init__.py:1-6, operators/*/wrapped.py, csrc/torch_bindings.cpp:24-35)."""
    from hf_rocm_kernels.combined_ops import llama_mlp_combined_ops
    from hf_rocm_kernels.operators.residual_rms import (generate_residual_rms_data, precise_residual_rms,
                                                         reference_residual_rms, residual_rms)
    from hf_rocm_kernels.operators.residual_rms.binding import _residual_rms
    from hf_rocm_kernels.operators.swiglu import generate_swiglu_data, reference_swiglu, swiglu
    from hf_rocm_kernels.operators.swiglu.binding import _swiglu

    assert pkg.swiglu is swiglu and pkg.residual_rms is residual_rms
    assert pkg.__all__ == ["increment", "residual_rms", "swiglu", "skinny_gemm"]      # the reference's list
    assert str(torch.ops._HFRK_C.increment.default._schema) == str(
        torch._C.parse_schema("_HFRK_C::increment(Tensor! x) -> ()"))
    assert list(inspect.signature(swiglu).parameters)[:5] == [
        "gate_up_proj", "scale_tensor", "next_buffer", "force_scalar", "num_threads"]
    assert list(inspect.signature(_swiglu).parameters) == [
        "gate_up_proj", "scale_tensor", "swiglu_out", "next_buffer", "num_threads", "force_scalar"]
    assert list(inspect.signature(reference_swiglu).parameters) == ["gate_up_proj", "scale_tensor", "next_buffer"]
    assert list(inspect.signature(generate_swiglu_data).parameters)[:4] == ["rows", "hidden_dim", "buffer_cols", "seed"]
    assert list(inspect.signature(residual_rms).parameters)[:8] == [
        "input", "residual", "weight", "epsilon", "scale_tensor", "next_buffer", "num_threads", "force_scalar"]
    assert list(inspect.signature(_residual_rms).parameters) == [
        "input", "residual", "weight", "scale_tensor", "epsilon", "output", "next_buffer", "num_threads",
        "force_scalar"]
    for fn in (reference_residual_rms, precise_residual_rms):
        assert list(inspect.signature(fn).parameters) == [
            "input", "residual", "weight", "epsilon", "scale_tensor", "next_buffer"]
    assert list(inspect.signature(generate_residual_rms_data).parameters)[:5] == [
        "rows", "cols", "buffer_cols", "dtype", "seed"]
    assert list(inspect.signature(llama_mlp_combined_ops).parameters)[:12] == [
        "attn_output", "residual", "rms_weight", "rms_epsilon", "gate_up_weight", "gate_up_input_scale",
        "gate_up_output_scale", "down_weight", "down_input_scale", "down_output_scale", "gate_up_gemm_hp",
        "down_gemm_hp"]

    for name, text in (
        ("residual_rms", "_HFRK_C::residual_rms(Tensor input, Tensor! residual, Tensor weight, Tensor scale_tensor, "
                         "float epsilon, Tensor! output, Tensor! next_buffer, int num_threads, bool force_scalar) -> ()"),
        ("swiglu", "_HFRK_C::swiglu(Tensor gate_up, Tensor scale_tensor, Tensor! output, Tensor! next_buffer, "
                   "int num_threads, bool force_scalar) -> ()"),
    ):
        schema = getattr(torch.ops._HFRK_C, name).default._schema
        assert str(schema) == str(torch._C.parse_schema(text))


def test_elementwise_references_agree_with_the_oracle_on_cpu(pkg, oracle_mod):
    """The package's torch statements (used by the GPU tests as the reference's criteria) against
    the numpy oracle, which is pinned to the reference's outputs."""
    import numpy as np

    import elementwise_oracle as ew
    from hf_rocm_kernels.operators.residual_rms import (generate_residual_rms_data, precise_residual_rms,
                                                         reference_residual_rms)
    from hf_rocm_kernels.operators.swiglu import generate_swiglu_data, reference_swiglu

    f16 = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16).view(np.float16)
    gate_up, scale, buf = generate_swiglu_data(5, 520, 24, seed=1, device="cpu")
    buf.fill_(1)
    got = reference_swiglu(gate_up, scale, buf).view(torch.uint8).numpy()
    assert float(buf.abs().sum()) == 0
    assert np.array_equal(got, ew.reference_swiglu(f16(gate_up), 2 * float(scale)))

    x, res, w, eps, scale, _ = generate_residual_rms_data(4, 1024, 0, torch.float8_e4m3fnuz, seed=2, device="cpu")
    out, new_res, doubled = reference_residual_rms(x.clone(), res.clone(), w, eps, scale)
    expect, expect_res = ew.reference_residual_rms(f16(x), f16(res), f16(w), eps, 2 * float(scale), form="torch")
    assert float(doubled) == 2 * float(scale)
    assert np.array_equal(f16(new_res).view(np.uint16), expect_res.view(np.uint16))
    assert (ew.fp8_step_distance(out.view(torch.uint8).numpy(), expect) != 0).mean() < 2e-3
    precise, _ = precise_residual_rms(x.clone(), res.clone(), w, eps, scale)
    expect_p = ew.precise_residual_rms(f16(x), f16(res), f16(w), eps, 2 * float(scale))
    assert (ew.fp8_step_distance(precise.view(torch.uint8).numpy(), expect_p) != 0).mean() < 2e-3
    out16, _, none = reference_residual_rms(x.clone(), res.clone(), w, eps, None)
    assert none is None and out16.dtype == torch.float16


def test_elementwise_checks(pkg):
    from hf_rocm_kernels.operators.residual_rms.wrapped import infer_num_threads, residual_rms_checks
    from hf_rocm_kernels.operators.swiglu.wrapped import swiglu_checks

    g = torch.zeros((2, 64), dtype=torch.float16)
    with pytest.raises(AssertionError, match="cuda"):
        swiglu_checks(g, torch.ones(1), torch.empty((2, 0), dtype=torch.float16))
    with pytest.raises(AssertionError, match="even"):
        swiglu_checks(torch.zeros((2, 63), dtype=torch.float16), torch.ones(1), torch.empty((2, 0), dtype=torch.float16))
    with pytest.raises(AssertionError, match="rows"):
        swiglu_checks(g, torch.ones(1), torch.empty((3, 8), dtype=torch.float16))
    x = torch.zeros((2, 64), dtype=torch.float16)
    with pytest.raises(AssertionError, match="same shape"):
        residual_rms_checks(x, torch.zeros((2, 32), dtype=torch.float16), torch.ones(64, dtype=torch.float16), None,
                            1e-5, torch.empty((2, 0), dtype=torch.float16))
    with pytest.raises(AssertionError, match="weight"):
        residual_rms_checks(x, x, torch.ones(32, dtype=torch.float16), None, 1e-5,
                            torch.empty((2, 0), dtype=torch.float16))
    with pytest.raises(AssertionError, match="cuda"):
        residual_rms_checks(x, x, torch.ones(64, dtype=torch.float16), None, 1e-5,
                            torch.empty((2, 0), dtype=torch.float16))
    with pytest.raises(ValueError):
        infer_num_threads(4, 2048)
    assert infer_num_threads(4, 0) == 0 and infer_num_threads(4, 512) == 512


def test_checks_reject_what_the_reference_rejects(pkg):
    from hf_rocm_kernels.operators.skinny_gemm.wrapped import infer_skinny_gemm_params, skinny_gemm_checks

    a = torch.zeros((4, 256), dtype=torch.float8_e4m3fnuz)
    w = torch.zeros((128, 256), dtype=torch.float8_e4m3fnuz)
    s = torch.ones(1)
    d = torch.zeros((4, 128), dtype=torch.float16)
    with pytest.raises(AssertionError, match="cuda"):
        skinny_gemm_checks(a, w.t(), s, d)                       # CPU tensors
    with pytest.raises(AssertionError, match="column-major"):
        skinny_gemm_checks(a, torch.zeros((256, 128), dtype=torch.float8_e4m3fnuz), s, d)
    with pytest.raises(AssertionError):
        skinny_gemm_checks(a, w.t(), torch.ones(2), d)           # scale must hold one element
    with pytest.raises(AssertionError):
        skinny_gemm_checks(a, w.t(), s, torch.zeros((4, 64), dtype=torch.float16))
    with pytest.raises(AssertionError):
        skinny_gemm_checks(a.float(), w.t(), s, d)               # dtype
    with pytest.raises(AssertionError):
        skinny_gemm_checks(a, w.t(), s.double(), d)
    params = infer_skinny_gemm_params(a, w.t())
    assert set(params) == {"split_k", "A_producers", "B_producers", "consumers", "a_lanes", "b_lanes", "qsize",
                           "op_m", "ops"}
    assert params["split_k"] == 0 and params["op_m"] == 16


def test_compare_helpers():
    from hf_rocm_kernels.utils.testing import compare_x_and_ref_to_precise, compare_x_with_ref, skinny_gemm_tolerance

    ref = torch.tensor([1.0, 2.0, 0.0, -4.0])
    x = torch.tensor([1.0, 2.5, 0.0, -4.0])
    max_abs, max_rel, changed = compare_x_with_ref(x, ref)
    assert max_abs == 0.5 and max_rel == 0.25 and changed == 1
    with pytest.raises(ValueError):
        compare_x_with_ref(x, ref[:2])
    out = compare_x_and_ref_to_precise(x, ref, ref)
    assert out[0] == 0.5 and out[1] == 0.0 and out[4] == 25.0
    tol = skinny_gemm_tolerance(torch.tensor([1.0, 64.0]), 4096, 1e-4, torch.bfloat16)
    assert torch.allclose(tol, torch.tensor([2.0 ** -7, 0.5], dtype=torch.float64) + 6.4e-6)


def test_workload_configurations():
    from hf_rocm_kernels.benchmarks.skinny_gemm import workloads as wl

    assert [len(wl.cases(c)) for c in range(5)] == [1, 20, 12, 4, 45]
    c0 = wl.cases(0)[0]
    assert (c0.m, c0.n, c0.k, c0.bias) == (1, 4096, 4096, False) and c0.seed == 0
    assert {(c.n, c.k) for c in wl.cases(1)} == {(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)}
    assert all(c.bias == (c.n == 6144) for c in wl.cases(1))
    assert {(c.n, c.k) for c in wl.cases(2)} == {(10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672)}
    assert {c.m for c in wl.cases(3)} == {1, 2, 8, 16}
    edge = wl.cases(4)
    assert {c.m for c in edge} == {3, 5, 7, 13, 16} and all(c.outliers for c in edge)
    assert [c.bias for c in edge[:4]] == [True, False, True, False]
    case = wl.Case(4, 1, "t", 3, 136, 1040, bias=True, outliers=True)
    x, y = wl.make_inputs(case), wl.make_inputs(case)
    assert torch.equal(x["a"].view(torch.uint8), y["a"].view(torch.uint8))  # seeded
    assert x["a"].dtype == torch.float8_e4m3fn and x["d_in"].shape == (3, 136) and x["d_in"].dtype == torch.bfloat16
    saturated = (x["w"].view(torch.uint8) & 0x7F) == 0x7E
    assert 0.005 < saturated.float().mean() < 0.02                           # ~1 % outliers pinned at +-448
    assert torch.equal(x["scale"], x["scale_a"] * x["scale_w"])
    assert case.algorithmic_bytes() == 136 * 1040 + 3 * 1040 + 2 * (3 * 136 * 2) + 4
    assert wl.n_split_rows(10240, 8, 3) == (3840, 5120) and wl.k_split_cols(28672, 8, 7) == (25088, 28672)
    with pytest.raises(ValueError):
        wl.n_split_rows(1000, 3, 0)


def test_the_package_fails_loudly_without_its_native_library(native_build, tmp_path):
    """No CPU or PyTorch fallback: with the shared library out of reach the import raises and names
    the build command; with it in place but no GPU, the operators refuse CPU tensors."""
    import os
    import shutil
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "hf-rocm-kernels_b200", "hf_rocm_kernels")
    copy = tmp_path / "hf_rocm_kernels"
    shutil.copytree(src, copy, ignore=shutil.ignore_patterns("*.so", "__pycache__"))
    probe = ("import sys; sys.path.insert(0, sys.argv[1])\n"
             "try:\n    import hf_rocm_kernels\nexcept ImportError as e:\n    print('IMPORT_ERROR', e)\n"
             "else:\n    print('IMPORTED')\n")
    out = subprocess.run([sys.executable, "-c", probe, str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert "IMPORT_ERROR" in out.stdout, out.stdout + out.stderr

    from hf_rocm_kernels import residual_rms, skinny_gemm, swiglu

    a = torch.zeros((4, 256), dtype=torch.float8_e4m3fn)
    w = torch.zeros((128, 256), dtype=torch.float8_e4m3fn)
    with pytest.raises(AssertionError, match="cuda"):
        skinny_gemm(a, w.t(), torch.ones(1), torch.zeros((4, 128), dtype=torch.bfloat16))
    with pytest.raises(AssertionError, match="cuda"):
        swiglu(torch.zeros((2, 64), dtype=torch.float16), torch.ones(1))
    with pytest.raises(AssertionError, match="cuda"):
        residual_rms(torch.zeros((2, 64), dtype=torch.float16), torch.zeros((2, 64), dtype=torch.float16),
                     torch.ones(64, dtype=torch.float16), 1e-5)


def test_ops_can_be_traced_with_meta_tensors(pkg):
    """A tracer that runs the model on meta tensors must get through the four ops (they work in
    place on caller-allocated tensors, so the shape-only implementations do nothing)."""
    meta = torch.device("meta")
    a = torch.empty((4, 256), dtype=torch.float8_e4m3fn, device=meta)
    w = torch.empty((128, 256), dtype=torch.float8_e4m3fn, device=meta)
    d = torch.empty((4, 128), dtype=torch.bfloat16, device=meta)
    s = torch.empty(1, device=meta)
    assert torch.ops._HFRK_C.skinny_gemm_tb(a, w.t(), d, s, 0, 1, 1, 1, 1, 1, 12, 16, 4) == 0
    gate_up = torch.empty((4, 64), dtype=torch.float16, device=meta)
    out = torch.empty((4, 32), dtype=torch.float8_e4m3fnuz, device=meta)
    buf = torch.empty((4, 0), dtype=torch.float16, device=meta)
    assert torch.ops._HFRK_C.swiglu(gate_up, s, out, buf, 64, False) is None
    x = torch.empty((4, 64), dtype=torch.float16, device=meta)
    weight = torch.empty(64, dtype=torch.float16, device=meta)
    assert torch.ops._HFRK_C.residual_rms(x, x, weight, s, 1e-5, torch.empty_like(x), buf, 0, False) is None
    assert torch.ops._HFRK_C.increment(x) is None
