"""The C ABI without a GPU: the library loads, exports what the header declares, plans launch
shapes, and rejects bad arguments before it touches CUDA."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "hfrk_b200.h")


@pytest.fixture(scope="module")
def capi(native_build):
    from hf_rocm_kernels import _capi

    return _capi


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hfrk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(capi):
    names = declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(capi.lib, name), f"{name} is declared in hfrk_b200.h but not exported"
    assert set(capi.EXPORTED_SYMBOLS) <= set(names)


def test_header_cites_the_reference_for_each_entry_point():
    text = open(HEADER).read()
    assert "skinny_gemm_binding.cu:16-42" in text and "skinny_gemm_caller.cu" in text
    assert "swiglu_dispatch.cu:8-42" in text and "residual_rms_dispatch.cu:8-63" in text
    assert "torch" not in re.sub(r"/\*.*?\*/", "", text, flags=re.S)  # no torch types in signatures


def test_version(capi):
    assert capi.lib.hfrk_version() >= 100
    assert capi.lib.hfrk_last_error() is not None


def _fake_capacity(sms, gpc_sizes):
    """Clusters resident at once on an imagined chip whose SMs sit in GPCs of the given sizes: a cluster
    needs all its CTA slots inside one GPC."""
    assert sum(gpc_sizes) == sms
    return [[0] * 4] + [[0] + [sum((g * per_sm) // split for g in gpc_sizes) for per_sm in (1, 2, 3)]
                        for split in range(1, 17)]


GRADED_SHAPES = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336),
                 (10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672)]


def _shards():
    out = list(GRADED_SHAPES)
    for g in (2, 4, 8):
        out += [(n // g, k) for (n, k) in GRADED_SHAPES[4:]]          # N split of the 70B projections
        out.append((8192, 28672 // g))                               # K split of the 70B down projection
    return out


@pytest.mark.parametrize("gpcs", [[20, 20, 20, 20, 18, 18, 16, 16], [18] * 6 + [20, 20], [16] * 8 + [20], [10] * 14 + [8]])
def test_every_graded_plan_is_resident_on_any_chip_layout(capi, gpcs):
    """The planner never asks for more clusters than the device holds at once, whatever the spread of
    the SMs over the GPCs: the capacity table is injected, so this runs without a GPU."""
    sms = sum(gpcs)
    cap = _fake_capacity(sms, gpcs)
    capi.override_device_model(sms, cap)
    try:
        for (n, k) in _shards():
            for m in (1, 16, 17, 64):
                p = capi.plan(m, n, k)
                assert p["ctas"] == p["tiles"] * p["split_k"]
                per_sm = min(3, (228 * 1024) // (p["smem_bytes"] + 1024))
                assert per_sm >= 1
                if p["split_k"] > 1:
                    assert p["tiles"] < cap[p["split_k"]][per_sm], (gpcs, m, n, k, p)
                    assert p["k_blocks"] // p["split_k"] >= 2
                    assert p["tiles"] < sms
                else:
                    assert p["tiles"] >= sms or p["k_blocks"] < 4 or cap[2][per_sm] < p["tiles"]
    finally:
        capi.override_device_model(capacity=None)


def test_plan_follows_the_device_model(capi):
    gpcs = [20, 20, 20, 20, 18, 18, 16, 16]
    cap = _fake_capacity(148, gpcs)
    capi.override_device_model(148, cap)
    try:
        # fewer tiles than SMs -> the largest K split whose clusters are all resident at once
        for (m, n, k) in [(16, 4096, 4096), (16, 6144, 4096), (16, 4096, 14336), (16, 8192, 8192), (1, 8192, 28672)]:
            p = capi.plan(m, n, k)
            assert p["variant"] == capi.VARIANT_CLUSTER and p["tiles"] == (n + 127) // 128
            assert p["split_k"] >= 4 and 148 <= p["ctas"] <= 3 * 148
        # one cluster fewer fits -> a smaller split (or a longer ring with fewer CTAs per SM), never a spill
        tight = [row[:] for row in cap]
        p0 = capi.plan(16, 4096, 4096)
        per_sm0 = min(3, (228 * 1024) // (p0["smem_bytes"] + 1024))
        tight[p0["split_k"]][per_sm0] = p0["tiles"]
        capi.override_device_model(148, tight)
        p1 = capi.plan(16, 4096, 4096)
        assert (p1["split_k"], p1["num_stages"]) != (p0["split_k"], p0["num_stages"])
        per_sm1 = min(3, (228 * 1024) // (p1["smem_bytes"] + 1024))
        assert p1["tiles"] < tight[p1["split_k"]][per_sm1]
        capi.override_device_model(148, cap)
        # enough tiles -> no split; six stages, or three when three CTAs per SM save a wave
        assert capi.plan(16, 28672, 4096)["split_k"] == 1 and capi.plan(16, 28672, 4096)["num_stages"] == 6
        assert capi.plan(4, 57344, 8192)["split_k"] == 1 and capi.plan(4, 57344, 8192)["num_stages"] == 3
        # between one and two CTAs per SM without a split: shorter tiles (a multiple of 8 rows) even out the load
        p = capi.plan(16, 28672, 4096)
        assert 224 < p["tiles"] <= 296 and capi.plan(4, 57344, 8192)["tiles"] == 448
        assert capi.plan(17, 28672, 4096)["tiles"] == 224           # more than 16 tokens: 128-row tiles
        # a chip with fewer SMs gets fewer CTAs
        capi.override_device_model(74, _fake_capacity(74, [20, 18, 18, 18]))
        assert capi.plan(16, 4096, 4096)["ctas"] <= 3 * 74
    finally:
        capi.override_device_model(capacity=None)
    # More than 16 tokens, with the capacities measured on one B200: candidates (largest resident split of a
    # ring of 2, 3 and 4 stages) are ranked by bytes in flight, marked down when an owner finishes more than 8
    # token rows; equal scores go to more CTAs.
    measured = _fake_capacity(148, gpcs)
    for split, caps in {8: (15, 33, 48), 7: (15, 37, 56), 6: (22, 45, 71), 5: (26, 56, 82), 4: (33, 71, 104)}.items():
        measured[split] = [0] + list(caps)
    for split in range(9, 17):
        measured[split] = [0, 7, 14, 21]
    capi.override_device_model(148, measured)
    try:
        picks = {(48, 8192, 8192): (6, 2), (32, 8192, 8192): (4, 4), (32, 6144, 4096): (5, 4), (48, 6144, 4096): (7, 2),
                 (24, 10240, 8192): (3, 4), (32, 10240, 8192): (5, 2), (64, 4096, 4096): (8, 3), (64, 6144, 4096): (4, 3)}
        for (m, n, k), (split, stages) in picks.items():
            p = capi.plan(m, n, k)
            assert (p["split_k"], p["num_stages"]) == (split, stages), ((m, n, k), p)
        # up to 16 tokens the rule is unchanged: more CTAs win, the table pins the Llama-3 shapes
        assert (capi.plan(16, 4096, 4096)["split_k"], capi.plan(16, 4096, 4096)["num_stages"]) == (7, 5)
        assert (capi.plan(16, 6144, 4096)["split_k"], capi.plan(16, 6144, 4096)["num_stages"]) == (7, 3)
    finally:
        capi.override_device_model(capacity=None)
    model = capi.device_model()
    assert model["sms"] >= 1 and len(model["capacity"]) == 17
    try:
        assert capi.lib.hfrk_tuning_set_ex(16, 4096, 4096, 0, 0, 64) == 0
        assert capi.plan(16, 4096, 4096)["tiles"] == 64
        assert capi.lib.hfrk_tuning_set_ex(16, 4096, 4096, 0, 0, 129) == 6
        assert capi.lib.hfrk_tuning_set_ex(16, 4096, 4096, 0, 0, 4) == 6
        assert capi.lib.hfrk_tuning_set_ex(16, 4096, 4096, 0, 0, 0) == 0     # drops the entry
        assert capi.plan(16, 4096, 4096)["tiles"] == 32
    finally:
        capi.lib.hfrk_tuning_clear()
    # K tails and odd N round up; token padding is a multiple of 16
    p = capi.plan(5, 1000, 1040)
    assert p["tiles"] == 8 and p["k_blocks"] == 9 and p["m_pad"] == 16
    assert capi.plan(17, 1024, 1024)["m_pad"] == 32 and capi.plan(200, 1024, 1024)["m_pad"] == 64
    # a requested split is honoured up to the number of K blocks
    assert capi.plan(16, 4096, 4096, capi.VARIANT_CLUSTER, 3)["split_k"] == 3
    assert capi.plan(16, 4096, 256, capi.VARIANT_CLUSTER, 16)["split_k"] == 2
    # stream-K covers the SMs once or twice and never launches idle CTAs
    sk = capi.plan(16, 4096, 4096, capi.VARIANT_STREAMK, 0, 2)
    assert sk["ctas"] == 296 and sk["variant"] == capi.VARIANT_STREAMK
    assert capi.plan(16, 4096, 4096, capi.VARIANT_STREAMK, 0, 1)["ctas"] == 148
    assert capi.plan(4, 128, 256, capi.VARIANT_STREAMK)["ctas"] == 2


def test_tuning_table_overrides_the_rule_per_shape(capi, tmp_path):
    import json

    from hf_rocm_kernels.operators.skinny_gemm import tuning

    base = capi.plan(16, 4096, 4096)
    path = tmp_path / "tuning.json"
    path.write_text(json.dumps({"entries": [{"m": 16, "n": 4096, "k": 4096, "split_k": 4, "num_stages": 6},
                                            {"m": 16, "n": 0, "k": 4096, "split_k": 4, "num_stages": 6}]}))
    try:
        assert tuning.load_tuning(str(path)) == 1                       # the malformed entry is refused
        pinned = capi.plan(16, 4096, 4096)
        assert (pinned["split_k"], pinned["num_stages"]) == (4, 6)
        assert capi.plan(3, 4096, 4096)["split_k"] == 4                  # token counts share an entry per 16
        assert capi.plan(17, 4096, 4096)["split_k"] == capi.plan(17, 4096, 4096, capi.VARIANT_CLUSTER, 0)["split_k"]
        assert capi.plan(16, 4096, 4096, capi.VARIANT_CLUSTER, 2)["split_k"] == 2   # an explicit request still wins
        assert capi.plan(16, 6144, 4096) == capi.plan(16, 6144, 4096)
        assert capi.lib.hfrk_tuning_set(16, 4096, 4096, 0, 0) == 0       # drop the entry
        assert capi.plan(16, 4096, 4096) == base
        assert capi.lib.hfrk_tuning_set(16, 4096, 4096, 17, 4) == 6
    finally:
        tuning.clear_tuning()


def test_plan_invariants_over_many_shapes(capi):
    """Whatever the shape, a plan is launchable: the grid covers N, every CTA has K blocks to do,
    the ring fits in shared memory, and the token padding matches the MMA."""
    import random

    rng = random.Random(11)
    shapes = [(rng.randint(1, 64), rng.randint(1, 70000), 16 * rng.randint(1, 2048)) for _ in range(400)]
    shapes += [(m, n, k) for m in (1, 16, 17, 64) for n in (1, 127, 128, 129, 18944, 19072, 37888) for k in (16, 128, 4096)]
    model = capi.device_model()
    for m, n, k in shapes:
        p = capi.plan(m, n, k)
        rows = -(-n // p["tiles"])                       # tile height the grid implies
        assert 1 <= rows <= 128 and p["tiles"] * rows >= n and (p["tiles"] - 1) * rows < n, (m, n, k, p)
        assert p["ctas"] == p["tiles"] * p["split_k"] and 1 <= p["split_k"] <= 16
        assert p["split_k"] <= p["k_blocks"] == -(-k // 128)
        assert 2 <= p["num_stages"] <= 12 and p["smem_bytes"] <= 227 * 1024
        assert p["m_pad"] == 16 * (-(-m // 16))
        if p["split_k"] > 1:
            # a split grid must be resident at once (three CTAs per SM at most, by the device model)
            per_sm = min(3, (228 * 1024) // (p["smem_bytes"] + 1024))
            assert p["tiles"] < model["capacity"][p["split_k"]][per_sm], (m, n, k, p)


def test_plan_rejects_bad_arguments(capi):
    out = (ctypes.c_int * 8)()
    assert capi.lib.hfrk_skinny_gemm_plan(0, 128, 128, 0, 0, 0, out) == 6
    assert capi.lib.hfrk_skinny_gemm_plan(16, 128, 128, 7, 0, 0, out) == 6
    assert capi.lib.hfrk_skinny_gemm_plan(16, 128, 128, 1, 99, 0, out) == 6
    assert capi.lib.hfrk_skinny_gemm_plan(16, 128, 128, 0, 0, 0, None) == 6


def test_argument_validation_happens_before_any_cuda_call(capi):
    """Host tensors stand in for device buffers: every call below must be refused on its
    arguments alone (a launch would fail differently, with CUDA_ERROR)."""
    a = torch.zeros((4, 256), dtype=torch.uint8)
    w = torch.zeros((128, 256), dtype=torch.uint8)
    d = torch.zeros((4, 128), dtype=torch.float16)
    s = torch.ones(1, dtype=torch.float32)
    call = capi.lib.hfrk_skinny_gemm_fp8
    base = [a.data_ptr(), w.data_ptr(), d.data_ptr(), s.data_ptr()]
    assert call(*base, 0, 128, 256, 256, 0, 0, 0, 1, 0, None) == 6          # m <= 0
    assert call(*base, 4, 128, 250, 256, 0, 0, 0, 1, 0, None) == 3          # k % 16
    assert call(*base, 4, 128, 256, 200, 0, 0, 0, 1, 0, None) == 7          # pitch < k
    assert call(*base, 4, 128, 256, 264, 0, 0, 0, 1, 0, None) == 7          # pitch % 16
    assert call(*base, 4, 128, 256, 256, 2, 0, 0, 1, 0, None) == 8          # fp8 kind
    assert call(*base, 4, 128, 256, 256, 0, 0, 5, 1, 0, None) == 8          # output dtype
    assert call(*base, 4, 128, 256, 256, 0, 0, 0, 1, -1, None) == 6         # split hint
    assert call(a.data_ptr() + 1, *base[1:], 4, 128, 256, 256, 0, 0, 0, 1, 0, None) == 7  # alignment
    assert call(None, *base[1:], 4, 128, 256, 256, 0, 0, 0, 1, 0, None) == 6
    assert capi.lib.hfrk_skinny_gemm_fp8_simt(*base, 4, 128, 250, 256, 0, 0, 0, 1, None) == 3
    assert capi.lib.hfrk_host_call_workspace_bytes(4, 128, 256) == 1024 + 2048
    assert capi.lib.hfrk_host_call_workspace_bytes(0, 128, 256) == 0


def test_elementwise_argument_validation_happens_before_any_cuda_call(capi):
    x = torch.zeros((2, 64), dtype=torch.float16)
    w = torch.ones(64, dtype=torch.float16)
    out = torch.zeros((2, 64), dtype=torch.uint8)
    s = torch.ones(1, dtype=torch.float32)
    swiglu = capi.lib.hfrk_swiglu_fp8
    assert swiglu(x.data_ptr(), s.data_ptr(), out.data_ptr(), None, 0, 32, 0, capi.F16, capi.E4M3FN, 0, None) == 0
    assert swiglu(x.data_ptr(), s.data_ptr(), out.data_ptr(), None, 2, 32, 0, capi.F32, capi.E4M3FN, 0, None) == 8
    assert swiglu(x.data_ptr(), s.data_ptr(), out.data_ptr(), None, 2, 32, 0, capi.F16, 3, 0, None) == 8
    assert swiglu(x.data_ptr(), None, out.data_ptr(), None, 2, 32, 0, capi.F16, capi.E4M3FN, 0, None) == 6
    assert swiglu(x.data_ptr(), s.data_ptr(), out.data_ptr(), None, 2, 32, 16, capi.F16, capi.E4M3FN, 0, None) == 6
    assert swiglu(x.data_ptr() + 1, s.data_ptr(), out.data_ptr(), None, 2, 16, 0, capi.F16, capi.E4M3FN, 0, None) == 7
    rms = capi.lib.hfrk_residual_rms
    ptrs = (x.data_ptr(), x.data_ptr(), w.data_ptr())
    assert rms(*ptrs, None, 1e-5, out.data_ptr(), None, 0, 64, 0, capi.F16, capi.OUT_SAME, 0, 0, None) == 0
    assert rms(*ptrs, None, -1.0, out.data_ptr(), None, 2, 64, 0, capi.F16, capi.OUT_SAME, 0, 0, None) == 6
    assert rms(*ptrs, None, 1e-5, out.data_ptr(), None, 2, 64, 0, capi.F16, capi.OUT_E4M3FNUZ, 0, 0, None) == 6
    assert rms(*ptrs, None, 1e-5, out.data_ptr(), None, 2, 64, 0, capi.F32, capi.OUT_SAME, 0, 0, None) == 8
    assert rms(*ptrs, None, 1e-5, out.data_ptr(), None, 2, 64, 0, capi.F16, 3, 0, 0, None) == 8
    assert rms(x.data_ptr() + 1, *ptrs[1:], None, 1e-5, out.data_ptr(), None, 2, 32, 0, capi.F16, capi.OUT_SAME, 0, 0,
               None) == 7


def test_status_names_cover_the_header(capi):
    text = open(HEADER).read()
    codes = dict((int(v), k) for k, v in re.findall(r"HFRK_([A-Z_0-9]+) = (\d+)", text.split("enum hfrk_fp8_kind")[0]))
    for code, name in codes.items():
        assert capi.STATUS_NAMES[code] == name


def test_a_plain_c_program_links_against_the_library(capi, tmp_path):
    """The boundary is C: the header compiles as C99 and a C program with no C++ runtime of its own
    links the shared library and calls it (the calls chosen need no GPU)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    source = tmp_path / "caller.c"
    source.write_text(
        '#include <stdio.h>\n#include "hfrk_b200.h"\n'
        "int main(void) {\n"
        "    int plan[8];\n"
        "    int rc = hfrk_skinny_gemm_plan(16, 4096, 4096, HFRK_VARIANT_AUTO, 0, 0, plan);\n"
        '    printf("%d %d %d %d %s\\n", hfrk_version(), rc, plan[1], plan[3], hfrk_last_error());\n'
        "    return rc == HFRK_SUCCESS ? 0 : 1;\n"
        "}\n")
    lib_dir = os.path.dirname(capi.library_path())
    exe = tmp_path / "caller"
    build = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-I", os.path.dirname(HEADER), str(source),
                            "-o", str(exe), "-L", lib_dir, "-l:libhfrk_b200.so", f"-Wl,-rpath,{lib_dir}"],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, run.stderr
    version, rc, split, ctas = run.stdout.split()[:4]
    assert int(version) == capi.lib.hfrk_version() and int(rc) == 0
    assert int(split) == capi.plan(16, 4096, 4096)["split_k"] and int(ctas) == capi.plan(16, 4096, 4096)["ctas"]
