"""Every benchmark command of the package runs to the end on a small case (so that the commands
quoted in the documentation keep working). Needs a B200; checks exit codes and that the
expected table or JSON comes out, not the numbers."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "hf-rocm-kernels_b200")

COMMANDS = [
    ("hf_rocm_kernels.benchmarks.skinny_gemm.no_knobs", ["--m", "4", "--n", "1024", "--k", "1024", "--iterations", "4"],
     "us"),
    ("hf_rocm_kernels.benchmarks.skinny_gemm.no_knobs", ["--m", "4", "--n", "1024", "--k", "1024", "--plain-calls", "2"],
     "checksum"),
    ("hf_rocm_kernels.benchmarks.skinny_gemm.all_knobs",
     ["--m", "4", "--n", "1024", "--k", "1024", "--split-k", "2", "--stages", "3", "--iterations", "4"], "us"),
    ("hf_rocm_kernels.benchmarks.skinny_gemm.row_parallel", ["--tokens", "4", "--n", "1024", "--k", "2048"],
     "fused one-shot"),
    ("hf_rocm_kernels.benchmarks.skinny_gemm.row_parallel", ["--tokens", "4", "-n", "1024", "-k", "2048",   # as under torchrun
                                                             "--plain-calls", "2"], "fused calls of m=4"),
    ("hf_rocm_kernels.benchmarks.swiglu.vs_reference", ["-r", "1", "16", "-i", "1024", "-b", "256"], "Vectorized"),
    ("hf_rocm_kernels.benchmarks.residual_rms.vs_reference", ["-r", "1", "16", "-c", "1024", "-b", "256"], "Vectorized"),
    ("hf_rocm_kernels.benchmarks.residual_rms.vs_reference", ["-r", "4", "-c", "1024", "--fp16-output"], "Vectorized"),
    ("hf_rocm_kernels.benchmarks.residual_rms.nb_threads", ["-r", "4", "-c", "2048", "-t", "0", "128", "256"], "threads"),
    ("hf_rocm_kernels.benchmarks.swiglu.vs_vllm", ["-r", "4", "-i", "1024"], "Ours (us)"),
    ("hf_rocm_kernels.benchmarks.residual_rms.vs_vllm", ["-r", "4", "-c", "1024"], "Ours (us)"),
    ("hf_rocm_kernels.benchmarks.llama_mlp.block", ["--tokens", "4", "--hidden", "1024", "--intermediate", "2048"],
     "four launches"),
    ("hf_rocm_kernels.benchmarks.llama_mlp.block", ["--tokens", "4", "--hidden", "1024", "--intermediate", "2048",
                                                    "--plain-calls", "2"], "blocks of 4 tokens run"),
]


@pytest.mark.parametrize("module,args,expect", COMMANDS, ids=[f"{c[0].split('.')[-2]}.{c[0].split('.')[-1]}-{i}"
                                                              for i, c in enumerate(COMMANDS)])
def test_benchmark_command_runs(native_build, module, args, expect):
    env = dict(os.environ, PYTHONPATH=PKG + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-m", module] + args, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert expect in proc.stdout, proc.stdout[-2000:]


def test_grid_search_writes_a_table_the_loader_accepts(native_build, tmp_path):
    out = tmp_path / "tuning.json"
    env = dict(os.environ, PYTHONPATH=PKG + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-m", "hf_rocm_kernels.benchmarks.skinny_gemm.grid_search", "--shapes",
                           "1024x2048", "--m", "16", "--iterations", "3", "--warmups", "2", "--out", str(out)],
                          env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    from hf_rocm_kernels.operators.skinny_gemm import tuning

    try:
        assert tuning.load_tuning(str(out)) >= 1
    finally:
        tuning.clear_tuning()


def test_general_timing_function_and_device_check(native_build):
    """benchmark_skinny_gemm_general (the reference's hand-knob timing entry point) with the
    operator and with torch._scaled_mm (split_k = 0), and Bench.check_device_is_free."""
    from hf_rocm_kernels.operators.skinny_gemm.benchmarking_fn import benchmark_skinny_gemm_general
    from hf_rocm_kernels.utils.benchmarking import Bench

    ours, _ = benchmark_skinny_gemm_general(4, 1024, 1024, split_k=2, A_producers=1, B_producers=2, consumers=3,
                                            a_lanes=1, b_lanes=2, qsize=3, op_m=8, ops=4, warmups=2, iterations=4)
    vendor, _ = benchmark_skinny_gemm_general(16, 1024, 1024, split_k=0, warmups=2, iterations=4)
    assert 0.5 < ours < 1000 and 0.5 < vendor < 1000
    metrics = Bench.check_device_is_free()
    assert set(metrics) == {"utilization", "memory_usage"}
