"""Shared pytest set-up: import paths, the ``gpu`` marker, and a one-off build of the native code.

Tests marked ``gpu`` are the parity tests proper (CUDA path vs the CPU oracle, through the C ABI);
everything else runs on a machine without a GPU.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for path in (ROOT, os.path.join(ROOT, "hf-rocm-kernels_b200"), os.path.join(ROOT, "oracle")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def native_build():
    """Builds libhfrk_b200.so, _HFRK_C.so and the C oracle if they are missing or stale."""
    import __graft_entry__

    __graft_entry__.build()


@pytest.fixture(scope="session")
def oracle_mod(native_build):
    import oracle

    return oracle


@pytest.fixture(scope="session")
def c_oracle(oracle_mod):
    return oracle_mod.load_c_oracle()


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


def pytest_sessionfinish(session, exitstatus):
    """With HFRK_PARITY_SUMMARY=<path>: one JSON line per parity case that the GPU tests checked
    (elements, how many lie beyond the stated bound, how many beyond bound + floor, worst ratio)."""
    path = os.environ.get("HFRK_PARITY_SUMMARY")
    module = sys.modules.get("test_gpu_parity")
    if not path or module is None or not getattr(module, "PARITY_ROWS", None):
        return
    import json

    with open(path, "w") as fh:
        for row in module.PARITY_ROWS:
            fh.write(json.dumps(row) + "\n")
