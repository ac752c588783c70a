"""Per-shape launch tuning for ``skinny_gemm``.

The reference keeps a hand-written table of tuned parameters per (n, k) and token bucket inside
``infer_skinny_gemm_params`` (``operators/skinny_gemm/wrapped.py:42-102``). Here the table is data:
the grid search (``benchmarks/skinny_gemm/grid_search.py``) writes a JSON file, and this module
loads it into the library, which consults it before its built-in rule. B200 chips differ in how
their SMs are spread over the GPCs, and with it the largest cluster shape that is resident at
once, so a table measured on the deployment's own GPUs can beat the rule by a few percent.

File format: ``{"entries": [{"m": 16, "n": 4096, "k": 4096, "split_k": 8, "num_stages": 4}, ...]}``;
an entry may also carry ``"tile_rows"`` (W rows per CTA, 8..128; absent or 0 = the built-in rule).
Set ``HFRK_TUNING_FILE`` to have it loaded when the operator is imported.
"""
import json
import os
from typing import Dict, Iterable, List

from hf_rocm_kernels import _capi


def apply_tuning(entries: Iterable[Dict[str, int]]) -> int:
    """Pins every entry; returns how many were accepted."""
    accepted = 0
    for e in entries:
        code = _capi.lib.hfrk_tuning_set_ex(int(e["m"]), int(e["n"]), int(e["k"]), int(e.get("split_k", 0)),
                                            int(e.get("num_stages", 0)), int(e.get("tile_rows", 0)))
        accepted += int(code == 0)
    return accepted


def load_tuning(path: str) -> int:
    with open(path) as fh:
        data = json.load(fh)
    entries: List[Dict[str, int]] = data["entries"] if isinstance(data, dict) else data
    return apply_tuning(entries)


def clear_tuning() -> None:
    _capi.lib.hfrk_tuning_clear()


def load_from_environment() -> int:
    path = os.environ.get("HFRK_TUNING_FILE")
    return load_tuning(path) if path else 0
