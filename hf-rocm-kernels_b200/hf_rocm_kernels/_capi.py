"""ctypes view of ``libhfrk_b200.so``, the C ABI declared in ``include/hfrk_b200.h``.

The torch op is a shim over the same library; this module lets benchmarks and tests reach the
entry points that have no torch schema (pinned launch shapes, host-buffer calls, the plan query).
There is no fallback: if the library is missing, importing this module raises.
"""
import ctypes
import os
from typing import Optional, Tuple

import torch

_LIB_NAME = "libhfrk_b200.so"
_PKG_DIR = os.path.dirname(os.path.abspath(__file__))

E4M3FN, E4M3FNUZ = 0, 1
F16, BF16, F32 = 0, 1, 2
VARIANT_AUTO, VARIANT_CLUSTER, VARIANT_STREAMK = 0, 1, 2
OUT_SAME, OUT_E4M3FN, OUT_E4M3FNUZ = 0, 1, 2
ROWPAR_AUTO, ROWPAR_ONE_SHOT, ROWPAR_TWO_SHOT = 0, 1, 2

STATUS_NAMES = {
    0: "SUCCESS", 1: "M_ABOVE_WARPTILE_M", 2: "N_NOT_EVEN", 3: "K_NOT_DIVISIBLE", 4: "TOO_MANY_WARPS",
    5: "QSIZE_TOO_SMALL", 6: "INVALID_CONFIG", 7: "BAD_ALIGNMENT", 8: "BAD_DTYPE", 9: "CUDA_ERROR",
    10: "DEVICE_TIMEOUT", 11: "BAD_WORLD", 12: "TOO_LARGE",
}

# Every symbol the header declares; tests check that the built library exports all of them.
EXPORTED_SYMBOLS = (
    "hfrk_skinny_gemm_fp8", "hfrk_skinny_gemm_fp8_ex", "hfrk_skinny_gemm_fp8_host",
    "hfrk_host_call_workspace_bytes", "hfrk_skinny_gemm_fp8_simt", "hfrk_skinny_gemm_plan",
    "hfrk_device_status", "hfrk_last_error", "hfrk_version", "hfrk_skinny_gemm_fp8_profile",
    "hfrk_rowpar_create", "hfrk_rowpar_ipc_handle", "hfrk_rowpar_connect", "hfrk_rowpar_connect_pointers",
    "hfrk_rowpar_local_block", "hfrk_rowpar_destroy", "hfrk_skinny_gemm_fp8_rowpar",
    "hfrk_skinny_gemm_fp8_noalloc", "hfrk_max_active_clusters", "hfrk_tuning_set", "hfrk_tuning_clear",
    "hfrk_swiglu_fp8", "hfrk_residual_rms", "hfrk_rowpar_set_mode",
    "hfrk_skinny_gemm_fp8_swiglu", "hfrk_skinny_gemm_fp8_host_async",
    "hfrk_tuning_set_ex", "hfrk_rowpar_set_wait_ms", "hfrk_device_model_get", "hfrk_device_model_override",
)


def library_path() -> str:
    return os.path.join(_PKG_DIR, _LIB_NAME)


def _load() -> ctypes.CDLL:
    path = library_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python hf-rocm-kernels_b200/build.py` "
            "(nvcc, sm_100a). This package has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(path)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    common = [vp, vp, vp, vp, i32, i32, i32, i64, i32, i32, i32, i32]
    lib.hfrk_skinny_gemm_fp8.argtypes = common + [i32, vp]
    lib.hfrk_skinny_gemm_fp8_ex.argtypes = common + [i32, i32, i32, i32, i32, vp]
    lib.hfrk_skinny_gemm_fp8_host.argtypes = common + [vp, vp]
    lib.hfrk_skinny_gemm_fp8_host_async.argtypes = common + [vp, vp]
    lib.hfrk_skinny_gemm_fp8_host_async.restype = i32
    lib.hfrk_skinny_gemm_fp8_profile.argtypes = common + [i32, i32, i32, i32, i32, vp, vp]
    lib.hfrk_skinny_gemm_fp8_profile.restype = i32
    lib.hfrk_rowpar_create.argtypes = [i32, i32, i32, i32, ctypes.POINTER(vp)]
    lib.hfrk_rowpar_ipc_handle.argtypes = [vp, vp]
    lib.hfrk_rowpar_connect.argtypes = [vp, vp]
    lib.hfrk_rowpar_connect_pointers.argtypes = [vp, ctypes.POINTER(vp)]
    lib.hfrk_rowpar_local_block.argtypes = [vp]
    lib.hfrk_rowpar_local_block.restype = vp
    lib.hfrk_rowpar_destroy.argtypes = [vp]
    lib.hfrk_rowpar_set_mode.argtypes = [vp, i32]
    lib.hfrk_rowpar_set_wait_ms.argtypes = [vp, i32]
    lib.hfrk_rowpar_set_wait_ms.restype = i32
    lib.hfrk_rowpar_set_mode.restype = i32
    lib.hfrk_rowpar_set_stamps.argtypes = [vp, vp]
    lib.hfrk_rowpar_set_stamps.restype = i32
    lib.hfrk_skinny_gemm_fp8_rowpar.argtypes = [vp] + common + [vp]
    for name in ("hfrk_rowpar_create", "hfrk_rowpar_ipc_handle", "hfrk_rowpar_connect",
                 "hfrk_rowpar_connect_pointers", "hfrk_rowpar_destroy", "hfrk_skinny_gemm_fp8_rowpar"):
        getattr(lib, name).restype = i32
    lib.hfrk_skinny_gemm_fp8_simt.argtypes = common + [vp]
    lib.hfrk_skinny_gemm_fp8_noalloc.argtypes = common + [vp]
    lib.hfrk_skinny_gemm_fp8_noalloc.restype = i32
    lib.hfrk_host_call_workspace_bytes.argtypes = [i32, i32, i32]
    lib.hfrk_host_call_workspace_bytes.restype = i64
    lib.hfrk_skinny_gemm_plan.argtypes = [i32, i32, i32, i32, i32, i32, ctypes.POINTER(i32)]
    lib.hfrk_device_status.argtypes = [i32, ctypes.POINTER(ctypes.c_uint)]
    lib.hfrk_max_active_clusters.argtypes = [i32, i32, ctypes.POINTER(i32)]
    lib.hfrk_max_active_clusters.restype = i32
    lib.hfrk_tuning_set.argtypes = [i32, i32, i32, i32, i32]
    lib.hfrk_tuning_set.restype = i32
    lib.hfrk_tuning_set_ex.argtypes = [i32, i32, i32, i32, i32, i32]
    lib.hfrk_tuning_set_ex.restype = i32
    lib.hfrk_tuning_clear.restype = i32
    lib.hfrk_device_model_get.argtypes = [ctypes.POINTER(i32), ctypes.POINTER(i32), ctypes.POINTER(i32)]
    lib.hfrk_device_model_get.restype = i32
    lib.hfrk_device_model_override.argtypes = [i32, ctypes.POINTER(i32)]
    lib.hfrk_device_model_override.restype = i32
    lib.hfrk_swiglu_fp8.argtypes = [vp, vp, vp, vp, i32, i32, i64, i32, i32, i32, vp]
    lib.hfrk_swiglu_fp8.restype = i32
    lib.hfrk_residual_rms.argtypes = [vp, vp, vp, vp, ctypes.c_float, vp, vp, i32, i32, i64, i32, i32, i32, i32, vp]
    lib.hfrk_residual_rms.restype = i32
    lib.hfrk_skinny_gemm_fp8_swiglu.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i32, i32, i32, i32, i64, vp]
    lib.hfrk_skinny_gemm_fp8_swiglu.restype = i32
    lib.hfrk_last_error.restype = ctypes.c_char_p
    for name in ("hfrk_skinny_gemm_fp8", "hfrk_skinny_gemm_fp8_ex", "hfrk_skinny_gemm_fp8_host",
                 "hfrk_skinny_gemm_fp8_simt", "hfrk_skinny_gemm_plan", "hfrk_device_status", "hfrk_version"):
        getattr(lib, name).restype = i32
    return lib


class HostCall(ctypes.Structure):
    """``hfrk_host_call`` of the header: one entry of a batch of host-buffer GEMM calls."""
    _fields_ = [("A_host", ctypes.c_void_p), ("W_dev", ctypes.c_void_p), ("D_host", ctypes.c_void_p),
                ("scale_dev", ctypes.c_void_p), ("m", ctypes.c_int), ("n", ctypes.c_int), ("k", ctypes.c_int),
                ("w_row_stride", ctypes.c_int64), ("a_kind", ctypes.c_int), ("w_kind", ctypes.c_int),
                ("d_dtype", ctypes.c_int), ("accumulate", ctypes.c_int), ("D_in_host", ctypes.c_void_p)]


lib = _load()
lib.hfrk_host_batch_workspace_bytes.argtypes = [ctypes.POINTER(HostCall), ctypes.c_int]
lib.hfrk_host_batch_workspace_bytes.restype = ctypes.c_int64
lib.hfrk_skinny_gemm_fp8_host_batch.argtypes = [ctypes.POINTER(HostCall), ctypes.c_int, ctypes.c_void_p, ctypes.c_int64,
                                                ctypes.c_void_p]
lib.hfrk_skinny_gemm_fp8_host_batch.restype = ctypes.c_int


class HfrkError(RuntimeError):
    def __init__(self, code: int):
        self.code = code
        detail = lib.hfrk_last_error().decode() if code == 9 else ""
        super().__init__(f"hfrk status {code} ({STATUS_NAMES.get(code, '?')}) {detail}".strip())


def check(code: int) -> None:
    if code != 0:
        raise HfrkError(code)


def fp8_kind(dtype: torch.dtype) -> int:
    if dtype == torch.float8_e4m3fn:
        return E4M3FN
    if dtype == torch.float8_e4m3fnuz:
        return E4M3FNUZ
    raise TypeError(f"expected float8_e4m3fn or float8_e4m3fnuz, got {dtype}")


def out_kind(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return F16
    if dtype == torch.bfloat16:
        return BF16
    if dtype == torch.float32:
        return F32
    raise TypeError(f"expected float16, bfloat16 or float32 output, got {dtype}")


def _common_args(a: torch.Tensor, w: torch.Tensor, d: torch.Tensor, scale: torch.Tensor, accumulate: bool):
    """(A[M,K], W[N,K] with unit inner stride, D[M,N], scale[1]) -> the leading C arguments."""
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and w.stride(1) == 1 and a.is_contiguous() and d.is_contiguous()
    assert tuple(d.shape) == (m, n) and scale.numel() == 1 and scale.dtype == torch.float32
    return (a.data_ptr(), w.data_ptr(), d.data_ptr(), scale.data_ptr(), m, n, k, w.stride(0),
            fp8_kind(a.dtype), fp8_kind(w.dtype), out_kind(d.dtype), int(accumulate))


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on_device(device: torch.device):
    """Context that makes ``device`` current; free when it already is (the usual case)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _stream_ptr(stream: Optional[torch.cuda.Stream], device: torch.device) -> int:
    return (stream or torch.cuda.current_stream(device)).cuda_stream


def skinny_gemm(a, w, d, scale, accumulate=True, split_k_hint=0, stream=None) -> int:
    """``hfrk_skinny_gemm_fp8`` on torch CUDA tensors; ``w`` is the [N,K] weight (rows may be padded)."""
    with torch.cuda.device(a.device):
        return lib.hfrk_skinny_gemm_fp8(*_common_args(a, w, d, scale, accumulate), split_k_hint,
                                        _stream_ptr(stream, a.device))


def skinny_gemm_ex(a, w, d, scale, accumulate=True, variant=VARIANT_AUTO, split_k=0, ctas_per_sm=0, num_stages=0,
                   use_pdl=False, stream=None) -> int:
    with torch.cuda.device(a.device):
        return lib.hfrk_skinny_gemm_fp8_ex(*_common_args(a, w, d, scale, accumulate), variant, split_k, ctas_per_sm,
                                           num_stages, int(use_pdl), _stream_ptr(stream, a.device))


def skinny_gemm_profile(a, w, d, scale, stamps, accumulate=True, variant=VARIANT_AUTO, split_k=0, ctas_per_sm=0,
                        num_stages=0, use_pdl=False, stream=None) -> int:
    """``hfrk_skinny_gemm_fp8_profile``: ``stamps`` is an int64 CUDA tensor of shape [ctas, 8]."""
    with torch.cuda.device(a.device):
        return lib.hfrk_skinny_gemm_fp8_profile(*_common_args(a, w, d, scale, accumulate), variant, split_k,
                                                ctas_per_sm, num_stages, int(use_pdl), stamps.data_ptr(),
                                                _stream_ptr(stream, a.device))


def skinny_gemm_simt(a, w, d, scale, accumulate=True, stream=None) -> int:
    with torch.cuda.device(a.device):
        return lib.hfrk_skinny_gemm_fp8_simt(*_common_args(a, w, d, scale, accumulate),
                                             _stream_ptr(stream, a.device))


def skinny_gemm_noalloc(a, w, d, scale, accumulate=True, stream=None) -> int:
    """``hfrk_skinny_gemm_fp8_noalloc``: the GEMM with its scratch in a fixed array of the library
    image, for callers that may not allocate device memory (m <= 16, n <= 524288)."""
    with torch.cuda.device(a.device):
        return lib.hfrk_skinny_gemm_fp8_noalloc(*_common_args(a, w, d, scale, accumulate),
                                                _stream_ptr(stream, a.device))


def skinny_gemm_host(a_host, w_dev, d_host, scale_dev, work_dev, accumulate=True, stream=None,
                     synchronise=True) -> int:
    """Host-buffer call: ``a_host``/``d_host`` are (pinned) CPU tensors, weights and scale stay on the
    GPU. With ``synchronise=False`` the copies and the GEMM are only queued on the stream
    (hfrk_skinny_gemm_fp8_host_async): ``d_host`` is valid after the caller synchronises it."""
    m, k = a_host.shape
    n = w_dev.shape[0]
    assert a_host.device.type == "cpu" and d_host.device.type == "cpu" and w_dev.stride(1) == 1
    assert work_dev.numel() * work_dev.element_size() >= lib.hfrk_host_call_workspace_bytes(m, n, k)
    entry = lib.hfrk_skinny_gemm_fp8_host if synchronise else lib.hfrk_skinny_gemm_fp8_host_async
    with _on_device(w_dev.device):
        return entry(
            a_host.data_ptr(), w_dev.data_ptr(), d_host.data_ptr(), scale_dev.data_ptr(), m, n, k, w_dev.stride(0),
            fp8_kind(a_host.dtype), fp8_kind(w_dev.dtype), out_kind(d_host.dtype), int(accumulate),
            work_dev.data_ptr(), _stream_ptr(stream, w_dev.device))


class HostBatch:
    """A fixed list of host-buffer GEMM calls, prepared once and queued with one library call per
    step (``hfrk_skinny_gemm_fp8_host_batch``). ``calls`` = [(a_host, w_dev, d_host, scale_dev, accumulate)] or
    [(a_host, w_dev, d_host, scale_dev, accumulate, d_in_host)]: with ``d_in_host`` (a read-only, bias-filled
    host tensor) D_in is read from there and ``d_host`` only receives the result. The tensors must outlive
    the object, the host ones should be page-locked."""

    def __init__(self, calls, device: torch.device):
        self.device = device
        self.array = (HostCall * len(calls))()
        self.keep = list(calls)
        for slot, call in zip(self.array, calls):
            a_host, w_dev, d_host, scale_dev, accumulate = call[:5]
            d_in_host = call[5] if len(call) > 5 else None
            m, k = a_host.shape
            n = w_dev.shape[0]
            assert a_host.device.type == "cpu" and d_host.device.type == "cpu" and w_dev.stride(1) == 1
            assert a_host.is_contiguous() and d_host.is_contiguous() and tuple(d_host.shape) == (m, n)
            slot.A_host, slot.W_dev, slot.D_host = a_host.data_ptr(), w_dev.data_ptr(), d_host.data_ptr()
            slot.scale_dev, slot.m, slot.n, slot.k = scale_dev.data_ptr(), m, n, k
            slot.w_row_stride, slot.a_kind, slot.w_kind = w_dev.stride(0), fp8_kind(a_host.dtype), fp8_kind(w_dev.dtype)
            slot.d_dtype, slot.accumulate = out_kind(d_host.dtype), int(accumulate)
            if d_in_host is not None:
                assert d_in_host.device.type == "cpu" and d_in_host.is_contiguous() and d_in_host.shape == d_host.shape
                assert d_in_host.dtype == d_host.dtype
                slot.D_in_host = d_in_host.data_ptr()
        self.work_bytes = lib.hfrk_host_batch_workspace_bytes(self.array, len(calls))
        assert self.work_bytes > 0, "invalid call in the batch"
        self.work = torch.empty(self.work_bytes, dtype=torch.uint8, device=device)

    def queue(self, stream: Optional[torch.cuda.Stream] = None) -> int:
        """Queues the whole batch; results are in the host buffers once ``stream`` is synchronised."""
        with _on_device(self.device):
            return lib.hfrk_skinny_gemm_fp8_host_batch(self.array, len(self.array), self.work.data_ptr(), self.work_bytes,
                                                       _stream_ptr(stream, self.device))


def swiglu(gate_up: torch.Tensor, scale: torch.Tensor, out: torch.Tensor, next_buffer: Optional[torch.Tensor] = None,
           force_scalar: bool = False, stream=None) -> int:
    """hfrk_swiglu_fp8 on torch tensors: gate_up [rows, 2*hidden] 16-bit, out [rows, hidden] fp8."""
    rows, two_hidden = gate_up.shape
    assert gate_up.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (rows, two_hidden // 2)
    buffer_cols = 0 if next_buffer is None or rows == 0 else next_buffer.numel() // rows
    with torch.cuda.device(gate_up.device):
        return lib.hfrk_swiglu_fp8(gate_up.data_ptr(), scale.data_ptr(), out.data_ptr(),
                                   0 if next_buffer is None else next_buffer.data_ptr(), rows, two_hidden // 2,
                                   buffer_cols, out_kind(gate_up.dtype), fp8_kind(out.dtype), int(force_scalar),
                                   _stream_ptr(stream, gate_up.device))


def skinny_gemm_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, act_out: torch.Tensor, scale: torch.Tensor,
                       act_scale: torch.Tensor, next_buffer: Optional[torch.Tensor] = None,
                       mid_dtype: torch.dtype = torch.bfloat16, stream=None) -> int:
    """hfrk_skinny_gemm_fp8_swiglu on torch tensors: a [m, k] fp8, w_gate_up [2*inter, k] fp8 with
    unit inner stride, act_out [m, inter] fp8."""
    m, k = a.shape
    inter = w_gate_up.shape[0] // 2
    assert w_gate_up.shape[1] == k and w_gate_up.stride(1) == 1 and a.is_contiguous() and act_out.is_contiguous()
    assert tuple(act_out.shape) == (m, inter) and w_gate_up.shape[0] == 2 * inter
    buffer_cols = 0 if next_buffer is None else next_buffer.numel() // m
    with torch.cuda.device(a.device):
        return lib.hfrk_skinny_gemm_fp8_swiglu(
            a.data_ptr(), w_gate_up.data_ptr(), act_out.data_ptr(), scale.data_ptr(), act_scale.data_ptr(),
            0 if next_buffer is None else next_buffer.data_ptr(), m, inter, k, w_gate_up.stride(0),
            fp8_kind(a.dtype), fp8_kind(w_gate_up.dtype), out_kind(mid_dtype), fp8_kind(act_out.dtype), buffer_cols,
            _stream_ptr(stream, a.device))


def residual_rms(input: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, scale: Optional[torch.Tensor],
                 epsilon: float, output: torch.Tensor, next_buffer: Optional[torch.Tensor] = None,
                 num_threads: int = 0, force_scalar: bool = False, stream=None) -> int:
    """hfrk_residual_rms on torch tensors; the output kind follows ``output.dtype``."""
    rows, cols = input.shape
    assert input.is_contiguous() and residual.is_contiguous() and weight.is_contiguous() and output.is_contiguous()
    kind = OUT_SAME if output.dtype == input.dtype else (OUT_E4M3FNUZ if fp8_kind(output.dtype) == E4M3FNUZ
                                                         else OUT_E4M3FN)
    buffer_cols = 0 if next_buffer is None or rows == 0 else next_buffer.numel() // rows
    with torch.cuda.device(input.device):
        return lib.hfrk_residual_rms(input.data_ptr(), residual.data_ptr(), weight.data_ptr(),
                                     0 if scale is None else scale.data_ptr(), epsilon, output.data_ptr(),
                                     0 if next_buffer is None else next_buffer.data_ptr(), rows, cols, buffer_cols,
                                     out_kind(input.dtype), kind, num_threads, int(force_scalar),
                                     _stream_ptr(stream, input.device))


def plan(m: int, n: int, k: int, variant: int = VARIANT_AUTO, split_k: int = 0, ctas_per_sm: int = 0) -> dict:
    out = (ctypes.c_int * 8)()
    check(lib.hfrk_skinny_gemm_plan(m, n, k, variant, split_k, ctas_per_sm, out))
    keys = ("variant", "split_k", "num_stages", "ctas", "smem_bytes", "m_pad", "k_blocks", "tiles")
    return dict(zip(keys, list(out)))


MODEL_MAX_SPLIT, MODEL_MAX_PER_SM = 16, 3


def device_model() -> dict:
    """``hfrk_device_model_get``: SM count and ``capacity[split][ctas_per_sm]`` (clusters resident at once)."""
    sms, measured = ctypes.c_int(0), ctypes.c_int(0)
    flat = (ctypes.c_int * ((MODEL_MAX_SPLIT + 1) * (MODEL_MAX_PER_SM + 1)))()
    check(lib.hfrk_device_model_get(ctypes.byref(sms), flat, ctypes.byref(measured)))
    cap = [[flat[s * (MODEL_MAX_PER_SM + 1) + p] for p in range(MODEL_MAX_PER_SM + 1)] for s in range(MODEL_MAX_SPLIT + 1)]
    return {"sms": sms.value, "measured": bool(measured.value), "capacity": cap}


def override_device_model(sms: int = 0, capacity=None) -> None:
    """``hfrk_device_model_override``; ``capacity[split][ctas_per_sm]`` or None to drop the override."""
    if capacity is None:
        check(lib.hfrk_device_model_override(0, None))
        return
    flat = (ctypes.c_int * ((MODEL_MAX_SPLIT + 1) * (MODEL_MAX_PER_SM + 1)))()
    for s in range(MODEL_MAX_SPLIT + 1):
        for p in range(MODEL_MAX_PER_SM + 1):
            flat[s * (MODEL_MAX_PER_SM + 1) + p] = int(capacity[s][p])
    check(lib.hfrk_device_model_override(sms, flat))


def max_active_clusters(split: int, smem_bytes: int) -> int:
    out = ctypes.c_int(0)
    check(lib.hfrk_max_active_clusters(split, smem_bytes, ctypes.byref(out)))
    return out.value


def device_status(clear: bool = True) -> Tuple[int, int]:
    word = ctypes.c_uint(0)
    code = lib.hfrk_device_status(int(clear), ctypes.byref(word))
    return code, word.value
