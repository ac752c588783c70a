"""Row-parallel (K split across GPUs) skinny GEMM with the all-reduce fused into its epilogue.

The benchmark specification places a "GEMM + allreduce" in ``combined_ops`` of the reference; the
reference tree itself has no collective anywhere (``combined_ops/llama_mlp.py`` is a single-GPU
chain), so there is nothing to mirror: this file defines the multi-GPU surface. One process per
GPU, ``torch.distributed`` for the plumbing (the 64-byte IPC handles of the exchange buffers are
all-gathered once through the process group); the data path is the kernel itself, which writes
fp32 partial tiles into the peers' buffers over NVLink and adds them in rank order.

``skinny_gemm_then_allreduce`` is the unfused baseline: fp32 partials from the single-GPU kernel,
an NCCL all-reduce, then scale/bias/cast as torch ops.
"""
import ctypes
from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor

from hf_rocm_kernels import _capi


class RowParallelSkinnyGemm:
    """``out = D_in + scale * sum_r (A_r @ W_r.T)`` on every rank of ``group``.

    Rank r passes its K shard: ``a_shard [M, K/world]`` (contiguous) and ``w_shard [N, K/world]``
    (unit inner stride; a column slice of the full weight works, its row pitch is kept). ``output``
    must hold the same values (zeros or the bias) on every rank and receives the full result on
    every rank. All ranks must make the same sequence of calls. ``max_m``/``max_n`` size the
    exchange buffer (``16 * (world + 1) * min(max_m, 16) * max_n`` bytes per rank).
    """

    def __init__(self, max_m: int, max_n: int, group: Optional[dist.ProcessGroup] = None,
                 device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _capi.check(_capi.lib.hfrk_rowpar_create(self.rank, self.world, max_m, max_n, ctypes.byref(handle)))
            self._handle = handle
            if self.world > 1:
                mine = (ctypes.c_ubyte * 64)()
                _capi.check(_capi.lib.hfrk_rowpar_ipc_handle(self._handle, mine))
                gathered = [None] * self.world
                dist.all_gather_object(gathered, bytes(mine), group=group)
                blob = b"".join(gathered)
                _capi.check(_capi.lib.hfrk_rowpar_connect(self._handle, blob))
                dist.barrier(group=group)

    def __call__(self, a_shard: Tensor, w_shard: Tensor, scale_tensor: Tensor, output: Tensor,
                 accumulate: bool = True, stream: Optional[torch.cuda.Stream] = None) -> Tensor:
        m, k_shard = a_shard.shape
        n = w_shard.shape[0]
        assert w_shard.shape[1] == k_shard and w_shard.stride(1) == 1 and a_shard.is_contiguous()
        assert output.is_contiguous() and tuple(output.shape) == (m, n)
        assert scale_tensor.numel() == 1 and scale_tensor.dtype == torch.float32
        with torch.cuda.device(a_shard.device):
            stream_ptr = (stream or torch.cuda.current_stream(a_shard.device)).cuda_stream
            _capi.check(_capi.lib.hfrk_skinny_gemm_fp8_rowpar(
                self._handle, a_shard.data_ptr(), w_shard.data_ptr(), output.data_ptr(), scale_tensor.data_ptr(),
                m, n, k_shard, w_shard.stride(0), _capi.fp8_kind(a_shard.dtype), _capi.fp8_kind(w_shard.dtype),
                _capi.out_kind(output.dtype), int(accumulate), stream_ptr))
        return output

    def set_mode(self, mode: str = "auto") -> None:
        """How partial tiles cross NVLink: "one_shot" (every rank sends to every peer), "two_shot"
        (an owner rank per tile position adds up and sends the sums back) or "auto" (by traffic).
        Every rank must choose the same."""
        code = {"auto": _capi.ROWPAR_AUTO, "one_shot": _capi.ROWPAR_ONE_SHOT, "two_shot": _capi.ROWPAR_TWO_SHOT}[mode]
        _capi.check(_capi.lib.hfrk_rowpar_set_mode(self._handle, code))

    def close(self) -> None:
        if getattr(self, "_handle", None) is not None:
            torch.cuda.synchronize(self.device)
            _capi.lib.hfrk_rowpar_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def skinny_gemm_then_allreduce(a_shard: Tensor, w_shard: Tensor, scale_tensor: Tensor, output: Tensor,
                               partial: Tensor, group: Optional[dist.ProcessGroup] = None) -> Tensor:
    """Unfused baseline: ``partial`` (float32 [M,N] scratch) <- A_r @ W_r.T with scale 1 folded
    later, NCCL all-reduce, then ``output += scale * partial`` in torch."""
    ones = getattr(skinny_gemm_then_allreduce, "_ones", None)
    if ones is None or ones.device != a_shard.device:
        ones = torch.ones(1, dtype=torch.float32, device=a_shard.device)
        skinny_gemm_then_allreduce._ones = ones
    _capi.check(_capi.skinny_gemm_ex(a_shard, w_shard, partial, ones, accumulate=False))
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, group=group)
    output.copy_((output.float() + partial * scale_tensor).to(output.dtype))
    return output
