"""The MLP block of a Llama decoder layer as a chain of this package's operators:

    residual_rms  ->  skinny_gemm (gate/up)  ->  swiglu  ->  skinny_gemm (down)

Same function and argument names as the reference's ``hf_rocm_kernels/combined_ops/llama_mlp.py:7-62``.
Each element-wise kernel quantises the next GEMM's input and zeroes the buffer that GEMM
accumulates into, so the chain is four launches with nothing between them; all four are
programmatic dependents of one another, which lets each GEMM stream weights while the kernel
before it is still running.

Two additions for B200: the activations are quantised to the weights' fp8 format (e4m3fnuz as in
the reference, or e4m3fn), and ``down_row_parallel`` runs the block tensor-parallel over the GPUs
of a process group: every rank holds a column shard of the gate/up weight (no exchange: N split)
and the matching K shard of the down weight, whose GEMM carries the all-reduce in its epilogue.
"""
from typing import Optional, Tuple

import torch
from torch import Tensor

import hf_rocm_kernels._HFRK_C  # noqa: F401  (registers torch.ops._HFRK_C)
from hf_rocm_kernels import residual_rms, skinny_gemm, swiglu
from hf_rocm_kernels.combined_ops.row_parallel import RowParallelSkinnyGemm


def can_fuse_swiglu(tokens: int, hidden: int, intermediate: int) -> bool:
    """True when the gate/up projection and swiglu can run as one launch: at most 16 tokens and
    output rows that split into 16-byte pieces."""
    del hidden
    return tokens <= 16 and intermediate % 16 == 0


def skinny_gemm_swiglu(
    skinny_a: Tensor,
    gate_up_weight: Tensor,
    scale_tensor: Tensor,
    act_scale_tensor: Tensor,
    next_buffer: Optional[Tensor] = None,
    mid_dtype: torch.dtype = torch.bfloat16,
    out_dtype: Optional[torch.dtype] = None,
) -> Tensor:
    """``fp8(silu(g) * u / act_scale)`` with ``[g | u] = round(scale * skinny_a @ gate_up_weight)``
    in one launch: the same bytes as ``skinny_gemm`` into a ``mid_dtype`` buffer followed by
    ``swiglu``. ``gate_up_weight`` is the (hidden, 2 * intermediate) column-major view, gate columns
    first; ``next_buffer`` (16-bit, tokens rows) is zeroed."""
    assert gate_up_weight.dim() == 2 and gate_up_weight.stride(0) == 1, "expected the column-major [K, N] view"
    assert mid_dtype in (torch.float16, torch.bfloat16), f"Expected a 16-bit mid_dtype but got {mid_dtype}"
    tokens, inter = skinny_a.size(0), gate_up_weight.size(1) // 2
    if tokens > 16:
        raise RuntimeError("skinny_gemm_swiglu takes at most 16 tokens; run skinny_gemm and swiglu instead")
    out = torch.empty((tokens, inter), dtype=out_dtype or gate_up_weight.dtype, device=skinny_a.device)
    if next_buffer is None:
        next_buffer = torch.empty((tokens, 0), dtype=mid_dtype, device=skinny_a.device)
    torch.ops._HFRK_C.skinny_gemm_swiglu(skinny_a, gate_up_weight, out, scale_tensor, act_scale_tensor, next_buffer,
                                         mid_dtype == torch.bfloat16)
    return out


def llama_mlp_combined_ops(
    attn_output: Tensor,
    residual: Tensor,
    rms_weight: Tensor,
    rms_epsilon: float,
    gate_up_weight: Tensor,
    gate_up_input_scale: Tensor,
    gate_up_output_scale: Tensor,
    down_weight: Tensor,
    down_input_scale: Tensor,
    down_output_scale: Tensor,
    gate_up_gemm_hp: Tuple[Optional[int], Optional[int]] = (None, None),
    down_gemm_hp: Tuple[Optional[int], Optional[int]] = (None, None),
    down_row_parallel: Optional[RowParallelSkinnyGemm] = None,
    fuse_swiglu: Optional[bool] = None,
) -> Tuple[Tensor, Tensor]:
    """Returns ``(mlp_output, residual)``; ``residual`` is updated in place to ``attn_output + residual``.

    Args:
        attn_output, residual: (tokens, hidden) fp16 or bf16
        rms_weight: (hidden,) post-attention RMS-norm weight
        gate_up_weight: fp8 (hidden, 2 * intermediate) column-major, i.e. ``w_nk.t()``; with
            ``down_row_parallel`` this rank's shard (hidden, 2 * intermediate / world) holding its
            slice of the gate columns followed by the same slice of the up columns
        gate_up_input_scale: scale the normalised activations are divided by before fp8
        gate_up_output_scale: product of the activation and weight scales of the gate/up GEMM
        down_weight: fp8 (intermediate, hidden) column-major; with ``down_row_parallel`` this
            rank's K shard, (intermediate / world, hidden)
        down_input_scale, down_output_scale: the same two scales for the down projection
        gate_up_gemm_hp, down_gemm_hp: (split_k, b_lanes) pairs of the reference's kernel;
            accepted so that existing callers keep working, not used (the library picks the
            launch shape per (m, n, k), or takes it from its tuning table)
        fuse_swiglu: run the gate/up projection and swiglu as one launch (same bytes as the two
            launches); ``None`` decides with :func:`can_fuse_swiglu`
        down_row_parallel: the exchange object of the ranks that share the block; every rank
            multiplies its slice of the swiglu output by its K shard of the down weight and all
            ranks receive the summed result (same bits on every rank)
    """
    del gate_up_gemm_hp, down_gemm_hp
    tokens = attn_output.size(0)
    act_dtype = gate_up_weight.dtype

    hidden, inter = gate_up_weight.size(0), gate_up_weight.size(1) // 2
    if fuse_swiglu is None:
        fuse_swiglu = can_fuse_swiglu(tokens, hidden, inter)
    mlp_output = torch.empty((tokens, down_weight.size(1)), dtype=attn_output.dtype, device=attn_output.device)
    if fuse_swiglu:
        normalized, residual = residual_rms(
            input=attn_output, residual=residual, weight=rms_weight, epsilon=rms_epsilon,
            scale_tensor=gate_up_input_scale, next_buffer=None, out_dtype=act_dtype,
        )
        swiglu_out = skinny_gemm_swiglu(normalized, gate_up_weight, gate_up_output_scale, down_input_scale,
                                        next_buffer=mlp_output, mid_dtype=attn_output.dtype,
                                        out_dtype=down_weight.dtype)
    else:
        gate_up_proj = torch.empty((tokens, 2 * inter), dtype=attn_output.dtype, device=attn_output.device)
        normalized, residual = residual_rms(
            input=attn_output,
            residual=residual,
            weight=rms_weight,
            epsilon=rms_epsilon,
            scale_tensor=gate_up_input_scale,
            next_buffer=gate_up_proj,
            out_dtype=act_dtype,
        )
        skinny_gemm(skinny_a=normalized, b=gate_up_weight, scale_tensor=gate_up_output_scale, output=gate_up_proj)
        swiglu_out = swiglu(
            gate_up_proj=gate_up_proj, scale_tensor=down_input_scale, next_buffer=mlp_output,
            out_dtype=down_weight.dtype,
        )
    if down_row_parallel is None:
        skinny_gemm(skinny_a=swiglu_out, b=down_weight, scale_tensor=down_output_scale, output=mlp_output)
    else:
        assert down_weight.size(0) == swiglu_out.size(1), \
            f"Expected a K shard of {swiglu_out.size(1)} rows but got {down_weight.shape = }"
        down_row_parallel(swiglu_out, down_weight.t(), down_output_scale, mlp_output)
    return mlp_output, residual
