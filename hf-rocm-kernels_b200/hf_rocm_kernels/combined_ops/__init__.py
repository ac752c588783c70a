from .llama_mlp import can_fuse_swiglu, llama_mlp_combined_ops, skinny_gemm_swiglu
from .row_parallel import RowParallelSkinnyGemm, skinny_gemm_then_allreduce

__all__ = ["llama_mlp_combined_ops", "skinny_gemm_swiglu", "can_fuse_swiglu", "RowParallelSkinnyGemm",
           "skinny_gemm_then_allreduce"]
