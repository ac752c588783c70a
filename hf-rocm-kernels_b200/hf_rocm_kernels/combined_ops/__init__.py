from .llama_mlp import llama_mlp_combined_ops
from .row_parallel import RowParallelSkinnyGemm, skinny_gemm_then_allreduce

__all__ = ["llama_mlp_combined_ops", "RowParallelSkinnyGemm", "skinny_gemm_then_allreduce"]
