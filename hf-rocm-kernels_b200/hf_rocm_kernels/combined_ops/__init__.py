from .row_parallel import RowParallelSkinnyGemm, skinny_gemm_then_allreduce

__all__ = ["RowParallelSkinnyGemm", "skinny_gemm_then_allreduce"]
