"""B200-native linear-layer GEMMs behind the reference's matmul_forward / matmul_backward."""
from .linear import (DGRAD_NT, FWD_NN, WGRAD_TN, Handle, LinearError, Plan, ce_shard_backward, ce_shard_loss,
                     ce_shard_rescale, ce_shard_stats, gemm, gemm_grouped, gemm_ld, lib, matmul_backward, matmul_backward_grouped, matmul_forward, swiglu_forward_gemm, forward_ce_stats,
                     plan_bf16, plan_grouped_bf16,
                     strerror)

__all__ = ["Handle", "LinearError", "Plan", "matmul_forward", "matmul_backward", "gemm", "gemm_ld", "gemm_grouped", "matmul_backward_grouped", "swiglu_forward_gemm", "forward_ce_stats", "plan_bf16", "plan_grouped_bf16",
           "strerror", "lib", "FWD_NN", "DGRAD_NT", "WGRAD_TN", "ce_shard_stats", "ce_shard_rescale", "ce_shard_loss",
           "ce_shard_backward"]
