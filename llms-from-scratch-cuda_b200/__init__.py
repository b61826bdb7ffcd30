"""B200-native linear-layer GEMMs behind the reference's matmul_forward / matmul_backward."""
from .linear import (DGRAD_NT, FWD_NN, WGRAD_TN, Handle, LinearError, Plan, gemm, lib, matmul_backward,
                     matmul_forward, plan_bf16, strerror)

__all__ = ["Handle", "LinearError", "Plan", "matmul_forward", "matmul_backward", "gemm", "plan_bf16",
           "strerror", "lib", "FWD_NN", "DGRAD_NT", "WGRAD_TN"]
