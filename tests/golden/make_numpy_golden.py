"""Generates tests/golden/numpy_f64.npz: small seeded inputs and their float64 products computed
by numpy (an implementation independent of oracle/oracle_gemm.c), plus known values of the
oracle's seeded generator and bf16 rounding taken from torch.  Run from the repository root:

    python tests/golden/make_numpy_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle  # noqa: E402

CASES = [(48, 40, 24), (1, 8, 8), (130, 40, 72), (40, 88, 72), (7, 5, 3)]


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    for i, (M, N, K) in enumerate(CASES):
        A = rng.standard_normal((M, K)).astype(np.float32)
        B = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
        dC = rng.standard_normal((M, N)).astype(np.float32)
        old = rng.standard_normal((K, N)).astype(np.float32)
        out[f"c{i}_dims"] = np.array([M, N, K], dtype=np.int32)
        out[f"c{i}_A"], out[f"c{i}_B"], out[f"c{i}_dC"], out[f"c{i}_old"] = A, B, dC, old
        A64, B64, dC64 = A.astype(np.float64), B.astype(np.float64), dC.astype(np.float64)
        out[f"c{i}_fwd"] = A64 @ B64
        out[f"c{i}_dgrad"] = dC64 @ B64.T
        out[f"c{i}_wgrad"] = old.astype(np.float64) + A64.T @ dC64
    # generator and rounding pins
    out["normal_seed7_first64"] = oracle.normal((64,), 7)
    x = rng.standard_normal(1024).astype(np.float32) * np.float32(3.0)
    x[:8] = np.array([0.0, -0.0, 1.0, 1.00390625, 1.0078125, 3.3895314e38, 1e-40, -2.5], dtype=np.float32)
    out["round_in"] = x
    out["round_out_torch"] = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    np.savez_compressed(os.path.join(HERE, "numpy_f64.npz"), **out)
    print("wrote", os.path.join(HERE, "numpy_f64.npz"))


if __name__ == "__main__":
    main()
