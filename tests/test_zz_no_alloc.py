"""The allocation-free weight-gradient entry point against the CPU oracle and the regular entry point.

Some hosts cannot let this library call cudaMalloc (they own all device memory through an arena
of their own, or cannot afford the device-wide stall an allocation causes in the middle of a
step).  `b200_linear_wgrad_bf16_noalloc` serves them from a fixed scratch array inside the
library.  Here two calls in a row (the second accumulating on top of the first and reusing the
scratch the first left behind) are checked against the oracle's restatement of the reference's
beta = 1 rounding sequence, bf16_rn(bf16_rn(A^T dC) + dB_old), and against
`b200_linear_gemm_bf16(WGRAD_TN, beta=1)`.  The file name sorts last on purpose, so a run that
stops at the first failure has already been through every other test."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2  # max |got - want| / max |want|, the bf16 tolerance of every GEMM test here


def _entry(pkg):
    fn = pkg.lib.b200_linear_wgrad_bf16_noalloc
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, ci, ci, ci, vp]
    fn.restype = ci
    st = pkg.lib.b200_linear_noalloc_status
    st.argtypes = [ctypes.POINTER(ci), vp]
    st.restype = ci
    return fn, st


def test_noalloc_wgrad_matches_oracle_and_regular_entry_point_twice(pkg, handle, oracle):
    fn, status = _entry(pkg)
    dt = torch.bfloat16
    # 768x2048 = 96 tiles; ragged 136x264; 768x256; 2048x1024 = exactly the 128-tile limit
    for (M, N, K) in [(8192, 2048, 768), (1000, 264, 136), (4096, 256, 768), (512, 1024, 2048)]:
        A = oracle.normal((M, K), 4000 + M, bf16=True)
        dC = oracle.normal((M, N), 5000 + N, bf16=True)
        start = oracle.normal((K, N), 6000 + K, bf16=True)
        a, dc = (torch.from_numpy(v).to(DEV, dt) for v in (A, dC))
        regular = torch.from_numpy(start).to(DEV, dt)
        got = regular.clone()
        product = oracle.gemm_f64(oracle.WGRAD_TN, A, dC, M, N, K)
        want = start
        for call in range(2):  # two calls in a row: the second accumulates and reuses the scratch
            want = oracle.reference_bf16_result(product, old=want)
            pkg.gemm(handle, pkg.WGRAD_TN, 1, regular, a, dc, M, N, K)
            handle.sync()
            rc = fn(got.data_ptr(), a.data_ptr(), dc.data_ptr(), M, N, K, None)
            assert rc == 0, pkg.strerror(rc)
            code = ctypes.c_int(-1)
            assert status(ctypes.byref(code), None) == 0 and code.value == 0
            g = got.float().cpu().numpy().astype(np.float64)
            scale = np.abs(want).max()
            assert np.abs(g - want).max() / scale <= TOL, (M, N, K, call)
            # the oracle models the reference's two roundings: all but a few one-ulp cases agree exactly
            assert (g != want).mean() <= 0.02, (M, N, K, call, (g != want).mean())
            r = regular.float().cpu().numpy().astype(np.float64)
            assert np.abs(g - r).max() / scale <= TOL, (M, N, K, call)
    # beyond the stated maximum: a clear error, nothing launched
    big = torch.zeros(8, device=DEV, dtype=dt)
    assert fn(big.data_ptr(), big.data_ptr(), big.data_ptr(), 64, 32000, 768, None) == 5  # B200_E_TOOBIG
    assert fn(big.data_ptr(), big.data_ptr(), big.data_ptr(), 64, 1024, 2048 + 8, None) == 5  # 136 tiles
    assert fn(big.data_ptr(), big.data_ptr(), big.data_ptr(), 64, 250, 768, None) == 1    # B200_E_BADARG
    assert fn(None, big.data_ptr(), big.data_ptr(), 64, 256, 768, None) == 1
