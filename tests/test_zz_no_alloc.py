"""The allocation-free weight-gradient entry point against the regular one.

Some hosts cannot let this library call cudaMalloc (they own all device memory through an arena
of their own, or cannot afford the device-wide stall an allocation causes in the middle of a
step).  `b200_linear_wgrad_bf16_noalloc` serves them from a fixed scratch array inside the
library; here it must agree with `b200_linear_gemm_bf16(WGRAD_TN, beta=1)` on two calls in a
row, the second one accumulating on top of the first and reusing the scratch the first left
behind.  The file name sorts last on purpose, so a run that stops at the first failure has
already been through every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_noalloc_wgrad_matches_regular_entry_point_twice(pkg, handle):
    fn = pkg.lib.b200_linear_wgrad_bf16_noalloc
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, ci, ci, ci, vp]
    fn.restype = ci
    dt = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(4242)
    for (M, N, K) in [(8192, 2048, 768), (1000, 264, 136), (4096, 256, 768)]:
        a = torch.randn(M, K, device=DEV, generator=g).to(dt)
        dc = torch.randn(M, N, device=DEV, generator=g).to(dt)
        start = torch.randn(K, N, device=DEV, generator=g).to(dt)
        want = start.clone()
        got = start.clone()
        for call in range(2):  # two calls in a row: the second accumulates and reuses the scratch
            pkg.gemm(handle, pkg.WGRAD_TN, 1, want, a, dc, M, N, K)
            handle.sync()
            rc = fn(got.data_ptr(), a.data_ptr(), dc.data_ptr(), M, N, K, None)
            assert rc == 0, pkg.strerror(rc)
            torch.cuda.synchronize()
            err = ((got.double() - want.double()).abs().max() / want.double().abs().max()).item()
            assert err <= 1e-2, (M, N, K, call, err)
    # beyond the stated maximum: a clear error, nothing launched
    big = torch.zeros(8, device=DEV, dtype=dt)
    assert fn(big.data_ptr(), big.data_ptr(), big.data_ptr(), 64, 32000, 768, None) == 5  # B200_E_TOOBIG
    assert fn(big.data_ptr(), big.data_ptr(), big.data_ptr(), 64, 250, 768, None) == 1    # B200_E_BADARG
    assert fn(None, big.data_ptr(), big.data_ptr(), 64, 256, 768, None) == 1
