"""The C-ABI library: it loads, exports every symbol include/*.h declares and the four mangled
kernels.cuh overloads, and refuses to work (instead of falling back) without a GPU."""
import ctypes
import glob
import os
import re
import subprocess

import pytest
import torch

from conftest import ROOT


def _declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(b200_\w+)\s*\(", text))
    return sorted(names)


def test_header_symbols_exported(pkg):
    names = _declared_symbols()
    assert len(names) >= 40
    for n in names:
        assert hasattr(pkg.lib, n), f"{n} declared in include/ but not exported"


def test_kernels_cuh_overloads_exported(pkg):
    # Itanium-mangled names of the reference's four overloads (cuda/kernels.cuh:47-65, 348-351)
    want = ["_Z14matmul_forwardP13cublasContextPfPKfS3_iii",
            "_Z15matmul_backwardP13cublasContextPfS1_PKfS3_S3_iii",
            "_Z14matmul_forwardP13cublasContextP13__nv_bfloat16PKS1_S4_iii",
            "_Z15matmul_backwardP13cublasContextP13__nv_bfloat16S2_PKS1_S4_S4_iii"]
    for n in want:
        assert hasattr(pkg.lib, n), n


def test_no_vendor_gemm_library_linked(pkg):
    out = subprocess.run(["ldd", pkg.linear.LIB_PATH], capture_output=True, text=True).stdout
    for bad in ("cublas", "cutlass", "cudnn", "nccl"):
        assert bad not in out.lower(), out


def test_cublas_shim_exports(pkg):
    path = os.path.join(os.path.dirname(pkg.linear.LIB_PATH), "libb200_cublas_shim.so")
    if not os.path.exists(path):
        pytest.skip("shim not built")
    shim = ctypes.CDLL(path)
    for n in ("cublasCreate_v2", "cublasDestroy_v2", "cublasSetMathMode"):
        assert hasattr(shim, n)
    h = ctypes.c_void_p()
    assert shim.cublasCreate_v2(ctypes.byref(h)) == 0 and h.value
    assert shim.cublasSetMathMode(h, 1) == 0
    assert shim.cublasDestroy_v2(h) == 0


def test_strerror_and_null_handling(pkg):
    assert pkg.strerror(0) == "ok"
    assert "argument" in pkg.strerror(1)
    assert pkg.lib.b200_linear_destroy(None) == 1
    assert pkg.lib.b200_linear_sync(None, None) == 1
    assert pkg.lib.b200_linear_forward_bf16(None, None, None, None, 8, 8, 8) == 1
    assert pkg.lib.b200_linear_create(None) == 1


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_create_fails_loudly_without_gpu(pkg):
    with pytest.raises(pkg.LinearError):
        pkg.Handle()
