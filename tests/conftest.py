import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    """The package, loaded by path (its directory name has hyphens). Building is the driver's
    build() step; importing fails loudly if the CUDA library is missing."""
    import __graft_entry__ as ge
    lib = os.path.join(ge.PKG_DIR, "libb200_linear.so")
    if not os.path.exists(lib):
        ge.build()
    return ge.load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import build as obuild
    obuild.build_oracle()
    from oracle import oracle as o
    return o


@pytest.fixture(scope="session")
def handle(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    h = pkg.Handle()
    yield h
    h.sync()
    h.destroy()


@pytest.fixture(scope="session")
def ref_lib():
    """The reference's own matmul.cu (cuBLAS), prebuilt into oracle/_ref/ (checker only)."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libref_matmul.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libref_matmul.so not built (reference checkout absent at build time)")
    lib = ctypes.CDLL(path)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.ref_create.argtypes = [ctypes.POINTER(vp)]
    lib.ref_create_fp32.argtypes = [ctypes.POINTER(vp)]
    lib.ref_destroy.argtypes = [vp]
    lib.ref_matmul_forward_bf16.argtypes = [vp, vp, vp, vp, ci, ci, ci]
    lib.ref_matmul_forward_f32.argtypes = [vp, vp, vp, vp, ci, ci, ci]
    lib.ref_matmul_backward_bf16.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci]
    lib.ref_matmul_backward_f32.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci]
    for n in ("ref_matmul_forward_bf16", "ref_matmul_forward_f32", "ref_matmul_backward_bf16",
              "ref_matmul_backward_f32"):
        getattr(lib, n).restype = None
    if hasattr(lib, "ref_crossentropy_forward_bf16"):
        lib.ref_crossentropy_forward_bf16.argtypes = [vp, vp, vp, ci, ci, ci]
        lib.ref_crossentropy_forward_bf16.restype = None
        lib.ref_crossentropy_backward_bf16.argtypes = [vp, vp, vp, ci, ci, ci, ctypes.c_float]
        lib.ref_crossentropy_backward_bf16.restype = None
    return lib
