"""ctypes doorway onto oracle/liboracle.so (TEST INFRASTRUCTURE — not part of the product).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference legs import this.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")

FWD_NN, DGRAD_NT, WGRAD_TN = 0, 1, 2


def _load():
    if not os.path.exists(_LIB):
        from . import build as _b  # noqa: F401  (package-relative when imported as oracle.oracle)
        _b.build_oracle()
    lib = ctypes.CDLL(_LIB)
    fp = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    dp = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
    ip = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
    ci = ctypes.c_int
    lib.oracle_fill_normal.argtypes = [fp, ctypes.c_size_t, ctypes.c_uint64, ctypes.c_float, ctypes.c_float]
    lib.oracle_fill_normal.restype = None
    lib.oracle_round_bf16.argtypes = [fp, ctypes.c_size_t]
    lib.oracle_round_bf16.restype = None
    lib.oracle_gemm_f64.argtypes = [ci, dp, ctypes.c_void_p, fp, fp, ci, ci, ci]
    lib.oracle_gemm_f64_samples.argtypes = [ci, dp, fp, fp, ci, ci, ci, ip, ip, ci]
    lib.oracle_gemm_f32.argtypes = [ci, ci, fp, fp, fp, ci, ci, ci]
    lib.oracle_num_threads.restype = ci
    return lib


lib = _load()


def out_shape(which, M, N, K):
    if which not in (FWD_NN, DGRAD_NT, WGRAD_TN):
        raise ValueError(f"unknown product {which}")
    return {FWD_NN: (M, N), DGRAD_NT: (M, K), WGRAD_TN: (K, N)}[which]


def in_shapes(which, M, N, K):
    return {FWD_NN: ((M, K), (K, N)), DGRAD_NT: ((M, N), (K, N)), WGRAD_TN: ((M, K), (M, N))}[which]


def normal(shape, seed, std=1.0, mean=0.0, bf16=False):
    """Seeded N(mean, std) float32 array; element i depends only on (seed, i)."""
    a = np.empty(shape, dtype=np.float32)
    lib.oracle_fill_normal(a.reshape(-1), a.size, seed, mean, std)
    if bf16:
        lib.oracle_round_bf16(a.reshape(-1), a.size)
    return a


def round_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float32).copy()
    lib.oracle_round_bf16(a.reshape(-1), a.size)
    return a


def reference_bf16_result(product64, old=None):
    """What the reference's bf16 path stores for a product whose exact value is `product64`:
    bf16_rn(product) for beta = 0 (cuda/matmul.cu:61,82 of the reference) and, for the beta = 1
    weight gradient (cuda/matmul.cu:94), bf16_rn(bf16_rn(product) + old): cuBLAS rounds the
    product to the output type before it adds the old value (observed bit for bit on a B200,
    tests/golden/reference_cublas.npz)."""
    r = round_bf16(np.asarray(product64, dtype=np.float64).astype(np.float32))
    if old is None:
        return r
    return round_bf16((r.astype(np.float64) + np.asarray(old, dtype=np.float64)).astype(np.float32))


def gemm_f64(which, x, y, M, N, K, old=None):
    """float64 result of product `which` (+ old when given)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.ascontiguousarray(y, dtype=np.float32)
    out = np.empty(out_shape(which, M, N, K), dtype=np.float64)
    oldp = None
    if old is not None:
        old = np.ascontiguousarray(old, dtype=np.float32)
        oldp = old.ctypes.data_as(ctypes.c_void_p)
    rc = lib.oracle_gemm_f64(which, out, oldp, x, y, M, N, K)
    if rc:
        raise ValueError("oracle_gemm_f64: bad arguments")
    return out


def gemm_f64_samples(which, x, y, M, N, K, rows, cols):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.ascontiguousarray(y, dtype=np.float32)
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    cols = np.ascontiguousarray(cols, dtype=np.int32)
    out = np.empty(rows.size, dtype=np.float64)
    rc = lib.oracle_gemm_f64_samples(which, out, x, y, M, N, K, rows, cols, rows.size)
    if rc:
        raise ValueError("oracle_gemm_f64_samples: bad arguments")
    return out


def gemm_f32(which, beta1, out, x, y, M, N, K):
    """In-place fp32 host GEMM (the timed CPU baseline)."""
    rc = lib.oracle_gemm_f32(which, int(bool(beta1)), out, x, y, M, N, K)
    if rc:
        raise ValueError("oracle_gemm_f32: bad arguments")
    return out


def num_threads():
    return int(lib.oracle_num_threads())
