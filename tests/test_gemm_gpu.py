"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle
(oracle/oracle_gemm.c), the committed fixtures and the reference's own cuBLAS build.

Error metric (stated once): max_ij |C - C64| / max_ij |C64| per product; tolerances
1e-2 for bf16 storage and 1e-5 for fp32, as the task's north star states them."""
import ctypes
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN

pytestmark = pytest.mark.gpu

TOL = {torch.bfloat16: 1e-2, torch.float32: 1e-5}
DEV = "cuda:0"


def rel_err(got, want64):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    return np.abs(got - want64).max() / max(np.abs(want64).max(), 1e-300)


def dev(a, dt):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV, dt)


def inputs(oracle, M, N, K, seed, bf16):
    A = oracle.normal((M, K), seed + 1, bf16=bf16)
    B = oracle.normal((K, N), seed + 2, std=0.02, bf16=bf16)
    dC = oracle.normal((M, N), seed + 3, bf16=bf16)
    return A, B, dC


# ----------------------------------------------------------------- config 1 of the baseline
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_config1_linear_layer_fwd_bwd(pkg, handle, oracle, dt):
    """X[8192,768] ~ N(0,1), W[768,768] ~ N(0,0.02), dY ~ N(0,1); Y, dX, and dW accumulated
    twice with beta=1, all against the fp64 host loop."""
    M, N, K = 8192, 768, 768
    A, B, dC = inputs(oracle, M, N, K, 1000, dt == torch.bfloat16)
    a, b, dc = dev(A, dt), dev(B, dt), dev(dC, dt)
    c = torch.empty(M, N, device=DEV, dtype=dt)
    da = torch.empty(M, K, device=DEV, dtype=dt)
    db = torch.zeros(K, N, device=DEV, dtype=dt)
    pkg.matmul_forward(handle, c, a, b, M, N, K)
    pkg.matmul_backward(handle, da, db, dc, a, b, M, N, K)
    handle.sync()
    db1 = db.clone()
    pkg.matmul_backward(handle, da, db, dc, a, b, M, N, K)
    handle.sync()
    tol = TOL[dt]
    assert rel_err(c, oracle.gemm_f64(0, A, B, M, N, K)) <= tol
    assert rel_err(da, oracle.gemm_f64(1, dC, B, M, N, K)) <= tol
    w1 = oracle.gemm_f64(2, A, dC, M, N, K)
    assert rel_err(db1, w1) <= tol
    # second micro-batch: the stored (rounded) dW is the beta=1 input, as in the reference
    w2 = oracle.gemm_f64(2, A, dC, M, N, K, old=db1.float().cpu().numpy())
    assert rel_err(db, w2) <= tol
    assert rel_err(db, 2.0 * w1) <= tol


def test_config1_bf16_agrees_with_fp32_path(pkg, handle, oracle):
    M, N, K = 8192, 768, 768
    A, B, dC = inputs(oracle, M, N, K, 1000, True)
    outs = {}
    for dt in (torch.bfloat16, torch.float32):
        a, b, dc = dev(A, dt), dev(B, dt), dev(dC, dt)
        c = torch.empty(M, N, device=DEV, dtype=dt)
        da = torch.empty(M, K, device=DEV, dtype=dt)
        db = torch.zeros(K, N, device=DEV, dtype=dt)
        pkg.matmul_forward(handle, c, a, b, M, N, K)
        pkg.matmul_backward(handle, da, db, dc, a, b, M, N, K)
        handle.sync()
        outs[dt] = (c.double(), da.double(), db.double())
    for x, y in zip(outs[torch.bfloat16], outs[torch.float32]):
        assert ((x - y).abs().max() / y.abs().max()).item() <= 1e-2


# ------------------------------------------------- config 2: one decoder layer + LM head
LAYER_SHAPES = [(8192, 768, 768), (8192, 256, 768), (8192, 2048, 768), (8192, 768, 2048),
                (8192, 1280, 768), (8192, 4096, 768), (8192, 32000, 768)]


def _sample_points(rng, rows, cols, n=4096):
    r = rng.integers(0, rows, n)
    c = rng.integers(0, cols, n)
    # tile-edge rows/columns: first/last of 128- and 256-wide tiles
    edges_r = np.array([0, 127, 128, rows - 129, rows - 128, rows - 1]) % rows
    edges_c = np.array([0, 63, 64, 255, 256, cols - 257, cols - 256, cols - 1]) % cols
    er, ec = np.meshgrid(edges_r, edges_c)
    return (np.concatenate([r, er.ravel()]).astype(np.int32), np.concatenate([c, ec.ravel()]).astype(np.int32))


@pytest.mark.parametrize("M,N,K", LAYER_SHAPES)
def test_config2_layer_shapes_sampled_fp64(pkg, handle, oracle, M, N, K):
    rng = np.random.default_rng(M + N + K)
    A, B, dC = inputs(oracle, M, N, K, 2000 + N, True)
    dt = torch.bfloat16
    a, b, dc = dev(A, dt), dev(B, dt), dev(dC, dt)
    c = torch.empty(M, N, device=DEV, dtype=dt)
    da = torch.empty(M, K, device=DEV, dtype=dt)
    db = torch.zeros(K, N, device=DEV, dtype=dt)
    pkg.matmul_forward(handle, c, a, b, M, N, K)
    pkg.matmul_backward(handle, da, db, dc, a, b, M, N, K)
    handle.sync()
    for which, got, x, y in ((0, c, A, B), (1, da, dC, B), (2, db, A, dC)):
        rows, cols = got.shape
        r, cc = _sample_points(rng, rows, cols)
        want = oracle.gemm_f64_samples(which, x, y, M, N, K, r, cc)
        g = got.float().cpu().numpy()[r, cc].astype(np.float64)
        scale = np.abs(want).max()
        assert np.abs(g - want).max() / scale <= 1e-2, (which, M, N, K)


def test_config2_dw_accumulates_over_16_microbatches(pkg, handle, oracle):
    """dW of the down projection accumulated over 16 micro-batches with different activations;
    compared with the oracle's sequence dW_{i+1} = bf16_rn(bf16_rn(acc_i) + float(dW_i)) (the
    reference's rounding) and with the fp64 sum."""
    M, N, K = 2048, 768, 2048
    dt = torch.bfloat16
    db = torch.zeros(K, N, device=DEV, dtype=dt)
    seq = np.zeros((K, N), np.float32)
    total = np.zeros((K, N), np.float64)
    for mb in range(16):
        A = oracle.normal((M, K), 3000 + 2 * mb, bf16=True)
        dC = oracle.normal((M, N), 3001 + 2 * mb, bf16=True)
        pkg.matmul_backward(handle, None, db, dev(dC, dt), dev(A, dt), None, M, N, K)
        acc = oracle.gemm_f64(2, A, dC, M, N, K)
        total += acc
        seq = oracle.reference_bf16_result(acc, seq)  # the reference's rounding of a beta=1 update
    handle.sync()
    got = db.float().cpu().numpy()
    scale = np.abs(total).max()
    assert np.abs(got - seq).max() / scale <= 8e-3   # within two bf16 ulps (at the largest magnitude) of the oracle's sequence
    # against the unrounded fp64 sum the 16 read-modify-write roundings of bf16 storage add up
    # (the reference accumulates in bf16 storage as well): allow 16 half-ulps at the top magnitude
    assert np.abs(got - total).max() / scale <= 16 * 2.0 ** -9


# ------------------------------------------------------------------ fixtures and the reference
def test_numpy_golden_fixtures(pkg, handle):
    g = np.load(os.path.join(GOLDEN, "numpy_f64.npz"))
    for case in range(5):
        M, N, K = (int(v) for v in g[f"c{case}_dims"])
        A, B, dC, old = (g[f"c{case}_{n}"] for n in ("A", "B", "dC", "old"))
        dt = torch.float32
        c = torch.empty(M, N, device=DEV, dtype=dt)
        da = torch.empty(M, K, device=DEV, dtype=dt)
        db = dev(old, dt)
        pkg.matmul_forward(handle, c, dev(A, dt), dev(B, dt), M, N, K)
        pkg.matmul_backward(handle, da, db, dev(dC, dt), dev(A, dt), dev(B, dt), M, N, K)
        handle.sync()
        for got, name in ((c, "fwd"), (da, "dgrad"), (db, "wgrad")):
            assert rel_err(got, g[f"c{case}_{name}"]) <= 1e-5, (case, name)


@pytest.mark.parametrize("dt,sfx", [(torch.bfloat16, "bf16"), (torch.float32, "f32")])
def test_against_reference_cublas_live(pkg, handle, oracle, ref_lib, dt, sfx):
    """Same seeded inputs through the reference's own matmul.cu (cuBLAS) and through this
    library, on the device, full matrices."""
    h = ctypes.c_void_p()
    create = ref_lib.ref_create if dt == torch.bfloat16 else ref_lib.ref_create_fp32
    assert create(ctypes.byref(h)) == 0
    try:
        for (M, N, K) in [(8192, 768, 768), (2048, 2048, 768), (1024, 32000, 768), (8192, 256, 768)]:
            A, B, dC = inputs(oracle, M, N, K, 4000 + N, dt == torch.bfloat16)
            a, b, dc = dev(A, dt), dev(B, dt), dev(dC, dt)
            old = dev(oracle.normal((K, N), 4100 + N, bf16=dt == torch.bfloat16), dt)
            res = []
            for side in ("ref", "ours"):
                c = torch.empty(M, N, device=DEV, dtype=dt)
                da = torch.empty(M, K, device=DEV, dtype=dt)
                db = old.clone()
                if side == "ref":
                    getattr(ref_lib, "ref_matmul_forward_" + sfx)(h, c.data_ptr(), a.data_ptr(), b.data_ptr(), M, N, K)
                    getattr(ref_lib, "ref_matmul_backward_" + sfx)(h, da.data_ptr(), db.data_ptr(), dc.data_ptr(),
                                                                  a.data_ptr(), b.data_ptr(), M, N, K)
                    torch.cuda.synchronize()
                else:
                    pkg.matmul_forward(handle, c, a, b, M, N, K)
                    pkg.matmul_backward(handle, da, db, dc, a, b, M, N, K)
                    handle.sync()
                res.append((c.double(), da.double(), db.double()))
            for r, o in zip(*res):
                # both round the same fp32-accumulated value: at most an ulp or two apart
                assert ((r - o).abs().max() / r.abs().max()).item() <= (8e-3 if dt == torch.bfloat16 else 1e-5)
    finally:
        ref_lib.ref_destroy(h)


def test_reference_golden_fixture(pkg, handle, oracle):
    path = os.path.join(GOLDEN, "reference_cublas.npz")
    if not os.path.exists(path):
        pytest.skip("tests/golden/reference_cublas.npz not generated yet")
    g = np.load(path)
    for i, (M, N, K) in enumerate(g["cases"]):
        M, N, K = int(M), int(N), int(K)
        for dt, sfx in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
            bf = dt == torch.bfloat16
            A = oracle.normal((M, K), 101 + 10 * i, bf16=bf)
            B = oracle.normal((K, N), 102 + 10 * i, std=0.02, bf16=bf)
            dC = oracle.normal((M, N), 103 + 10 * i, bf16=bf)
            old = oracle.normal((K, N), 104 + 10 * i, bf16=bf)
            c = torch.empty(M, N, device=DEV, dtype=dt)
            da = torch.empty(M, K, device=DEV, dtype=dt)
            db = dev(old, dt)
            pkg.matmul_forward(handle, c, dev(A, dt), dev(B, dt), M, N, K)
            pkg.matmul_backward(handle, da, db, dev(dC, dt), dev(A, dt), dev(B, dt), M, N, K)
            handle.sync()
            for got, name in ((c, "fwd"), (da, "dgrad"), (db, "wgrad")):
                want = g[f"{sfx}_{i}_{name}"]
                if bf:
                    want = (want.astype(np.uint32) << 16).view(np.float32)
                assert rel_err(got, want.astype(np.float64)) <= (8e-3 if bf else 1e-5), (sfx, i, name)


@pytest.mark.gpu
@pytest.mark.parametrize("sm_dgrad", [0, 24, 48, 100, 140])
def test_backward_side_by_side_on_sm_shares(pkg, handle, oracle, sm_dgrad):
    """matmul_backward with dgrad and wgrad on complementary shares of the SMs (0 = the cost model's choice):
    same results as the oracle for every share, dB accumulated over two calls."""
    rng = np.random.default_rng(sm_dgrad)
    dt = torch.bfloat16
    try:
        handle.force_backward_split(sm_dgrad)
        for M, N, K in ((8192, 768, 768), (8192, 256, 768), (4096, 2048, 768), (1000, 768, 2048)):
            A, B, dC = inputs(oracle, M, N, K, 3000 + N + sm_dgrad, True)
            a, b, dc = dev(A, dt), dev(B, dt), dev(dC, dt)
            da = torch.empty(M, K, device=DEV, dtype=dt)
            db = torch.zeros(K, N, device=DEV, dtype=dt)
            pkg.matmul_backward(handle, da, db, dc, a, b, M, N, K)
            pkg.matmul_backward(handle, da, db, dc, a, b, M, N, K)
            handle.sync()
            for which, got, x, y, mult in ((1, da, dC, B, 1.0), (2, db, A, dC, 2.0)):
                rows, cols = got.shape
                r, cc = _sample_points(rng, rows, cols)
                want = mult * oracle.gemm_f64_samples(which, x, y, M, N, K, r, cc)
                g = got.float().cpu().numpy()[r, cc].astype(np.float64)
                assert np.abs(g - want).max() / np.abs(want).max() <= 1e-2, (sm_dgrad, which, M, N, K)
    finally:
        handle.force_backward_split(0)
