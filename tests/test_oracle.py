"""The CPU oracle against fixtures it did not produce: numpy float64 products, torch's bf16
rounding, and (when the fixture is present) outputs of the reference's own cuBLAS build."""
import os

import numpy as np
import pytest

from conftest import GOLDEN


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLDEN, "numpy_f64.npz"))


@pytest.mark.parametrize("case", range(5))
def test_f64_products_match_numpy(oracle, gold, case):
    M, N, K = (int(v) for v in gold[f"c{case}_dims"])
    A, B, dC, old = (gold[f"c{case}_{n}"] for n in ("A", "B", "dC", "old"))
    fwd = oracle.gemm_f64(oracle.FWD_NN, A, B, M, N, K)
    dgrad = oracle.gemm_f64(oracle.DGRAD_NT, dC, B, M, N, K)
    wgrad = oracle.gemm_f64(oracle.WGRAD_TN, A, dC, M, N, K, old=old)
    # same float64 arithmetic, different summation order: agree to ~1e-13 relative
    for got, name in ((fwd, "fwd"), (dgrad, "dgrad"), (wgrad, "wgrad")):
        want = gold[f"c{case}_{name}"]
        assert got.shape == want.shape
        assert np.abs(got - want).max() <= 1e-12 * max(1.0, np.abs(want).max())


def test_samples_match_full(oracle, gold):
    M, N, K = (int(v) for v in gold["c2_dims"])
    A, B, dC = gold["c2_A"], gold["c2_B"], gold["c2_dC"]
    rng = np.random.default_rng(1)
    for which, x, y in ((0, A, B), (1, dC, B), (2, A, dC)):
        full = oracle.gemm_f64(which, x, y, M, N, K)
        r = rng.integers(0, full.shape[0], 200).astype(np.int32)
        c = rng.integers(0, full.shape[1], 200).astype(np.int32)
        got = oracle.gemm_f64_samples(which, x, y, M, N, K, r, c)
        assert np.abs(got - full[r, c]).max() <= 1e-12


def test_f32_host_gemm_matches_f64(oracle, gold):
    for case in range(5):
        M, N, K = (int(v) for v in gold[f"c{case}_dims"])
        A, B, dC, old = (gold[f"c{case}_{n}"] for n in ("A", "B", "dC", "old"))
        for which, x, y, name, beta in ((0, A, B, "fwd", 0), (1, dC, B, "dgrad", 0), (2, A, dC, "wgrad", 1)):
            out = old.copy() if beta else np.zeros(oracle.out_shape(which, M, N, K), np.float32)
            oracle.gemm_f32(which, beta, out, x, y, M, N, K)
            want = gold[f"c{case}_{name}"]
            assert np.abs(out - want).max() <= 1e-5 * max(1e-6, np.abs(want).max())


def test_round_bf16_matches_torch(oracle, gold):
    got = oracle.round_bf16(gold["round_in"])
    want = gold["round_out_torch"]
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_generator_is_pinned_and_counter_based(oracle, gold):
    a = oracle.normal((64,), 7)
    assert np.array_equal(a, gold["normal_seed7_first64"])
    b = oracle.normal((4, 1000), 7)
    assert np.array_equal(b.reshape(-1)[:64], a)  # element i depends on (seed, i) only
    big = oracle.normal((200000,), 9, std=0.02, mean=0.5)
    assert abs(big.mean() - 0.5) < 3e-4 and abs(big.std() - 0.02) < 2e-4


def test_linearity_and_zero(oracle):
    M, N, K = 33, 24, 17
    x1, x2 = oracle.normal((M, K), 1), oracle.normal((M, K), 2)
    y = oracle.normal((K, N), 3)
    s = oracle.gemm_f64(0, x1, y, M, N, K) + oracle.gemm_f64(0, x2, y, M, N, K)
    t = oracle.gemm_f64(0, (x1.astype(np.float64) + x2).astype(np.float32), y, M, N, K)
    assert np.abs(s - t).max() < 1e-5
    assert not oracle.gemm_f64(0, np.zeros((M, K), np.float32), y, M, N, K).any()


def test_bad_arguments_rejected(oracle):
    with pytest.raises(ValueError):
        oracle.gemm_f64(5, np.zeros((2, 2), np.float32), np.zeros((2, 2), np.float32), 2, 2, 2)
    with pytest.raises(ValueError):
        oracle.gemm_f64(0, np.zeros((2, 2), np.float32), np.zeros((2, 2), np.float32), 0, 2, 2)


def test_against_reference_cublas_outputs(oracle):
    """Pins the oracle to the reference itself: outputs of the reference's unmodified matmul.cu
    (cuBLAS on a B200) on inputs regenerated here from (seed, shape).

    bf16, beta=0: the reference equals bf16_rn(product) (fp32 vs fp64 accumulation moves a few
    elements by one ulp).  bf16, beta=1: the reference equals bf16_rn(bf16_rn(product) + dB_old),
    i.e. it rounds the product to bf16 before adding the old gradient."""
    path = os.path.join(GOLDEN, "reference_cublas.npz")
    if not os.path.exists(path):
        pytest.skip("tests/golden/reference_cublas.npz not generated yet")
    g = np.load(path)
    for i, (M, N, K) in enumerate(g["cases"]):
        M, N, K = int(M), int(N), int(K)
        for sfx, tol in (("bf16", 1e-2), ("f32", 1e-5)):
            bf = sfx == "bf16"
            A = oracle.normal((M, K), 101 + 10 * i, bf16=bf)
            B = oracle.normal((K, N), 102 + 10 * i, std=0.02, bf16=bf)
            dC = oracle.normal((M, N), 103 + 10 * i, bf16=bf)
            old = oracle.normal((K, N), 104 + 10 * i, bf16=bf)
            prod = {"fwd": oracle.gemm_f64(0, A, B, M, N, K), "dgrad": oracle.gemm_f64(1, dC, B, M, N, K),
                    "wgrad": oracle.gemm_f64(2, A, dC, M, N, K)}
            for name, w in prod.items():
                got = g[f"{sfx}_{i}_{name}"]
                exact = w + old if name == "wgrad" else w
                if bf:
                    got = (got.astype(np.uint32) << 16).view(np.float32)
                    model = oracle.reference_bf16_result(w, old if name == "wgrad" else None)
                    assert (got == model).mean() >= 0.99, (i, name)
                    ulp = np.abs(model) * 2.0 ** -7 + 2.0 ** -8 * np.abs(w) * (name == "wgrad") + 1e-30
                    assert (np.abs(got - model) <= ulp).all(), (i, name)
                err = np.abs(got.astype(np.float64) - exact).max() / np.abs(exact).max()
                assert err <= tol, (sfx, i, name, err)
