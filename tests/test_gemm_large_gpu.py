"""Largest shapes of the baseline's configurations, checked through size-independent properties
(exact copies through a selection-matrix weight) and sampled fp64 values."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_llama3_lm_head_full_size_forward_is_exact_for_selection_weights(pkg, handle):
    """Config 4's LM head: [16384 tokens, 768] x [768, 128256]; a 0/1 selection matrix as weight makes
    every logit a copy of one input element, so all 2.1e9 outputs can be checked bit for bit."""
    dt = torch.bfloat16
    M, N, K = 16384, 128256, 768
    g = torch.Generator(device=DEV).manual_seed(11)
    a = torch.randn(M, K, device=DEV, generator=g).to(dt)
    sel = torch.randint(0, K, (N,), device=DEV, generator=g)
    b = torch.zeros(K, N, device=DEV, dtype=dt)
    b[sel, torch.arange(N, device=DEV)] = 1
    c = torch.empty(M, N, device=DEV, dtype=dt)
    pkg.matmul_forward(handle, c, a, b, M, N, K)
    handle.sync()
    for r0 in range(0, M, 2048):  # compare in slabs to bound the temporary
        assert torch.equal(c[r0:r0 + 2048], a[r0:r0 + 2048][:, sel])
    del c, b
    torch.cuda.empty_cache()


def test_llama3_lm_head_backward_sampled(pkg, handle, oracle):
    """dX and dW of the same LM head at M = 4096 tokens against sampled fp64 dot products."""
    dt = torch.bfloat16
    M, N, K = 4096, 128256, 768
    A = oracle.normal((M, K), 71, bf16=True)
    B = oracle.normal((K, N), 72, std=0.02, bf16=True)
    dC = oracle.normal((M, N), 73, bf16=True)
    a, b, dc = (torch.from_numpy(v).to(DEV, dt) for v in (A, B, dC))
    da = torch.empty(M, K, device=DEV, dtype=dt)
    db = torch.zeros(K, N, device=DEV, dtype=dt)
    pkg.matmul_backward(handle, da, db, dc, a, b, M, N, K)
    handle.sync()
    rng = np.random.default_rng(5)
    for which, got, x, y in ((1, da, dC, B), (2, db, A, dC)):
        rows, cols = got.shape
        r = rng.integers(0, rows, 2048).astype(np.int32)
        c = rng.integers(0, cols, 2048).astype(np.int32)
        want = oracle.gemm_f64_samples(which, x, y, M, N, K, r, c)
        g = got.float().cpu().numpy()[r, c].astype(np.float64)
        assert np.abs(g - want).max() / np.abs(want).max() <= 1e-2


def test_longest_token_dimension(pkg, handle):
    """M = 65536 tokens (the sweep's largest): wgrad contracts over all of them; B = I makes it checkable:
    dW = A^T dC with dC = one-hot rows picks and sums rows of A exactly when each sum has one term."""
    dt = torch.bfloat16
    M, N, K = 65536, 768, 768
    g = torch.Generator(device=DEV).manual_seed(3)
    a = torch.randn(M, K, device=DEV, generator=g).to(dt)
    eye = torch.eye(K, device=DEV, dtype=dt)
    c = torch.empty(M, N, device=DEV, dtype=dt)
    pkg.matmul_forward(handle, c, a, eye, M, N, K)
    da = torch.empty(M, K, device=DEV, dtype=dt)
    pkg.matmul_backward(handle, da, None, a, None, eye, M, N, K)  # dA = dC * I^T with dC := a
    handle.sync()
    assert torch.equal(c, a) and torch.equal(da, a)
    # wgrad: A = one-hot rows (row m selects column m % K): dW[k, :] = sum of dC rows with m % K == k
    onehot = torch.zeros(M, K, device=DEV, dtype=dt)
    onehot[torch.arange(M, device=DEV), torch.arange(M, device=DEV) % K] = 1
    dc = torch.randint(-3, 4, (M, N), device=DEV, generator=g).to(dt)  # small integers: sums are exact in fp32
    db = torch.zeros(K, N, device=DEV, dtype=dt)
    pkg.matmul_backward(handle, None, db, dc, onehot, None, M, N, K)
    handle.sync()
    want = dc.float().view(M // K if M % K == 0 else -1, K, N).sum(0) if M % K == 0 else None
    if want is None:
        want = torch.zeros(K, N, device=DEV)
        want.index_add_(0, torch.arange(M, device=DEV) % K, dc.float())
    assert torch.equal(db.float(), want)  # |sums| <= 3 * 86 fits bf16's integer range exactly
