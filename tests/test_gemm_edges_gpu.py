"""GPU edge cases and size-independent properties of the linear-layer GEMMs (through the C ABI)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(pkg, handle, which, beta, x, y, old, M, N, K):
    out = old.clone()
    pkg.gemm(handle, which, beta, out, x, y, M, N, K)
    handle.sync()
    return out


def _ref64(which, beta, x, y, old):
    xd, yd = x.double(), y.double()
    r = {0: lambda: xd @ yd, 1: lambda: xd @ yd.T, 2: lambda: xd.T @ yd}[which]()
    return r + old.double() if beta else r


def _shapes(which, M, N, K):
    ins = {0: ((M, K), (K, N)), 1: ((M, N), (K, N)), 2: ((M, K), (M, N))}[which]
    out = {0: (M, N), 1: (M, K), 2: (K, N)}[which]
    return ins, out


# ragged sizes: M free; N, K multiples of 8 (tensor-core path with tails) and not (CUDA-core path)
RAGGED = [(1, 8, 8), (127, 136, 72), (129, 264, 200), (1000, 520, 1032), (257, 250, 130), (33, 7, 5),
          (4100, 768, 24), (300, 8, 4096)]


@pytest.mark.parametrize("which", [0, 1, 2])
@pytest.mark.parametrize("dt,tol", [(torch.bfloat16, 1e-2), (torch.float32, 1e-5)])
def test_ragged_shapes(pkg, handle, which, dt, tol):
    g = torch.Generator(device=DEV).manual_seed(1234 + which)
    for (M, N, K) in RAGGED:
        ins, outs = _shapes(which, M, N, K)
        x = torch.randn(ins[0], device=DEV, generator=g).to(dt)
        y = torch.randn(ins[1], device=DEV, generator=g).to(dt)
        old = torch.randn(outs, device=DEV, generator=g).to(dt)
        for beta in (0, 1):
            got = _run(pkg, handle, which, beta, x, y, old, M, N, K)
            want = _ref64(which, beta, x, y, old)
            err = ((got.double() - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()
            assert err <= tol, (which, dt, M, N, K, beta, err)


@pytest.mark.parametrize("bn,pair", [(64, 0), (128, 0), (192, 0), (256, 0), (128, 1), (256, 1)])
@pytest.mark.parametrize("which", [0, 1, 2])
def test_every_tile_shape_and_split(pkg, handle, which, bn, pair):
    """Each tile width, single CTA and CTA pair, with and without split-K, beta 0 and 1."""
    g = torch.Generator(device=DEV).manual_seed(99)
    dt = torch.bfloat16
    try:
        for (M, N, K) in [(384, 512, 320), (1000, 264, 136), (2048, 768, 768)]:
            ins, outs = _shapes(which, M, N, K)
            x = torch.randn(ins[0], device=DEV, generator=g).to(dt)
            y = torch.randn(ins[1], device=DEV, generator=g).to(dt)
            old = torch.randn(outs, device=DEV, generator=g).to(dt)
            for splits, beta in ((1, 0), (1, 1), (3, 0), (2, 1)):
                handle.force_plan(bn, pair, splits)
                got = _run(pkg, handle, which, beta, x, y, old, M, N, K)
                want = _ref64(which, beta, x, y, old)
                err = ((got.double() - want).abs().max() / want.abs().max()).item()
                assert err <= 1e-2, (which, bn, pair, splits, beta, M, N, K, err)
    finally:
        handle.force_plan(-1, 0, 0)


@pytest.mark.parametrize("bn,pair,members", [(256, 0, 2), (256, 0, 3), (256, 0, 8), (192, 0, 3), (128, 0, 4), (64, 0, 2),
                                             (256, 1, 2), (256, 1, 3), (256, 1, 4), (128, 1, 4)])
@pytest.mark.parametrize("which", [0, 1, 2])
def test_cluster_split_through_distributed_shared_memory(pkg, handle, which, bn, pair, members):
    """Every tile shared by a cluster whose members each take one range of the contraction and add
    their partial sums up through distributed shared memory (no global-memory round trip)."""
    g = torch.Generator(device=DEV).manual_seed(77)
    dt = torch.bfloat16
    try:
        for (M, N, K) in [(512, 256, 512), (1000, 264, 520), (2048, 768, 768)]:
            ins, outs = _shapes(which, M, N, K)
            x = torch.randn(ins[0], device=DEV, generator=g).to(dt)
            y = torch.randn(ins[1], device=DEV, generator=g).to(dt)
            old = torch.randn(outs, device=DEV, generator=g).to(dt)
            for beta in (0, 1):
                handle.force_plan(bn, pair, -members)
                got = _run(pkg, handle, which, beta, x, y, old, M, N, K)
                want = _ref64(which, beta, x, y, old)
                err = ((got.double() - want).abs().max() / want.abs().max()).item()
                assert err <= 1e-2, (which, bn, pair, members, beta, M, N, K, err)
                again = _run(pkg, handle, which, beta, x, y, old, M, N, K)
                assert torch.equal(got, again)  # member order, not arrival order, fixes the sum
    finally:
        handle.force_plan(-1, 0, 0)


def test_identity_weight_is_exact(pkg, handle):
    """B = I: forward returns A and dgrad returns dC bit for bit; A = I: wgrad returns dC + old."""
    dt = torch.bfloat16
    M = N = K = 1024
    g = torch.Generator(device=DEV).manual_seed(5)
    a = torch.randn(M, K, device=DEV, generator=g).to(dt)
    eye = torch.eye(K, device=DEV, dtype=dt)
    c = torch.empty(M, N, device=DEV, dtype=dt)
    pkg.matmul_forward(handle, c, a, eye, M, N, K)
    da = torch.empty(M, K, device=DEV, dtype=dt)
    db = torch.zeros(K, N, device=DEV, dtype=dt)
    pkg.matmul_backward(handle, da, db, a, eye, eye, M, N, K)  # dC := a, A := I
    handle.sync()
    assert torch.equal(c, a)
    assert torch.equal(da, a)
    assert torch.equal(db, a)


def test_permutation_at_full_lm_head_width(pkg, handle):
    """At the 32000-wide LM head: a 0/1 selection matrix as weight makes every output element a
    copy of one input element, so the result is exact at any size."""
    dt = torch.bfloat16
    M, N, K = 8192, 32000, 768
    g = torch.Generator(device=DEV).manual_seed(6)
    a = torch.randn(M, K, device=DEV, generator=g).to(dt)
    sel = torch.randint(0, K, (N,), device=DEV, generator=g)
    b = torch.zeros(K, N, device=DEV, dtype=dt)
    b[sel, torch.arange(N, device=DEV)] = 1
    c = torch.empty(M, N, device=DEV, dtype=dt)
    pkg.matmul_forward(handle, c, a, b, M, N, K)
    handle.sync()
    assert torch.equal(c, a[:, sel])


def test_zero_inputs_and_beta(pkg, handle):
    dt = torch.bfloat16
    M, N, K = 512, 256, 384
    z = torch.zeros(M, K, device=DEV, dtype=dt)
    dc = torch.randn(M, N, device=DEV).to(dt)
    old = torch.randn(K, N, device=DEV).to(dt)
    db = old.clone()
    pkg.matmul_backward(handle, None, db, dc, z, None, M, N, K)  # A = 0: dB unchanged by beta=1
    handle.sync()
    assert torch.equal(db, old)
    out = torch.full((K, N), 7.0, device=DEV, dtype=dt)
    pkg.gemm(handle, 2, 0, out, z, dc, M, N, K)                    # beta = 0 overwrites
    handle.sync()
    assert not out.any()


@pytest.mark.parametrize("which", [0, 1, 2])
def test_run_to_run_determinism(pkg, handle, which):
    dt = torch.bfloat16
    M, N, K = 8192, 768, 768
    ins, outs = _shapes(which, M, N, K)
    x = torch.randn(ins[0], device=DEV).to(dt)
    y = torch.randn(ins[1], device=DEV).to(dt)
    old = torch.randn(outs, device=DEV).to(dt)
    first = _run(pkg, handle, which, 1, x, y, old, M, N, K)
    for _ in range(3):
        assert torch.equal(_run(pkg, handle, which, 1, x, y, old, M, N, K), first)


def test_linearity_in_fp32(pkg, handle):
    M, N, K = 640, 384, 256
    x1 = torch.randn(M, K, device=DEV)
    x2 = torch.randn(M, K, device=DEV)
    y = torch.randn(K, N, device=DEV)
    z = torch.zeros(M, N, device=DEV)
    s = _run(pkg, handle, 0, 0, x1, y, z, M, N, K) + _run(pkg, handle, 0, 0, x2, y, z, M, N, K)
    t = _run(pkg, handle, 0, 0, x1 + x2, y, z, M, N, K)
    assert ((s - t).abs().max() / t.abs().max()).item() <= 1e-5


def test_bad_arguments_return_errors(pkg, handle):
    t = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    for args in ((t, t, t, 0, 64, 64), (t, t, t, 64, -1, 64), (t, t, t, 64, 64, 0)):
        with pytest.raises(pkg.LinearError) as e:
            pkg.matmul_forward(handle, *args)
        assert e.value.code == 1
    with pytest.raises(pkg.LinearError):
        pkg.matmul_forward(handle, None, t, t, 64, 64, 64)
    with pytest.raises(pkg.LinearError):
        pkg.matmul_backward(handle, None, None, t, t, t, 64, 64, 64)
    with pytest.raises(pkg.LinearError):
        pkg.gemm(handle, 7, 0, t, t, t, 64, 64, 64)
    with pytest.raises(pkg.LinearError):
        pkg.matmul_forward(handle, t, t.cpu(), t, 64, 64, 64)
    handle.sync()  # the context is still usable
    pkg.matmul_forward(handle, t, t, t, 64, 64, 64)
    handle.sync()


def test_launch_counter_counts_our_kernels(pkg, handle):
    t = torch.zeros(256, 256, device=DEV, dtype=torch.bfloat16)
    before = handle.launches
    pkg.matmul_forward(handle, t.clone(), t, t, 256, 256, 256)
    handle.sync()
    assert handle.launches > before


def test_misaligned_pointers_take_the_cuda_core_path(pkg, handle):
    dt = torch.bfloat16
    M, N, K = 200, 72, 40
    buf = torch.randn(M * K + 1, device=DEV).to(dt)
    a = buf[1:].view(M, K)  # 2-byte aligned only
    b = torch.randn(K, N, device=DEV).to(dt)
    c = torch.empty(M, N, device=DEV, dtype=dt)
    pkg.matmul_forward(handle, c, a.data_ptr(), b, M, N, K, dtype="bf16")
    handle.sync()
    want = a.double() @ b.double()
    assert ((c.double() - want).abs().max() / want.abs().max()).item() <= 1e-2


@pytest.mark.parametrize("which", [0, 1, 2])
def test_column_ranges_of_wider_matrices(pkg, handle, which):
    """Operands with a row pitch: the weight (and its gradient) as a column range of a wider matrix, which is
    how a rank works on its vocabulary shard of the LM head in place.  Every plan variant the dispatcher may
    pick for such a shard, plus the automatic one; columns outside the range must stay untouched."""
    dt = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(321 + which)
    M, K, V, c0, N = 1024, 768, 2304, 512, 1280
    a = torch.randn(M, K, device=DEV, generator=g).to(dt)
    w_full = (0.05 * torch.randn(K, V, device=DEV, generator=g)).to(dt)
    dc_full = torch.randn(M, V, device=DEV, generator=g).to(dt)      # logits-like buffer, also pitched
    w, dc = w_full[:, c0:c0 + N], dc_full[:, c0:c0 + N]
    try:
        for plan in (None, (256, 1, 0), (128, 0, 2), (192, 0, 0), (128, 0, -2)):
            if plan:
                handle.force_plan(*plan)
            for beta in (0, 1):
                if which == 0:      # logits shard = a @ w, written into a column range of a [M, V] buffer
                    out_full = torch.randn(M, V, device=DEV, generator=g).to(dt)
                    keep = out_full.clone()
                    out = out_full[:, c0:c0 + N]
                    want = a.double() @ w.double() + (keep[:, c0:c0 + N].double() if beta else 0)
                    pkg.gemm_ld(handle, 0, beta, out, a, w, M, N, K)
                elif which == 1:    # d(input) = dlogits shard @ w^T, dense output
                    out_full = torch.randn(M, K, device=DEV, generator=g).to(dt)
                    keep = out_full.clone()
                    out = out_full
                    want = dc.double() @ w.double().T + (keep.double() if beta else 0)
                    pkg.gemm_ld(handle, 1, beta, out, dc, w, M, N, K)
                else:               # dW shard += a^T @ dlogits shard, written into a column range of dW [K, V]
                    out_full = torch.randn(K, V, device=DEV, generator=g).to(dt)
                    keep = out_full.clone()
                    out = out_full[:, c0:c0 + N]
                    want = a.double().T @ dc.double() + (keep[:, c0:c0 + N].double() if beta else 0)
                    pkg.gemm_ld(handle, 2, beta, out, a, dc, M, N, K)
                handle.sync()
                err = ((out.double() - want).abs().max() / want.abs().max()).item()
                assert err <= 1e-2, (which, plan, beta, err)
                if which != 1:      # nothing outside the column range was written
                    assert torch.equal(out_full[:, :c0], keep[:, :c0])
                    assert torch.equal(out_full[:, c0 + N:], keep[:, c0 + N:])
    finally:
        handle.force_plan(-1, 0, 0)
    # pitches the tensor maps cannot describe are refused, not silently mis-read
    with pytest.raises(pkg.LinearError):
        pkg.gemm_ld(handle, 0, 0, (a.data_ptr(), N), a, (w.data_ptr(), V + 4), M, N, K)
    with pytest.raises(pkg.LinearError):
        pkg.gemm_ld(handle, 0, 0, (a.data_ptr(), N - 8), a, w, M, N, K)


def test_bounded_wait_that_runs_out_is_reported_and_the_context_survives(pkg, handle, oracle):
    """A device wait that gives up: the probe kernel waits about a millisecond on a barrier that nothing
    completes, records its code and returns.  The next sync reports B200_E_DEVICE_WAIT (code 4) once, clears
    it, and an ordinary product on the same context is correct afterwards.  Nothing faults or hangs."""
    handle.sync()
    handle.selftest_wait_timeout(2_000_000)
    with pytest.raises(pkg.LinearError) as e:
        handle.sync()
    assert e.value.code == 4 and "102" in str(e.value)   # DEV_TIMEOUT_FULL is what the probe records
    handle.sync()                                          # cleared: the second sync is clean
    M, N, K = 512, 768, 2048
    A = oracle.normal((M, K), 71, bf16=True)
    dC = oracle.normal((M, N), 72, bf16=True)
    a, dc = (torch.from_numpy(v).to(DEV, torch.bfloat16) for v in (A, dC))
    db = torch.zeros(K, N, device=DEV, dtype=torch.bfloat16)
    pkg.gemm(handle, 2, 1, db, a, dc, M, N, K)              # a split product: uses the counters sync() reset
    handle.sync()
    want = oracle.gemm_f64(2, A, dC, M, N, K)
    assert np.abs(db.float().cpu().numpy() - want).max() / np.abs(want).max() <= 1e-2
    with pytest.raises(pkg.LinearError):
        handle.selftest_wait_timeout(0)


def test_context_belongs_to_its_device(pkg, handle):
    """A context is tied to the device that was current when it was created (its kernels' shared-memory opt-in, scratch
    and tensor maps are that device's): a call made with another device current is refused, and a second context on the
    second device works (the opt-in is tracked per device)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    dt = torch.bfloat16
    a0 = torch.randn(256, 256, device="cuda:0").to(dt)
    try:
        torch.cuda.set_device(1)
        with pytest.raises(pkg.LinearError) as e:
            pkg.matmul_forward(handle, a0.clone(), a0, a0, 256, 256, 256)
        assert e.value.code == 1
        h1 = pkg.Handle()
        a1 = torch.randn(512, 768, device="cuda:1").to(dt)
        b1 = torch.randn(768, 512, device="cuda:1").to(dt)
        c1 = torch.empty(512, 512, device="cuda:1", dtype=dt)
        pkg.matmul_forward(h1, c1, a1, b1, 512, 512, 768)
        h1.sync()
        want = a1.double() @ b1.double()
        assert ((c1.double() - want).abs().max() / want.abs().max()).item() <= 1e-2
        h1.destroy()
    finally:
        torch.cuda.set_device(0)
    pkg.matmul_forward(handle, a0.clone(), a0, a0, 256, 256, 256)
    handle.sync()


def _rel(got, want):
    return ((got.double() - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()


GROUPS = [(8192, (768, 256, 256), 768),     # Q, K, V of the 125M model
          (2048, (2048, 2048), 768),        # gate, up
          (1000, (128, 64, 192), 320),      # ragged token count, three different widths
          (384, (1024, 256), 1024),         # llama3-like K / V widths
          (520, (72, 136), 264)]            # widths that are not multiples of 64: runs as single products


@pytest.mark.parametrize("M,Ns,K", GROUPS)
def test_grouped_forward_and_weight_gradient(pkg, handle, M, Ns, K):
    """Several products on one input in one launch: Y_i = X W_i and dW_i += X^T dY_i, against float64 and against the
    single-product entry point (same arithmetic: equal up to the order of fp32 partial sums where the contraction is split)."""
    g = torch.Generator(device=DEV).manual_seed(4321)
    dt = torch.bfloat16
    x = torch.randn(M, K, device=DEV, generator=g).to(dt)
    ws = [torch.randn(K, n, device=DEV, generator=g).to(dt) for n in Ns]
    outs = [torch.full((M, n), float("nan"), device=DEV, dtype=dt) for n in Ns]
    pkg.gemm_grouped(handle, pkg.FWD_NN, 0, outs, x, ws, M, list(Ns), K)
    handle.sync()
    for o, w, n in zip(outs, ws, Ns):
        assert _rel(o, x.double() @ w.double()) <= 1e-2
        single = torch.empty_like(o)
        pkg.gemm(handle, pkg.FWD_NN, 0, single, x, w, M, n, K)
        handle.sync()
        assert _rel(o, single.double()) <= 4e-3
    dys = [torch.randn(M, n, device=DEV, generator=g).to(dt) for n in Ns]
    olds = [torch.randn(K, n, device=DEV, generator=g).to(dt) for n in Ns]
    for beta in (0, 1):
        dws = [o.clone() for o in olds]
        pkg.gemm_grouped(handle, pkg.WGRAD_TN, beta, dws, x, dys, M, list(Ns), K)
        handle.sync()
        for dw, dy, old in zip(dws, dys, olds):
            prod = x.double().T @ dy.double()
            # beta = 1 rounds like the reference's cuBLAS call: bf16(bf16(product) + old)
            want = (prod.to(dt).double() + old.double()) if beta else prod
            assert _rel(dw, want) <= 1e-2, (beta, _rel(dw, want))


@pytest.mark.parametrize("M,Ns,K", GROUPS)
def test_grouped_input_gradient_is_one_sum(pkg, handle, M, Ns, K):
    """dX (+)= sum_i dY_i W_i^T through one accumulator: the float64 sum rounded once."""
    g = torch.Generator(device=DEV).manual_seed(8765)
    dt = torch.bfloat16
    dys = [torch.randn(M, n, device=DEV, generator=g).to(dt) for n in Ns]
    ws = [torch.randn(K, n, device=DEV, generator=g).to(dt) for n in Ns]
    old = torch.randn(M, K, device=DEV, generator=g).to(dt)
    total = sum(dy.double() @ w.double().T for dy, w in zip(dys, ws))
    for beta in (0, 1):
        dx = old.clone()
        pkg.gemm_grouped(handle, pkg.DGRAD_NT, beta, dx, dys, ws, M, list(Ns), K)
        handle.sync()
        assert _rel(dx, total + old.double() if beta else total) <= 1e-2, (beta,)
    if all(n % 64 == 0 for n in Ns):   # the one-launch path: a single rounding, so far tighter than three
        dx = torch.empty_like(old)
        pkg.gemm_grouped(handle, pkg.DGRAD_NT, 0, dx, dys, ws, M, list(Ns), K)
        handle.sync()
        assert torch.equal(dx, total.to(dt)) or _rel(dx, total) <= 4e-3


@pytest.mark.parametrize("bn,pair,splits", [(64, 0, 1), (128, 0, 1), (256, 0, 1), (128, 1, 1), (256, 1, 1), (128, 0, 3), (256, 1, 2),
                                            (64, 0, -2), (128, 1, -3)])
def test_grouped_launch_with_every_tile_shape_and_split(pkg, handle, bn, pair, splits):
    """The grouped launches under forced tile widths, CTA pairs, split contraction (workspace and cluster)."""
    g = torch.Generator(device=DEV).manual_seed(2468)
    dt = torch.bfloat16
    M, Ns, K = 1536, (768, 256, 256), 768
    x = torch.randn(M, K, device=DEV, generator=g).to(dt)
    ws = [torch.randn(K, n, device=DEV, generator=g).to(dt) for n in Ns]
    dys = [torch.randn(M, n, device=DEV, generator=g).to(dt) for n in Ns]
    olds = [torch.randn(K, n, device=DEV, generator=g).to(dt) for n in Ns]
    try:
        handle.force_plan(bn, pair, splits)
        outs = [torch.empty(M, n, device=DEV, dtype=dt) for n in Ns]
        pkg.gemm_grouped(handle, pkg.FWD_NN, 0, outs, x, ws, M, list(Ns), K)
        dws = [o.clone() for o in olds]
        pkg.gemm_grouped(handle, pkg.WGRAD_TN, 1, dws, x, dys, M, list(Ns), K)
        dx = torch.empty(M, K, device=DEV, dtype=dt)
        pkg.gemm_grouped(handle, pkg.DGRAD_NT, 0, dx, dys, ws, M, list(Ns), K)
        handle.sync()
    finally:
        handle.force_plan(-1, 0, 0)
    for o, w in zip(outs, ws):
        assert _rel(o, x.double() @ w.double()) <= 1e-2
    for dw, dy, old in zip(dws, dys, olds):
        assert _rel(dw, (x.double().T @ dy.double()).to(dt).double() + old.double()) <= 1e-2
    assert _rel(dx, sum(dy.double() @ w.double().T for dy, w in zip(dys, ws))) <= 1e-2


def test_grouped_backward_matches_separate_calls(pkg, handle):
    """matmul_backward for a group (dA = sum, dB_i += ...; two launches side by side) against matmul_backward per product
    with the input gradients added in float64."""
    g = torch.Generator(device=DEV).manual_seed(1357)
    dt = torch.bfloat16
    M, Ns, K = 4096, (768, 256, 256), 768
    a = torch.randn(M, K, device=DEV, generator=g).to(dt)
    bs = [torch.randn(K, n, device=DEV, generator=g).to(dt) for n in Ns]
    dcs = [torch.randn(M, n, device=DEV, generator=g).to(dt) for n in Ns]
    olds = [torch.randn(K, n, device=DEV, generator=g).to(dt) for n in Ns]
    dbs = [o.clone() for o in olds]
    da = torch.empty(M, K, device=DEV, dtype=dt)
    pkg.matmul_backward_grouped(handle, da, dbs, dcs, a, bs, M, list(Ns), K)
    handle.sync()
    da_sum = torch.zeros(M, K, dtype=torch.float64, device=DEV)
    for b, dc, old, db, n in zip(bs, dcs, olds, dbs, Ns):
        da1, db1 = torch.empty(M, K, device=DEV, dtype=dt), old.clone()
        pkg.matmul_backward(handle, da1, db1, dc, a, b, M, n, K)
        handle.sync()
        da_sum += da1.double()
        assert _rel(db, db1.double()) <= 4e-3
    assert _rel(da, da_sum) <= 1e-2


@pytest.mark.parametrize("M,ff,K", [(8192, 2048, 768), (1000, 384, 320), (130, 128, 64), (4096, 1024, 1024)])
def test_swiglu_forward_in_the_gemm_epilogue(pkg, handle, M, ff, K):
    """gate, up, hidden from one launch: gate and up equal the single-product results bit for bit (same tile arithmetic,
    whole tiles), hidden equals SiLU(gate) * up formed from those bf16 values (float64 reference, one bf16 rounding)."""
    g = torch.Generator(device=DEV).manual_seed(97531)
    dt = torch.bfloat16
    x = torch.randn(M, K, device=DEV, generator=g).to(dt)
    wg = (torch.randn(K, ff, device=DEV, generator=g) / K ** 0.5).to(dt)
    wu = (torch.randn(K, ff, device=DEV, generator=g) / K ** 0.5).to(dt)
    gate, up, hidden = (torch.full((M, ff), float("nan"), device=DEV, dtype=dt) for _ in range(3))
    pkg.swiglu_forward_gemm(handle, gate, up, hidden, x, wg, wu, M, ff, K)
    handle.sync()
    assert _rel(gate, x.double() @ wg.double()) <= 1e-2 and _rel(up, x.double() @ wu.double()) <= 1e-2
    g1, u1 = torch.empty_like(gate), torch.empty_like(up)
    pkg.gemm(handle, pkg.FWD_NN, 0, g1, x, wg, M, ff, K)
    pkg.gemm(handle, pkg.FWD_NN, 0, u1, x, wu, M, ff, K)
    handle.sync()
    assert _rel(gate, g1.double()) <= 4e-3 and _rel(up, u1.double()) <= 4e-3
    g64, u64 = gate.double(), up.double()
    want = g64 * torch.sigmoid(g64) * u64
    assert _rel(hidden, want) <= 4e-3
    # one bf16 rounding of the float64 value, up to the fast exponential: at most one unit in the last place
    ulp = (hidden.double() - want).abs() / want.abs().clamp_min(1e-30)
    assert ulp[want.abs() > 1e-3].max().item() <= 2 ** -7


def test_swiglu_forward_gemm_refuses_what_it_cannot_tile(pkg, handle):
    x = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(64, 72, device=DEV, dtype=torch.bfloat16)
    o = torch.zeros(64, 72, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(pkg.LinearError):
        pkg.swiglu_forward_gemm(handle, o, o.clone(), o.clone(), x, w, w, 64, 72, 64)
