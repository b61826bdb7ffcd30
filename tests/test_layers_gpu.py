"""GPU parity tests of the layer drop-ins (attention with the fused softmax(QK^T)V core, RoPE, SwiGLU, whole-row
cross-entropy), called through the C ABI of include/b200_layers.h, against
  * oracle/layers_oracle.py -- the float64 restatement of the reference's layer mathematics, and
  * the reference's own, unmodified attention.cu / swiglu.cu / rope.cu / crossentropy.cu run live from oracle/_ref.

Error metric: max|x - x64| / max|x64| per tensor; tolerances 1e-2 for bf16 storage and 1e-5 for fp32 (the task's
tolerances for the GEMMs; 2e-5 where an fp32 result has gone through exp / rotation as well as GEMMs)."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.bfloat16: 1e-2, torch.float32: 2e-5}


def rel(got, want64):
    g = got.detach().double().cpu()
    return ((g - want64).abs().max() / want64.abs().max().clamp_min(1e-300)).item()


def rnd(shape, seed, dt, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (std * torch.randn(*shape, generator=g)).to(dt)


@pytest.fixture(scope="module")
def layers(pkg):
    import importlib
    return importlib.import_module(pkg.__name__ + ".layers")


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,T,nh,nkv", [(2, 256, 12, 4), (1, 130, 6, 2), (1, 64, 4, 4), (1, 1024, 3, 1), (3, 33, 2, 1),
                                       (1, 2100, 3, 1)])   # long enough for the forward kernel with four threads per row
def test_fused_attention_core_forward_and_backward(layers, handle, dt, B, T, nh, nkv):
    """context, lse, dq, dk, dv of the fused kernels against float64, including sequence lengths that are not a
    multiple of the tile, grouped (nh > nkv) and ungrouped heads; and run-to-run determinism of the backward."""
    from oracle import layers_oracle as lo
    hd = 64
    q, k, v = rnd((B * T, nh * hd), 1, dt), rnd((B * T, nkv * hd), 2, dt), rnd((B * T, nkv * hd), 3, dt)
    dctx = rnd((B * T, nh * hd), 4, dt)
    qd, kd, vd, dd = (t.to(DEV) for t in (q, k, v, dctx))
    ctx = torch.empty(B * T, nh * hd, device=DEV, dtype=dt)
    lse = torch.empty(B, nh, T, device=DEV, dtype=torch.float32)
    layers.flash_attention_forward(ctx, lse, qd, kd, vd, B, T, nh, nkv, hd)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    layers.flash_attention_backward(dq, dk, dv, dd, qd, kd, vd, lse, B, T, nh, nkv, hd, context=ctx)
    torch.cuda.synchronize()
    c64, l64 = lo.attention_core(q.double(), k.double(), v.double(), B, T, nh, nkv, hd)
    assert rel(ctx, c64) <= TOL[dt]
    assert (lse.double().cpu() - l64).abs().max().item() <= 1e-4
    g64 = lo.attention_core_grads(dctx.double(), q.double(), k.double(), v.double(), B, T, nh, nkv, hd)
    for got, want, name in zip((dq, dk, dv), g64, "qkv"):
        assert rel(got, want) <= TOL[dt], (name, rel(got, want))
    # the reference's argument list has no context: the call recomputes it and must give the same gradients
    dq2, dk2, dv2 = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    layers.flash_attention_backward(dq2, dk2, dv2, dd, qd, kd, vd, lse, B, T, nh, nkv, hd)
    torch.cuda.synchronize()
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


def test_rope_against_float64_and_its_inverse(layers):
    from oracle import layers_oracle as lo
    B, T, nh, nkv, hd = 2, 512, 12, 4, 64
    for theta in (10000.0, 500000.0):
        q, k = rnd((B * T, nh * hd), 5, torch.bfloat16), rnd((B * T, nkv * hd), 6, torch.bfloat16)
        qd, kd = q.to(DEV), k.to(DEV)
        layers.rope_forward(qd, kd, B, T, nh, nkv, hd, theta)
        torch.cuda.synchronize()
        assert rel(qd, lo.rope(q.double(), B, T, nh, hd, theta)) <= 4e-3      # one bf16 rounding
        assert rel(kd, lo.rope(k.double(), B, T, nkv, hd, theta)) <= 4e-3
        layers.rope_backward(qd, kd, B, T, nh, nkv, hd, theta)
        torch.cuda.synchronize()
        assert rel(qd, q.double()) <= 8e-3 and rel(kd, k.double()) <= 8e-3   # there and back: two roundings


def _attention_inputs(dt, B, T, C, nh, nkv):
    kv = C // nh * nkv
    inp = rnd((B * T, C), 11, dt)
    ws = [rnd(s, 12 + i, dt, std=0.05) for i, s in enumerate(((C, C), (C, kv), (C, kv), (C, C)))]
    dout = rnd((B * T, C), 17, dt)
    return inp, ws, dout


@pytest.mark.parametrize("env", [{"B200_ATTN_ROW_THREADS": "4"}, {"B200_ATTN_ROW_THREADS": "2"}, {"B200_ATTN_P_TMEM": "0"},
                                 {"B200_ATTN_DKV_TRANSPOSED": "1"}, {"B200_ATTN_DKV_TRANSPOSED": "1", "B200_ATTN_ROW_THREADS": "4"}])
@pytest.mark.parametrize("B,T,nh,nkv", [(2, 300, 6, 2), (1, 2100, 3, 1)])
def test_fused_attention_kernel_variants(layers, handle, monkeypatch, env, B, T, nh, nkv):
    """The tensor-core attention kernels in their other forms (two / four softmax threads per row, P and dS through shared
    memory instead of tensor memory, the dK / dV kernel with the keys on the TMEM lanes) against float64."""
    from oracle import layers_oracle as lo
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    dt, hd = torch.bfloat16, 64
    q, k, v = rnd((B * T, nh * hd), 1, dt), rnd((B * T, nkv * hd), 2, dt), rnd((B * T, nkv * hd), 3, dt)
    dctx = rnd((B * T, nh * hd), 4, dt)
    qd, kd, vd, dd = (t.to(DEV) for t in (q, k, v, dctx))
    ctx = torch.empty(B * T, nh * hd, device=DEV, dtype=dt)
    lse = torch.empty(B, nh, T, device=DEV, dtype=torch.float32)
    layers.flash_attention_forward(ctx, lse, qd, kd, vd, B, T, nh, nkv, hd)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    layers.flash_attention_backward(dq, dk, dv, dd, qd, kd, vd, lse, B, T, nh, nkv, hd, context=ctx)
    torch.cuda.synchronize()
    c64, l64 = lo.attention_core(q.double(), k.double(), v.double(), B, T, nh, nkv, hd)
    assert rel(ctx, c64) <= TOL[dt]
    assert (lse.double().cpu() - l64).abs().max().item() <= 1e-4
    g64 = lo.attention_core_grads(dctx.double(), q.double(), k.double(), v.double(), B, T, nh, nkv, hd)
    for got, want, name in zip((dq, dk, dv), g64, "qkv"):
        assert rel(got, want) <= TOL[dt], (env, name, rel(got, want))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,T,C,nh,nkv,theta", [(2, 256, 768, 12, 4, 10000.0), (1, 64, 256, 4, 2, 500000.0)])
def test_attention_layer_against_float64(layers, handle, dt, B, T, C, nh, nkv, theta):
    """attention_forward / attention_backward as the model calls them: forward, then backward with the same `att`
    buffer, the weight gradients accumulating over two calls.  T = 64 is the short-sequence case in which `att` is too
    small to keep the context and the backward pass recomputes it."""
    from oracle import layers_oracle as lo
    kv = C // nh * nkv
    inp, ws, dout = _attention_inputs(dt, B, T, C, nh, nkv)
    d = lambda t: t.to(DEV)
    inp_d, ws_d, dout_d = d(inp), [d(w) for w in ws], d(dout)
    out = torch.empty(B * T, C, device=DEV, dtype=dt)
    q, k, v = (torch.empty(B * T, n, device=DEV, dtype=dt) for n in (C, kv, kv))
    att = torch.zeros(B * nh * T * T, device=DEV, dtype=dt)
    layers.attention_forward(handle, out, q, k, v, att, inp_d, *ws_d, B, T, C, nh, nkv, theta)
    dinp = torch.empty_like(inp_d)
    dws = [torch.zeros_like(w) for w in ws_d]
    for _ in range(2):
        layers.attention_backward(handle, dinp, *dws, dout_d, inp_d, q, k, v, att, *ws_d, B, T, C, nh, nkv, theta)
    handle.sync()
    w64 = [w.double() for w in ws]
    o64, q64, k64, v64, _, _ = lo.attention_layer(inp.double(), *w64, B, T, C, nh, nkv, theta)
    tol = TOL[dt]
    assert rel(out, o64) <= tol and rel(q, q64) <= tol and rel(k, k64) <= tol and rel(v, v64) <= tol
    g64 = lo.attention_layer_grads(dout.double(), inp.double(), *w64, B, T, C, nh, nkv, theta)
    assert rel(dinp, g64[0]) <= tol
    for got, want in zip(dws, g64[1:]):
        assert rel(got, 2.0 * want) <= tol   # two backward calls accumulate (beta = 1)


def test_attention_layer_against_the_reference_kernels_live(layers, handle, ref_lib):
    """The reference's own attention.cu (with its rope.cu, softmax.cu and cuBLAS GEMMs) on the same inputs: both are
    within the bf16 tolerance of float64, and of each other within twice that."""
    if not hasattr(ref_lib, "ref_attention_forward_bf16"):
        pytest.skip("oracle/_ref was built without the reference's attention.cu")
    from oracle import layers_oracle as lo
    dt = torch.bfloat16
    B, T, C, nh, nkv, theta = 2, 256, 768, 12, 4, 10000.0
    kv = C // nh * nkv
    inp, ws, dout = _attention_inputs(dt, B, T, C, nh, nkv)
    inp_d, ws_d, dout_d = inp.to(DEV), [w.to(DEV) for w in ws], dout.to(DEV)
    vpt, ci = ctypes.c_void_p, ctypes.c_int
    ref_lib.ref_attention_forward_bf16.argtypes = [vpt] * 11 + [ci] * 5 + [ctypes.c_float]
    ref_lib.ref_attention_forward_bf16.restype = None
    ref_lib.ref_attention_backward_bf16.argtypes = [vpt] * 16 + [ci] * 5 + [ctypes.c_float]
    ref_lib.ref_attention_backward_bf16.restype = None
    hd = vpt()
    assert ref_lib.ref_create(ctypes.byref(hd)) == 0
    res = {}
    for name in ("ours", "reference"):
        out = torch.empty(B * T, C, device=DEV, dtype=dt)
        q, k, v = (torch.empty(B * T, n, device=DEV, dtype=dt) for n in (C, kv, kv))
        att = torch.zeros(B * nh * T * T, device=DEV, dtype=dt)
        dinp = torch.empty_like(inp_d)
        dws = [torch.zeros_like(w) for w in ws_d]
        p = lambda t: t.data_ptr()
        if name == "ours":
            layers.attention_forward(handle, out, q, k, v, att, inp_d, *ws_d, B, T, C, nh, nkv, theta)
            layers.attention_backward(handle, dinp, *dws, dout_d, inp_d, q, k, v, att, *ws_d, B, T, C, nh, nkv, theta)
            handle.sync()
        else:
            ref_lib.ref_attention_forward_bf16(hd, p(out), p(q), p(k), p(v), p(att), p(inp_d), *[p(w) for w in ws_d], B, T, C, nh,
                                               nkv, theta)
            ref_lib.ref_attention_backward_bf16(hd, p(dinp), *[p(w) for w in dws], p(dout_d), p(inp_d), p(q), p(k), p(v), p(att),
                                                *[p(w) for w in ws_d], B, T, C, nh, nkv, theta)
            torch.cuda.synchronize()
        res[name] = [out, dinp] + dws
    w64 = [w.double() for w in ws]
    o64 = lo.attention_layer(inp.double(), *w64, B, T, C, nh, nkv, theta)[0]
    g64 = lo.attention_layer_grads(dout.double(), inp.double(), *w64, B, T, C, nh, nkv, theta)
    for i, want in enumerate([o64] + list(g64)):
        e_ours, e_ref = rel(res["ours"][i], want), rel(res["reference"][i], want)
        # the reference rounds scores, probabilities and every intermediate gradient to bf16 and adds with bf16
        # atomics: it sits further from float64 than the fused kernels do
        assert e_ours <= 1e-2, (i, e_ours)
        assert e_ref <= 4e-2, (i, e_ref)
        assert rel(res["ours"][i], res["reference"][i].double().cpu()) <= 5e-2, i


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_swiglu_against_float64_and_the_reference_live(layers, handle, ref_lib, dt):
    from oracle import layers_oracle as lo
    BT, C, ff = 1024, 768, 2048
    inp, dout = rnd((BT, C), 21, dt), rnd((BT, C), 22, dt)
    wg, wu, wd = rnd((C, ff), 23, dt, 0.05), rnd((C, ff), 24, dt, 0.05), rnd((ff, C), 25, dt, 0.05)
    dev = [t.to(DEV) for t in (inp, wg, wu, wd, dout)]
    out = torch.empty(BT, C, device=DEV, dtype=dt)
    gate, up, hidden = (torch.empty(BT, ff, device=DEV, dtype=dt) for _ in range(3))
    layers.swiglu_forward(handle, out, gate, up, hidden, dev[0], dev[1], dev[2], dev[3], BT, C, ff)
    dinp = torch.empty(BT, C, device=DEV, dtype=dt)
    dws = [torch.zeros_like(w) for w in dev[1:4]]
    for _ in range(2):
        layers.swiglu_backward(handle, dinp, *dws, dev[4], dev[0], gate, up, dev[1], dev[2], dev[3], BT, C, ff)
    handle.sync()
    i64, w64 = inp.double(), [w.double() for w in (wg, wu, wd)]
    o64, g64, u64, h64 = lo.swiglu(i64, *w64)
    tol = TOL[dt]
    assert rel(out, o64) <= tol and rel(gate, g64) <= tol and rel(up, u64) <= tol and rel(hidden, h64) <= tol
    grads = lo.swiglu_grads(dout.double(), i64, *w64)
    assert rel(dinp, grads[0]) <= tol
    for got, want in zip(dws, grads[1:]):
        assert rel(got, 2.0 * want) <= tol
    if dt == torch.bfloat16 and hasattr(ref_lib, "ref_swiglu_forward_bf16"):
        vpt, ci = ctypes.c_void_p, ctypes.c_int
        ref_lib.ref_swiglu_forward_bf16.argtypes = [vpt] * 9 + [ci] * 3
        ref_lib.ref_swiglu_forward_bf16.restype = None
        ref_lib.ref_swiglu_backward_bf16.argtypes = [vpt] * 12 + [ci] * 3
        ref_lib.ref_swiglu_backward_bf16.restype = None
        hd = vpt()
        assert ref_lib.ref_create(ctypes.byref(hd)) == 0
        p = lambda t: t.data_ptr()
        r_out, r_gate, r_up, r_hid, r_dinp = (torch.empty_like(t) for t in (out, gate, up, hidden, dinp))
        r_dws = [torch.zeros_like(w) for w in dev[1:4]]
        ref_lib.ref_swiglu_forward_bf16(hd, p(r_out), p(r_gate), p(r_up), p(r_hid), p(dev[0]), p(dev[1]), p(dev[2]), p(dev[3]), BT, C, ff)
        ref_lib.ref_swiglu_backward_bf16(hd, p(r_dinp), *[p(w) for w in r_dws], p(dev[4]), p(dev[0]), p(r_gate), p(r_up), p(dev[1]),
                                         p(dev[2]), p(dev[3]), BT, C, ff)
        torch.cuda.synchronize()
        assert rel(out, r_out.double().cpu()) <= 1e-2 and rel(hidden, r_hid.double().cpu()) <= 1e-2
        assert rel(dinp, r_dinp.double().cpu()) <= 1e-2
        one = [torch.zeros_like(w) for w in dev[1:4]]
        layers.swiglu_backward(handle, torch.empty_like(dinp), *one, dev[4], dev[0], gate, up, dev[1], dev[2], dev[3], BT, C, ff)
        handle.sync()
        for got, want in zip(one, r_dws):
            assert rel(got, want.double().cpu()) <= 1e-2


@pytest.mark.parametrize("rows_bt,V", [((2, 256), 32000), ((1, 256), 4099), ((1, 512), 128256)])
def test_whole_row_cross_entropy_follows_the_reference_rounding(layers, ref_lib, rows_bt, V):
    """Loss and in-place probabilities against the restatement of the reference's rounding sequence
    (oracle/ce_oracle.py::reference_bf16, pinned by the reference's kernels) and against those kernels live;
    dlogits likewise.  V = 4099 exercises rows that are not 16-byte aligned."""
    from oracle import ce_oracle
    B, T = rows_bt
    rows = B * T
    g = torch.Generator().manual_seed(V)
    logits = (3.0 * torch.randn(rows, V, generator=g)).to(torch.bfloat16)
    targets = torch.randint(0, V, (rows,), generator=g, dtype=torch.int32)
    ld, td = logits.to(DEV), targets.to(DEV)
    losses = torch.empty(rows, device=DEV, dtype=torch.float32)
    probs = ld.clone()
    layers.crossentropy_forward(losses, probs, td, B, T, V)
    dl = torch.empty_like(probs)
    layers.crossentropy_softmax_backward(dl, probs, td, B, T, V, 1.0)
    torch.cuda.synchronize()
    o_loss, o_d = ce_oracle.reference_bf16(logits, targets)
    l64, d64 = ce_oracle.exact(logits, targets)
    assert (losses.cpu() - o_loss).abs().max().item() <= 2e-3 * max(1.0, o_loss.abs().max().item())
    assert (losses.double().cpu() - l64).abs().max().item() <= 1.6e-2      # -log of a twice-rounded bf16 probability
    assert rel(dl, d64) <= 1e-2
    mism = (dl.cpu().float() != o_d.float()).float().mean().item()
    assert mism <= 0.02, mism                                               # sum order / exp implementation: rare one-ulp flips
    if hasattr(ref_lib, "ref_crossentropy_forward_bf16") and rows % 256 == 0:
        r_probs, r_loss = ld.clone(), torch.empty_like(losses)
        ref_lib.ref_crossentropy_forward_bf16(r_loss.data_ptr(), r_probs.data_ptr(), td.data_ptr(), B, T, V)
        torch.cuda.synchronize()
        assert (losses - r_loss).abs().max().item() <= 2e-3 * max(1.0, r_loss.abs().max().item())
        assert (probs.float() - r_probs.float()).abs().max().item() <= 2.0 ** -8 * r_probs.float().abs().max().item()


def test_whole_row_cross_entropy_fp32(layers):
    from oracle import ce_oracle
    B, T, V = 1, 128, 5003
    g = torch.Generator().manual_seed(9)
    logits = 3.0 * torch.randn(B * T, V, generator=g)
    targets = torch.randint(0, V, (B * T,), generator=g, dtype=torch.int32)
    probs, td = logits.to(DEV), targets.to(DEV)
    losses = torch.empty(B * T, device=DEV, dtype=torch.float32)
    layers.crossentropy_forward(losses, probs, td, B, T, V)
    dl = torch.empty_like(probs)
    layers.crossentropy_softmax_backward(dl, probs, td, B, T, V)
    torch.cuda.synchronize()
    l64, d64 = ce_oracle.exact(logits, targets)
    assert (losses.double().cpu() - l64).abs().max().item() <= 2e-5 * l64.abs().max().item()
    assert rel(dl, d64) <= 2e-5


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,C", [(8192, 768), (300, 100), (1000, 1024), (77, 256), (4096, 512), (130, 2048)])
def test_rmsnorm_against_float64(layers, dt, rows, C):
    """cuda/rmsnorm.cu restated in float64 (forward formula at :27-33, backward at :60-72), the weight gradient
    accumulating over two calls onto a non-zero start."""
    x, dy = rnd((rows, C), 31, dt), rnd((rows, C), 32, dt)
    w = (1.0 + 0.1 * rnd((C,), 33, torch.float32)).to(dt)
    dw0 = rnd((C,), 34, dt)
    eps = 1e-5
    xd, dyd, wd = x.to(DEV), dy.to(DEV), w.to(DEV)
    out, rrms = torch.empty_like(xd), torch.empty(rows, device=DEV, dtype=torch.float32)
    layers.rmsnorm_forward(out, rrms, xd, wd, eps, rows, C)
    dinp, dw = torch.empty_like(xd), dw0.to(DEV)
    layers.rmsnorm_backward(dinp, dw, dyd, xd, wd, rrms, rows, C)
    dw1 = dw.clone()
    layers.rmsnorm_backward(dinp, dw, dyd, xd, wd, rrms, rows, C)
    torch.cuda.synchronize()
    x64, dy64, w64 = x.double(), dy.double(), w.double()
    inv = torch.rsqrt((x64 * x64).mean(dim=1) + eps)
    tol = TOL[dt]
    assert rel(out, x64 * inv[:, None] * w64) <= tol
    assert (rrms.double().cpu() - inv).abs().max().item() <= 1e-5 * inv.abs().max().item()
    s = (dy64 * w64 * x64).sum(dim=1)
    assert rel(dinp, inv[:, None] * (dy64 * w64 - x64 * (inv * inv * s / C)[:, None])) <= tol
    dw64 = (dy64 * x64 * inv[:, None]).sum(dim=0)
    assert rel(dw1, dw0.double() + dw64) <= tol
    assert rel(dw, dw1.double().cpu() + dw64) <= tol


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,offset", [(8192 * 768, 0), (1000003, 0), (4099, 1)])
def test_residual_add_is_exact(layers, dt, n, offset):
    """out = a + b and da += dout, db += dout (cuda/residual.cu): one rounding per element, so the result equals the
    same arithmetic in torch bit for bit; lengths that are not a multiple of the vector width and unaligned starts
    included; the in-place form the model uses (out = a)."""
    a = rnd((n + offset,), 41, dt).to(DEV)[offset:]
    b = rnd((n + offset,), 42, dt).to(DEV)[offset:]
    want = (a.float() + b.float()).to(dt)
    out = torch.empty(n + offset, device=DEV, dtype=dt)[offset:]
    layers.residual_forward(out, a, b, n)
    x = a.clone() if offset == 0 else None
    if x is not None:
        layers.residual_forward(x, x, b, n)
    da, db = rnd((n + offset,), 43, dt).to(DEV)[offset:], rnd((n + offset,), 44, dt).to(DEV)[offset:]
    want_da, want_db = (da.float() + a.float()).to(dt), (db.float() + a.float()).to(dt)
    layers.residual_backward(da, db, a, n)
    torch.cuda.synchronize()
    assert torch.equal(out, want) and (x is None or torch.equal(x, want))
    assert torch.equal(da, want_da) and torch.equal(db, want_db)


def _adamw64(p, g, m, v, lr, b1, b2, eps, wd, t):
    """cuda/adamw.cu:12-40 in float64."""
    m2 = b1 * m + (1 - b1) * g
    v2 = b2 * v + (1 - b2) * g * g
    p2 = p - lr * ((m2 / (1 - b1 ** t)) / ((v2 / (1 - b2 ** t)).sqrt() + eps) + wd * p)
    return p2, m2, v2


@pytest.mark.parametrize("n", [768 * 768, 100003])
def test_adamw_against_float64_and_the_reference_live(layers, ref_lib, n):
    """Three steps of both overloads against float64 (fp32 state: 1e-5 relative; the bf16 weights are the rounding of the
    master weights, exactly), and against the reference's own adamw.cu on the same state."""
    lr, b1, b2, eps, wd, gs = 3e-4, 0.9, 0.95, 1e-8, 0.1, 1.0 / 1024
    p0, g_all = rnd((n,), 1, torch.float32, 0.02), [rnd((n,), 10 + t, torch.float32) for t in range(3)]
    # fp32 overload
    p, m, v = p0.to(DEV), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    p64, m64, v64 = p0.double(), torch.zeros(n).double(), torch.zeros(n).double()
    for t in range(1, 4):
        layers.adamw_update(p, g_all[t - 1].to(DEV), m, v, lr, b1, b2, eps, wd, t, n)
        p64, m64, v64 = _adamw64(p64, g_all[t - 1].double(), m64, v64, lr, b1, b2, eps, wd, t)
    torch.cuda.synchronize()
    assert rel(p, p64) <= 1e-5 and rel(m, m64) <= 1e-5 and rel(v, v64) <= 1e-5
    # mixed precision: bf16 weights and scaled bf16 gradients, fp32 master weights and moments
    master, m, v = p0.to(DEV), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    pb = master.to(torch.bfloat16)
    r_master, r_m, r_v, r_pb = master.clone(), m.clone(), v.clone(), pb.clone()
    p64, m64, v64 = p0.double(), torch.zeros(n).double(), torch.zeros(n).double()
    have_ref = hasattr(ref_lib, "ref_adamw_update_bf16")
    if have_ref:
        vpt, cf, ci = ctypes.c_void_p, ctypes.c_float, ctypes.c_int
        ref_lib.ref_adamw_update_bf16.argtypes = [vpt] * 5 + [cf] * 6 + [ci, ci]
        ref_lib.ref_adamw_update_bf16.restype = None
    for t in range(1, 4):
        gb = (g_all[t - 1] * 1024).to(torch.bfloat16)
        gd = gb.to(DEV)
        layers.adamw_update(pb, gd, m, v, lr, b1, b2, eps, wd, t, n, master_params=master, grad_scale=gs)
        p64, m64, v64 = _adamw64(p64, gb.double() * gs, m64, v64, lr, b1, b2, eps, wd, t)
        if have_ref:
            ref_lib.ref_adamw_update_bf16(r_pb.data_ptr(), r_master.data_ptr(), gd.data_ptr(), r_m.data_ptr(), r_v.data_ptr(),
                                          lr, b1, b2, eps, wd, gs, t, n)
    torch.cuda.synchronize()
    assert rel(master, p64) <= 1e-5 and rel(m, m64) <= 1e-5 and rel(v, v64) <= 1e-5
    assert torch.equal(pb, master.to(torch.bfloat16))
    if have_ref:   # the reference is built with fast-math (approximate pow, divide, sqrt): close, not bit-equal
        assert rel(r_master, p64) <= 1e-4
        assert rel(master, r_master.double().cpu()) <= 1e-4


def test_gradient_norm_sanitizes_and_matches_float64(layers, ref_lib):
    """compute_grad_norm_bf16: float64 norm of the unscaled gradient over both parts; inf / nan / > 65000 entries of
    the bf16 part are zeroed in place and left out of the sum; twice the same answer (fixed summation order)."""
    emb_n, rest_n, scale = 32000 * 768 // 8, 5_000_003, 1024.0
    dwte = rnd((emb_n,), 1, torch.float32, 3.0)
    g = rnd((rest_n,), 2, torch.float32, 50.0).to(torch.bfloat16)
    g[17], g[4099], g[rest_n - 1] = float("inf"), float("nan"), 7.0e7 * 1.0   # 7e7 / 1024 > 65000
    g[5] = -float("inf")
    keep = torch.ones(rest_n, dtype=torch.bool)
    keep[[5, 17, 4099, rest_n - 1]] = False
    want = ((dwte.double() / scale).pow(2).sum() + (g.double()[keep] / scale).pow(2).sum()).sqrt().item()
    dw_d, g_d = dwte.to(DEV), g.to(DEV)
    got = layers.compute_grad_norm_bf16(dw_d, emb_n, g_d, rest_n, scale)
    assert abs(got - want) <= 1e-5 * want, (got, want)
    cleaned = g.clone()
    cleaned[~keep] = 0
    assert torch.equal(g_d.cpu(), cleaned)
    assert layers.compute_grad_norm_bf16(dw_d, emb_n, g_d, rest_n, scale) == got
    if hasattr(ref_lib, "ref_grad_norm_bf16"):
        vpt, ci = ctypes.c_void_p, ctypes.c_int
        ref_lib.ref_grad_norm_bf16.argtypes = [vpt, ci, vpt, ci, ctypes.c_float]
        ref_lib.ref_grad_norm_bf16.restype = ctypes.c_float
        g_r = g.to(DEV)
        ref = ref_lib.ref_grad_norm_bf16(dw_d.data_ptr(), emb_n, g_r.data_ptr(), rest_n, scale)
        assert abs(ref - want) <= 1e-4 * want and torch.equal(g_r, g_d)


def test_layer_entry_points_refuse_bad_arguments(layers, handle):
    t = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    lse = torch.zeros(64, device=DEV, dtype=torch.float32)
    with pytest.raises(Exception):
        layers.flash_attention_forward(t, lse, t, t, t, 1, 64, 1, 1, 32)     # head dimension other than 64
    with pytest.raises(Exception):
        layers.flash_attention_forward(t, lse, t, t, t, 1, 64, 3, 2, 64)     # heads not a multiple of KV heads
    with pytest.raises(Exception):
        layers.swiglu_forward(handle, t, t, t, t, t, t, t, t, 0, 64, 64)
    handle.sync()
