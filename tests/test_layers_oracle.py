"""CPU checks of oracle/layers_oracle.py (the float64 restatement of the reference's attention, RoPE and SwiGLU):
the vectorised restatement against explicit loops that index the way the reference's kernels do, the rotation
against its inverse, and the automatic-differentiation gradients against finite differences."""
import numpy as np
import torch

from oracle import layers_oracle as lo


def test_attention_core_matches_explicit_loops():
    g = torch.Generator().manual_seed(1)
    B, T, nh, nkv, hd = 2, 9, 6, 2, 8
    q = torch.randn(B * T, nh * hd, generator=g, dtype=torch.float64)
    k = torch.randn(B * T, nkv * hd, generator=g, dtype=torch.float64)
    v = torch.randn(B * T, nkv * hd, generator=g, dtype=torch.float64)
    ctx, lse = lo.attention_core(q, k, v, B, T, nh, nkv, hd)
    ctx2, lse2 = lo.attention_core_naive(q, k, v, B, T, nh, nkv, hd)
    assert torch.allclose(ctx, ctx2, atol=1e-12) and torch.allclose(lse, lse2, atol=1e-12)
    # causality: the first token attends to itself only, so its context is its own value row (per KV group)
    for h in range(nh):
        assert torch.allclose(ctx[0, h * hd:(h + 1) * hd], v[0, (h // 3) * hd:(h // 3 + 1) * hd])


def test_rope_is_a_rotation_and_backward_is_its_inverse():
    g = torch.Generator().manual_seed(2)
    B, T, nh, hd = 2, 33, 3, 16
    x = torch.randn(B * T, nh * hd, generator=g, dtype=torch.float64)
    y = lo.rope(x, B, T, nh, hd, 10000.0)
    assert torch.allclose(y[0], x[0])                                      # position 0 is not rotated
    assert torch.allclose(y.reshape(-1, 2).norm(dim=1), x.reshape(-1, 2).norm(dim=1))
    assert torch.allclose(lo.rope(y, B, T, nh, hd, 10000.0, backward=True), x, atol=1e-12)
    ang = lo.rope_angles(8, 4, 100.0)                                       # pairs rotate at 1 and 100^(-1/2) = 0.1
    assert np.allclose(ang[:, 0].numpy(), np.arange(8)) and np.allclose(ang[:, 1].numpy(), np.arange(8) * np.float32(0.1), rtol=1e-7)


def test_gradients_against_finite_differences():
    g = torch.Generator().manual_seed(3)
    B, T, C, nh, nkv, ff = 1, 5, 8, 2, 1, 12
    inp = torch.randn(B * T, C, generator=g, dtype=torch.float64)
    ws = [0.3 * torch.randn(*s, generator=g, dtype=torch.float64) for s in ((C, C), (C, C // 2), (C, C // 2), (C, C))]
    dout = torch.randn(B * T, C, generator=g, dtype=torch.float64)
    grads = lo.attention_layer_grads(dout, inp, *ws, B, T, C, nh, nkv, 10000.0)
    f = lambda i, w: (lo.attention_layer(i, *w, B, T, C, nh, nkv, 10000.0)[0] * dout).sum()
    eps = 1e-6
    for (r, c) in ((0, 0), (3, 5)):
        d = torch.zeros_like(inp); d[r, c] = eps
        assert abs((f(inp + d, ws) - f(inp - d, ws)).item() / (2 * eps) - grads[0][r, c].item()) < 1e-6
    d = torch.zeros_like(ws[1]); d[2, 1] = eps
    fd = (f(inp, [ws[0], ws[1] + d, ws[2], ws[3]]) - f(inp, [ws[0], ws[1] - d, ws[2], ws[3]])).item() / (2 * eps)
    assert abs(fd - grads[2][2, 1].item()) < 1e-6
    wg, wu, wd = (0.3 * torch.randn(*s, generator=g, dtype=torch.float64) for s in ((C, ff), (C, ff), (ff, C)))
    sg = lo.swiglu_grads(dout, inp, wg, wu, wd)
    fs = lambda i: (lo.swiglu(i, wg, wu, wd)[0] * dout).sum()
    d = torch.zeros_like(inp); d[1, 2] = eps
    assert abs((fs(inp + d) - fs(inp - d)).item() / (2 * eps) - sg[0][1, 2].item()) < 1e-6
