"""CPU restatement (torch, float64) of the reference's layers around the linear-layer GEMMs.

TEST INFRASTRUCTURE ONLY: imported by tests/ (and nothing in the product path).

Follows chriskuchar/llms-from-scratch-cuda:
  * rotary embedding       cuda/rope.cu:15-57 (forward), :63-101 (backward = the inverse rotation)
  * attention              cuda/attention.cu:8-70 (scores with causal mask, value product), cuda/softmax.cu,
                           host sequence cuda/attention.cu:235-292 (projections, RoPE, scores, softmax, value, output)
  * SwiGLU                 cuda/swiglu.cu:12-24 (SiLU(gate) * up), host sequence :49-70
  * backward passes        by automatic differentiation of the float64 forward, which is what the reference's
                           hand-written backward kernels (attention.cu:72-231, swiglu.cu:27-47) implement
No intermediate rounding: this is the exact mathematics the reference's fp32 and bf16 kernels approximate.  The
reference ships no test or golden vector for these functions (parity unpinned by the reference itself); the pin
is tests/test_layers_gpu.py, which runs the reference's own unmodified attention.cu / swiglu.cu / rope.cu
(compiled from its checkout into oracle/_ref) next to this restatement on the same inputs.
One deliberate detail: the rotation angle is the fp32 product of the position and the fp32-rounded frequency
theta^(-2i/hd) (the reference forms both in fp32, rope.cu:29-30); only cos and sin are taken in float64.
"""
import numpy as np
import torch


def rope_angles(T, head_dim, theta):
    """[T, head_dim/2] float64 angles: fp32(t) * fp32(theta^(-2i/head_dim)), the product rounded to fp32."""
    i = np.arange(head_dim // 2, dtype=np.float64)
    freq = (1.0 / np.power(np.float64(theta), 2.0 * i / head_dim)).astype(np.float32)
    t = np.arange(T, dtype=np.float32)
    return torch.from_numpy((t[:, None] * freq[None, :]).astype(np.float32).astype(np.float64))


def rope(x, B, T, n_heads, head_dim, theta, backward=False):
    """x [B*T, n_heads*head_dim] float64 -> rotated copy (cuda/rope.cu:41-56; backward: :86-100)."""
    ang = rope_angles(T, head_dim, theta)
    cos, sin = torch.cos(ang), torch.sin(ang)
    if backward:
        sin = -sin
    xr = x.reshape(B, T, n_heads, head_dim // 2, 2)
    x0, x1 = xr[..., 0], xr[..., 1]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    out = torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)
    return out.reshape(B * T, n_heads * head_dim)


def attention_core(q, k, v, B, T, n_head, n_kv_head, head_dim):
    """context [B*T, n_head*hd] and lse [B, n_head, T] of causal grouped-query attention (attention.cu:8-70)."""
    ratio = n_head // n_kv_head
    qh = q.reshape(B, T, n_head, head_dim).permute(0, 2, 1, 3)
    kh = k.reshape(B, T, n_kv_head, head_dim).permute(0, 2, 1, 3).repeat_interleave(ratio, dim=1)
    vh = v.reshape(B, T, n_kv_head, head_dim).permute(0, 2, 1, 3).repeat_interleave(ratio, dim=1)
    s = qh @ kh.transpose(-1, -2) / np.sqrt(head_dim)
    mask = torch.ones(T, T, dtype=torch.bool).triu(1)
    s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    ctx = torch.softmax(s, dim=-1) @ vh
    return ctx.permute(0, 2, 1, 3).reshape(B * T, n_head * head_dim), lse


def attention_core_grads(dcontext, q, k, v, B, T, n_head, n_kv_head, head_dim):
    q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
    ctx, _ = attention_core(q, k, v, B, T, n_head, n_kv_head, head_dim)
    ctx.backward(dcontext)
    return q.grad, k.grad, v.grad


def attention_layer(inp, wq, wk, wv, wo, B, T, C, n_head, n_kv_head, theta):
    """attention_forward (attention.cu:235-292): returns out, q, k (both rotated), v, context, lse."""
    hd = C // n_head
    q = rope(inp @ wq, B, T, n_head, hd, theta)
    k = rope(inp @ wk, B, T, n_kv_head, hd, theta)
    v = inp @ wv
    ctx, lse = attention_core(q, k, v, B, T, n_head, n_kv_head, hd)
    return ctx @ wo, q, k, v, ctx, lse


def attention_layer_grads(dout, inp, wq, wk, wv, wo, B, T, C, n_head, n_kv_head, theta):
    """attention_backward (attention.cu:294-414): dinp, dwq, dwk, dwv, dwo (the dW of one call, not accumulated)."""
    leaves = [t.clone().requires_grad_(True) for t in (inp, wq, wk, wv, wo)]
    out = attention_layer(*leaves, B, T, C, n_head, n_kv_head, theta)[0]
    out.backward(dout)
    return [t.grad for t in leaves]


def swiglu(inp, w_gate, w_up, w_down):
    """swiglu_forward (swiglu.cu:49-70): out, gate, up, hidden."""
    gate, up = inp @ w_gate, inp @ w_up
    hidden = gate * torch.sigmoid(gate) * up
    return hidden @ w_down, gate, up, hidden


def swiglu_grads(dout, inp, w_gate, w_up, w_down):
    """swiglu_backward (swiglu.cu:72-130): dinp, dw_gate, dw_up, dw_down."""
    leaves = [t.clone().requires_grad_(True) for t in (inp, w_gate, w_up, w_down)]
    swiglu(*leaves)[0].backward(dout)
    return [t.grad for t in leaves]


def attention_core_naive(q, k, v, B, T, n_head, n_kv_head, head_dim):
    """The same mathematics as explicit loops over (b, h, t1, t2), the way the reference's kernels index it
    (attention.cu:18-37, 51-69): small sizes only; pins attention_core."""
    q, k, v = (t.numpy() for t in (q, k, v))
    ratio = n_head // n_kv_head
    ctx = np.zeros((B * T, n_head * head_dim))
    lse = np.zeros((B, n_head, T))
    scale = 1.0 / np.sqrt(head_dim)
    for b in range(B):
        for h in range(n_head):
            kvh = h // ratio
            for t1 in range(T):
                qv = q[b * T + t1, h * head_dim:(h + 1) * head_dim]
                sc = np.array([qv @ k[b * T + t2, kvh * head_dim:(kvh + 1) * head_dim] * scale for t2 in range(t1 + 1)])
                m = sc.max()
                e = np.exp(sc - m)
                lse[b, h, t1] = m + np.log(e.sum())
                p = e / e.sum()
                for t2 in range(t1 + 1):
                    ctx[b * T + t1, h * head_dim:(h + 1) * head_dim] += p[t2] * v[b * T + t2, kvh * head_dim:(kvh + 1) * head_dim]
    return torch.from_numpy(ctx), torch.from_numpy(lse)
