"""Host-side mirror of the reference's layer-level interface (cuda/kernels.cuh of
chriskuchar/llms-from-scratch-cuda) over the C ABI declared in include/b200_layers.h:

    flash_attention_forward / flash_attention_backward     kernels.cuh:316-341, 420-437
    rope_forward / rope_backward                           kernels.cuh:119-139, 365-368
    attention_forward / attention_backward                 kernels.cuh:156-206, 371-388
    swiglu_forward / swiglu_backward                       kernels.cuh:211-247, 390-396
    crossentropy_forward / crossentropy_softmax_backward   kernels.cuh:260-277, 402-404
    rmsnorm_forward / rmsnorm_backward                     kernels.cuh:85-108, 357-362
    residual_forward / residual_backward                   kernels.cuh:280-289, 407-408
    adamw_update / compute_grad_norm_bf16                  kernels.cuh:299-309, 411-418

Same names, argument order and meaning as the reference (the cublasHandle_t argument becomes a `Handle`, first
instead of last); the dtype overload is picked from the tensors.  Arguments are torch CUDA tensors used as
device memory only.  Errors raise `LinearError`; there is no CPU or library fallback.
"""
import ctypes

import torch

from .linear import LinearError, lib, strerror

vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _declare():
    for sfx in ("bf16", "f32"):
        getattr(lib, "b200_flash_attention_forward_" + sfx).argtypes = [vp] * 5 + [ci] * 5 + [vp]
        getattr(lib, "b200_flash_attention_backward_" + sfx).argtypes = [vp] * 9 + [ci] * 5 + [vp]
        getattr(lib, "b200_attention_forward_" + sfx).argtypes = [vp] * 11 + [ci] * 5 + [cf]
        getattr(lib, "b200_attention_backward_" + sfx).argtypes = [vp] * 16 + [ci] * 5 + [cf]
        getattr(lib, "b200_swiglu_forward_" + sfx).argtypes = [vp] * 9 + [ci] * 3
        getattr(lib, "b200_swiglu_backward_" + sfx).argtypes = [vp] * 12 + [ci] * 3
        getattr(lib, "b200_crossentropy_forward_" + sfx).argtypes = [vp, vp, vp, ci, ci, ci]
    lib.b200_crossentropy_backward_bf16.argtypes = [vp, vp, vp, ci, ci, ci, cf]
    lib.b200_crossentropy_backward_f32.argtypes = [vp, vp, vp, ci, ci, ci]
    lib.b200_rope_bf16.argtypes = [vp, vp, ci, ci, ci, ci, ci, cf, ci, vp]


_declare()


def _p(t):
    if t is None:
        return None
    if not t.is_cuda or not t.is_contiguous():
        raise LinearError(1, "argument", " (need contiguous CUDA tensors)")
    return t.data_ptr()


def _sfx(t):
    if t.dtype == torch.bfloat16:
        return "bf16"
    if t.dtype == torch.float32:
        return "f32"
    raise LinearError(1, "argument", f" (unsupported dtype {t.dtype})")


def _check(rc, what):
    if rc:
        raise LinearError(rc, what, f" ({strerror(rc)})")


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def flash_attention_forward(context, lse, q, k, v, B, T, n_head, n_kv_head, head_dim):
    fn = getattr(lib, "b200_flash_attention_forward_" + _sfx(q))
    _check(fn(_p(context), _p(lse), _p(q), _p(k), _p(v), B, T, n_head, n_kv_head, head_dim, _stream()), "flash_attention_forward")


def flash_attention_backward(dq, dk, dv, dcontext, q, k, v, lse, B, T, n_head, n_kv_head, head_dim, context=None):
    """`context` (the forward output) is optional: the reference's argument list has none, and without it the
    forward pass is run again."""
    fn = getattr(lib, "b200_flash_attention_backward_" + _sfx(q))
    _check(fn(_p(dq), _p(dk), _p(dv), _p(dcontext), _p(q), _p(k), _p(v), _p(lse), _p(context), B, T, n_head, n_kv_head,
              head_dim, _stream()), "flash_attention_backward")


def rope_forward(q, k, B, T, n_head, n_kv_head, head_dim, theta):
    _check(lib.b200_rope_bf16(_p(q), _p(k), B, T, n_head, n_kv_head, head_dim, theta, 0, _stream()), "rope_forward")


def rope_backward(dq, dk, B, T, n_head, n_kv_head, head_dim, theta):
    _check(lib.b200_rope_bf16(_p(dq), _p(dk), B, T, n_head, n_kv_head, head_dim, theta, 1, _stream()), "rope_backward")


def attention_forward(handle, out, q, k, v, att, inp, wq, wk, wv, wo, B, T, C, n_head, n_kv_head, rope_theta):
    fn = getattr(lib, "b200_attention_forward_" + _sfx(inp))
    _check(fn(handle._h, _p(out), _p(q), _p(k), _p(v), _p(att), _p(inp), _p(wq), _p(wk), _p(wv), _p(wo), B, T, C, n_head,
              n_kv_head, rope_theta), "attention_forward")


def attention_backward(handle, dinp, dwq, dwk, dwv, dwo, dout, inp, q, k, v, att, wq, wk, wv, wo, B, T, C, n_head, n_kv_head,
                       rope_theta):
    fn = getattr(lib, "b200_attention_backward_" + _sfx(inp))
    _check(fn(handle._h, _p(dinp), _p(dwq), _p(dwk), _p(dwv), _p(dwo), _p(dout), _p(inp), _p(q), _p(k), _p(v), _p(att), _p(wq),
              _p(wk), _p(wv), _p(wo), B, T, C, n_head, n_kv_head, rope_theta), "attention_backward")


def swiglu_forward(handle, out, gate, up, hidden, inp, w_gate, w_up, w_down, B_T, C, ffn_hidden):
    fn = getattr(lib, "b200_swiglu_forward_" + _sfx(inp))
    _check(fn(handle._h, _p(out), _p(gate), _p(up), _p(hidden), _p(inp), _p(w_gate), _p(w_up), _p(w_down), B_T, C, ffn_hidden),
           "swiglu_forward")


def swiglu_backward(handle, dinp, dw_gate, dw_up, dw_down, dout, inp, gate, up, w_gate, w_up, w_down, B_T, C, ffn_hidden):
    fn = getattr(lib, "b200_swiglu_backward_" + _sfx(inp))
    _check(fn(handle._h, _p(dinp), _p(dw_gate), _p(dw_up), _p(dw_down), _p(dout), _p(inp), _p(gate), _p(up), _p(w_gate),
              _p(w_up), _p(w_down), B_T, C, ffn_hidden), "swiglu_backward")


def rmsnorm_forward(out, rrms, inp, weight, eps, B_T, C):
    fn = getattr(lib, "b200_rmsnorm_forward_" + _sfx(inp))
    fn.argtypes = [vp, vp, vp, vp, cf, ci, ci]
    _check(fn(_p(out), _p(rrms), _p(inp), _p(weight), eps, B_T, C), "rmsnorm_forward")


def rmsnorm_backward(dinp, dweight, dout, inp, weight, rrms, B_T, C):
    """dinp overwritten, dweight accumulated."""
    fn = getattr(lib, "b200_rmsnorm_backward_" + _sfx(inp))
    fn.argtypes = [vp] * 6 + [ci, ci]
    _check(fn(_p(dinp), _p(dweight), _p(dout), _p(inp), _p(weight), _p(rrms), B_T, C), "rmsnorm_backward")


def residual_forward(out, a, b, N):
    """out = a + b (out may be a)."""
    fn = getattr(lib, "b200_residual_forward_" + _sfx(a))
    fn.argtypes = [vp, vp, vp, ctypes.c_longlong]
    _check(fn(_p(out), _p(a), _p(b), N), "residual_forward")


def residual_backward(da, db, dout, N):
    """da += dout, db += dout."""
    fn = getattr(lib, "b200_residual_backward_" + _sfx(dout))
    fn.argtypes = [vp, vp, vp, ctypes.c_longlong]
    _check(fn(_p(da), _p(db), _p(dout), N), "residual_backward")


def crossentropy_forward(losses, logits, targets, B, T, V):
    """Per-row loss; the probabilities replace the logits in place, as in the reference."""
    fn = getattr(lib, "b200_crossentropy_forward_" + _sfx(logits))
    _check(fn(_p(losses), _p(logits), _p(targets), B, T, V), "crossentropy_forward")


def crossentropy_softmax_backward(dlogits, probs, targets, B, T, V, loss_scale=1.0):
    if probs.dtype == torch.bfloat16:
        rc = lib.b200_crossentropy_backward_bf16(_p(dlogits), _p(probs), _p(targets), B, T, V, loss_scale)
    else:
        rc = lib.b200_crossentropy_backward_f32(_p(dlogits), _p(probs), _p(targets), B, T, V)
    _check(rc, "crossentropy_softmax_backward")


def adamw_update(params, grads, m, v, lr, beta1, beta2, eps, weight_decay, t, N, master_params=None, grad_scale=1.0):
    """One AdamW step in place.  With `master_params` (fp32) the mixed-precision overload: bf16 `params` and `grads`,
    the gradient multiplied by `grad_scale` first (adamw.cu:63-88); otherwise all fp32 (adamw.cu:12-40)."""
    cll = ctypes.c_longlong
    if master_params is not None:
        lib.b200_adamw_update_bf16.argtypes = [vp] * 5 + [cf] * 6 + [ci, cll]
        rc = lib.b200_adamw_update_bf16(_p(params), _p(master_params), _p(grads), _p(m), _p(v), lr, beta1, beta2, eps,
                                        weight_decay, grad_scale, t, N)
    else:
        lib.b200_adamw_update_f32.argtypes = [vp] * 4 + [cf] * 5 + [ci, cll]
        rc = lib.b200_adamw_update_f32(_p(params), _p(grads), _p(m), _p(v), lr, beta1, beta2, eps, weight_decay, t, N)
    _check(rc, "adamw_update")


def compute_grad_norm_bf16(dwte_fp32, emb_N, grads_bf16, rest_N, loss_scale):
    """Global L2 norm of the unscaled gradient; zeroes non-finite bf16 entries in place (adamw.cu:171-191)."""
    cll = ctypes.c_longlong
    lib.b200_grad_norm_bf16.argtypes = [ctypes.POINTER(cf), vp, cll, vp, cll, cf]
    out = cf(0.0)
    _check(lib.b200_grad_norm_bf16(ctypes.byref(out), _p(dwte_fp32), emb_N, _p(grads_bf16), rest_N, loss_scale),
           "compute_grad_norm_bf16")
    return out.value
