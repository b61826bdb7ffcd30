"""Host-side mirror of the reference's GEMM-leaf interface over the C ABI of libb200_linear.so.

The reference's interface is C++ (cuda/kernels.cuh:47-65, 348-351 of
chriskuchar/llms-from-scratch-cuda):

    matmul_forward (handle, C, A, B, M, N, K)             C[M,N]  = A[M,K] @ B[K,N]
    matmul_backward(handle, dA, dB, dC, A, B, M, N, K)    dA[M,K] = dC @ B^T ; dB[K,N] += A^T @ dC

The functions below keep those names, argument order and meaning; the dtype overload
(float* vs __nv_bfloat16*) is picked from the tensors' dtype.  Arguments are torch CUDA
tensors (used only as device memory: `data_ptr()`) or raw integer device addresses.
Unlike the reference (which prints and exits, cuda/tensor.h:10-29) errors raise
`LinearError`.  There is no CPU or library fallback: if the CUDA library is missing the
import of this module fails.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200_linear.so")

FWD_NN, DGRAD_NT, WGRAD_TN = 0, 1, 2


class LinearError(RuntimeError):
    def __init__(self, code, what, detail=""):
        self.code = code
        super().__init__(f"{what}: b200_linear error {code}{detail}")


class Plan(ctypes.Structure):
    _fields_ = [("bn", ctypes.c_int), ("cta_pair", ctypes.c_int), ("splits", ctypes.c_int),
                ("m_fastest", ctypes.c_int), ("tiles", ctypes.c_int), ("waves_x100", ctypes.c_int),
                ("dp_tiles", ctypes.c_int), ("sk_items", ctypes.c_int), ("cluster_split", ctypes.c_int),
                ("est_ns", ctypes.c_int)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python llms-from-scratch-cuda_b200/build.py` "
            "(there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.b200_linear_create.argtypes = [ctypes.POINTER(vp)]
    lib.b200_linear_destroy.argtypes = [vp]
    lib.b200_linear_set_stream.argtypes = [vp, vp]
    lib.b200_linear_sync.argtypes = [vp, ctypes.POINTER(ci)]
    lib.b200_linear_launch_count.argtypes = [vp]
    lib.b200_linear_launch_count.restype = ctypes.c_longlong
    lib.b200_linear_last_cuda_error.argtypes = [vp]
    lib.b200_linear_strerror.argtypes = [ci]
    lib.b200_linear_strerror.restype = ctypes.c_char_p
    for name in ("b200_linear_forward_bf16", "b200_linear_forward_f32"):
        getattr(lib, name).argtypes = [vp, vp, vp, vp, ci, ci, ci]
    for name in ("b200_linear_backward_bf16", "b200_linear_backward_f32"):
        getattr(lib, name).argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci]
    for name in ("b200_linear_gemm_bf16", "b200_linear_gemm_f32"):
        getattr(lib, name).argtypes = [vp, ci, ci, vp, vp, vp, ci, ci, ci]
    lib.b200_linear_gemm_bf16_ld.argtypes = [vp, ci, ci, vp, ctypes.c_longlong, vp, ctypes.c_longlong, vp,
                                             ctypes.c_longlong, ci, ci, ci]
    lib.b200_linear_selftest_wait_timeout.argtypes = [vp, ctypes.c_longlong]
    lib.b200_linear_plan_bf16.argtypes = [ci, ci, ci, ci, ci, ci, ctypes.POINTER(Plan)]
    lib.b200_linear_force_plan.argtypes = [vp, ci, ci, ci]
    lib.b200_linear_force_backward_split.argtypes = [vp, ci]
    ll, cf = ctypes.c_longlong, ctypes.c_float
    lib.b200_ce_shard_stats_bf16.argtypes = [vp, ci, ci, ll, vp, ci, vp, vp, vp, vp]
    lib.b200_ce_shard_rescale.argtypes = [vp, vp, vp, ci, vp]
    lib.b200_ce_shard_loss.argtypes = [vp, vp, vp, vp, ci, vp]
    lib.b200_ce_shard_backward_bf16.argtypes = [vp, vp, ci, ci, ll, vp, ci, vp, vp, cf, vp]
    return lib


lib = _load()


def strerror(code):
    return lib.b200_linear_strerror(int(code)).decode()


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if not t.is_cuda:
        raise LinearError(1, "argument", " (tensor is not on a CUDA device)")
    if not t.is_contiguous():
        raise LinearError(1, "argument", " (tensor is not contiguous)")
    return t.data_ptr()


def _suffix(*tensors):
    for t in tensors:
        if t is None or isinstance(t, int):
            continue
        if t.dtype == torch.bfloat16:
            return "bf16"
        if t.dtype == torch.float32:
            return "f32"
        raise LinearError(1, "argument", f" (unsupported dtype {t.dtype})")
    raise LinearError(1, "argument", " (dtype cannot be inferred from raw pointers; pass dtype=)")


class Handle:
    """What the reference keeps in its cublasHandle_t: one per process and GPU."""

    def __init__(self, stream=None):
        h = ctypes.c_void_p()
        rc = lib.b200_linear_create(ctypes.byref(h))
        if rc:
            raise LinearError(rc, "b200_linear_create", f" ({strerror(rc)})")
        self._h = h
        if stream is not None:
            self.set_stream(stream)

    def set_stream(self, stream):
        s = stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)
        self._check(lib.b200_linear_set_stream(self._h, ctypes.c_void_p(s)), "set_stream")

    def _check(self, rc, what):
        if rc:
            raise LinearError(rc, what, f" ({strerror(rc)}; cuda {lib.b200_linear_last_cuda_error(self._h)})")

    def sync(self):
        """Wait for the stream and raise if any kernel recorded a timed-out wait."""
        code = ctypes.c_int(0)
        rc = lib.b200_linear_sync(self._h, ctypes.byref(code))
        if rc:
            raise LinearError(rc, "b200_linear_sync", f" ({strerror(rc)}; device code {code.value})")

    def selftest_wait_timeout(self, limit_cycles=2_000_000):
        """Launch the one-warp probe whose bounded wait runs out after `limit_cycles` SM clocks; the
        next sync() then raises LinearError with code B200_E_DEVICE_WAIT and the handle stays usable."""
        self._check(lib.b200_linear_selftest_wait_timeout(self._h, int(limit_cycles)), "selftest_wait_timeout")

    @property
    def launches(self):
        return int(lib.b200_linear_launch_count(self._h))

    def force_plan(self, bn=-1, cta_pair=0, splits=0):
        self._check(lib.b200_linear_force_plan(self._h, bn, cta_pair, splits), "force_plan")

    def force_backward_split(self, sm_dgrad=0):
        """SMs given to dgrad when matmul_backward runs its two products side by side (0 = cost model)."""
        self._check(lib.b200_linear_force_backward_split(self._h, sm_dgrad), "force_backward_split")

    def destroy(self):
        if self._h:
            lib.b200_linear_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def matmul_forward(handle, C, A, B, M, N, K, dtype=None):
    """C[M,N] = A[M,K] @ B[K,N]  (reference: cuda/matmul.cu:4-18 fp32, :55-71 bf16)."""
    sfx = dtype or _suffix(C, A, B)
    fn = getattr(lib, "b200_linear_forward_" + sfx)
    handle._check(fn(handle._h, _ptr(C), _ptr(A), _ptr(B), M, N, K), "matmul_forward")


def matmul_backward(handle, dA, dB, dC, A, B, M, N, K, dtype=None):
    """dA[M,K] = dC @ B^T (overwrite); dB[K,N] += A^T @ dC  (reference: cuda/matmul.cu:21-48, 73-104)."""
    sfx = dtype or _suffix(dA, dB, dC)
    fn = getattr(lib, "b200_linear_backward_" + sfx)
    handle._check(fn(handle._h, _ptr(dA), _ptr(dB), _ptr(dC), _ptr(A), _ptr(B), M, N, K), "matmul_backward")


def gemm(handle, which, beta1, out, x, y, M, N, K, dtype=None):
    """One product (FWD_NN / DGRAD_NT / WGRAD_TN) with beta in {0,1}: the sweep entry point."""
    sfx = dtype or _suffix(out, x, y)
    fn = getattr(lib, "b200_linear_gemm_" + sfx)
    handle._check(fn(handle._h, which, int(bool(beta1)), _ptr(out), _ptr(x), _ptr(y), M, N, K), "gemm")


def _ptr_ld(t):
    """Device address and row pitch (elements) of a 2-D tensor whose rows are contiguous: a dense matrix
    or a column range of a wider one."""
    if isinstance(t, tuple):
        return t
    if not t.is_cuda or t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise LinearError(1, "argument", " (need a CUDA matrix with contiguous rows)")
    return t.data_ptr(), t.stride(0)


def gemm_ld(handle, which, beta1, out, x, y, M, N, K):
    """bf16 product on operands with a row pitch: torch views such as W[:, c0:c1] (a vocabulary shard of
    the LM head where it lies), or (address, pitch) pairs."""
    (po, lo), (px, lx), (py, ly) = _ptr_ld(out), _ptr_ld(x), _ptr_ld(y)
    handle._check(lib.b200_linear_gemm_bf16_ld(handle._h, which, int(bool(beta1)), po, lo, px, lx, py, ly, M, N, K),
                  "gemm_ld")


def _ptr_array(tensors, n=3):
    arr = (ctypes.c_void_p * n)()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr() if t is not None else None
    return arr


def gemm_grouped(handle, which, beta1, outs, xs, ys, M, Ns, K):
    """Up to three bf16 products that share an operand in one launch (include/b200_linear.h,
    b200_linear_gemm_bf16_grouped): lists of torch CUDA tensors; xs may be a single tensor for FWD_NN / WGRAD_TN,
    outs a single tensor for DGRAD_NT."""
    n = len(Ns)
    outs = list(outs) if isinstance(outs, (list, tuple)) else [outs] * n
    xs = list(xs) if isinstance(xs, (list, tuple)) else [xs] * n
    lib.b200_linear_gemm_bf16_grouped.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                                  ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
    ns = (ctypes.c_int * 3)(*Ns)
    handle._check(lib.b200_linear_gemm_bf16_grouped(handle._h, which, int(bool(beta1)), n, _ptr_array(outs), _ptr_array(xs),
                                                    _ptr_array(ys), M, ns, K), "gemm_grouped")


def matmul_backward_grouped(handle, dA, dBs, dCs, A, Bs, M, Ns, K, accumulate_dA=False):
    """matmul_backward for several products on one input: dA (+)= sum_i dCs[i] Bs[i]^T, dBs[i] += A^T dCs[i]."""
    n = len(Ns)
    lib.b200_linear_backward_bf16_grouped.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                                      ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                      ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
    ns = (ctypes.c_int * 3)(*Ns)
    handle._check(lib.b200_linear_backward_bf16_grouped(
        handle._h, n, dA.data_ptr() if dA is not None else None, int(bool(accumulate_dA)),
        _ptr_array(dBs) if dBs is not None else None, _ptr_array(dCs), A.data_ptr() if A is not None else None,
        _ptr_array(Bs) if Bs is not None else None, M, ns, K), "matmul_backward_grouped")


def forward_ce_stats(handle, logits, x, w, M, N, K, targets, col0):
    """logits = x w (bf16; torch views with a row pitch allowed, as in gemm_ld) and, from the GEMM's epilogue, the
    cross-entropy statistics of the N local columns: returns (row_max, row_sum, row_target) fp32 [M], the outputs of
    ce_shard_stats without its pass over the stored logits (b200_linear_forward_ce_stats_bf16)."""
    import torch
    (po, lo), (px, lx), (pw, lw) = _ptr_ld(logits), _ptr_ld(x), _ptr_ld(w)
    out = [torch.empty(M, device=logits.device, dtype=torch.float32) for _ in range(3)]
    ll = ctypes.c_longlong
    lib.b200_linear_forward_ce_stats_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ll, ctypes.c_void_p, ll, ctypes.c_void_p, ll,
                                                      ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                                      ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    handle._check(lib.b200_linear_forward_ce_stats_bf16(handle._h, po, lo, px, lx, pw, lw, M, N, K, targets.data_ptr(), col0,
                                                        out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr()), "forward_ce_stats")
    return tuple(out)


def swiglu_forward_gemm(handle, gate, up, hidden, x, w_gate, w_up, M, ff, K):
    """gate = x w_gate, up = x w_up, hidden = SiLU(gate) * up in one launch (b200_linear_swiglu_forward_bf16)."""
    lib.b200_linear_swiglu_forward_bf16.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 3
    handle._check(lib.b200_linear_swiglu_forward_bf16(handle._h, gate.data_ptr(), up.data_ptr(), hidden.data_ptr(), x.data_ptr(),
                                                      w_gate.data_ptr(), w_up.data_ptr(), M, ff, K), "swiglu_forward_gemm")


def plan_bf16(which, beta1, M, N, K, sm_count=148):
    p = Plan()
    rc = lib.b200_linear_plan_bf16(which, int(bool(beta1)), M, N, K, sm_count, ctypes.byref(p))
    if rc:
        raise LinearError(rc, "plan_bf16", f" ({strerror(rc)})")
    return p


def plan_grouped_bf16(which, M, Ns, K, sm_count=148):
    """The plan of a grouped launch (host arithmetic only); bn == 0: the products would run one by one."""
    p = Plan()
    ns = (ctypes.c_int * 3)(*Ns)
    lib.b200_linear_plan_grouped_bf16.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                                  ctypes.c_int, ctypes.c_void_p]
    rc = lib.b200_linear_plan_grouped_bf16(which, len(Ns), M, ns, K, sm_count, ctypes.byref(p))
    if rc:
        raise LinearError(rc, "plan_grouped_bf16", f" ({strerror(rc)})")
    return p


# ---- cross-entropy over a vocabulary sharded across GPUs: the per-shard kernels (torch CUDA tensors in,
# ---- launched on torch's current stream; cuda/crossentropy.cu:96-132 is what they replace in that mode)
def _ce_check(rc, what):
    if rc != 0:
        raise LinearError(rc, what)


def _ce_args(logits, targets):
    import torch
    if not (logits.is_cuda and targets.is_cuda):
        raise LinearError(1, "ce_shard", "tensors must live on a CUDA device: there is no host path")
    if logits.dtype != torch.bfloat16 or logits.dim() != 2 or logits.stride(1) != 1 and logits.shape[1] > 0:
        raise LinearError(1, "ce_shard", "logits must be a row-major bf16 matrix")
    if targets.dtype != torch.int32 or not targets.is_contiguous() or targets.numel() != logits.shape[0]:
        raise LinearError(1, "ce_shard", "targets must be contiguous int32 [rows]")
    ld = logits.stride(0) if logits.shape[1] > 0 else 0
    return logits.shape[0], logits.shape[1], max(ld, logits.shape[1]), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ce_shard_stats(logits, targets, col0):
    """Row maximum, sum of exp(l - maximum) and target logit (0 where another shard owns the target) of this
    rank's logits [rows, V_r] = global columns [col0, col0 + V_r)."""
    import torch
    rows, cols, ld, stream = _ce_args(logits, targets)
    out = torch.empty(3, rows, device=logits.device, dtype=torch.float32)
    _ce_check(lib.b200_ce_shard_stats_bf16(logits.data_ptr() if cols else None, rows, cols, ld, targets.data_ptr(), col0,
                                            out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), stream),
              "ce_shard_stats")
    return out[0], out[1], out[2]


def ce_shard_rescale(local_max, global_max, row_sum):
    """row_sum *= exp(local_max - global_max), in place."""
    import torch
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _ce_check(lib.b200_ce_shard_rescale(local_max.data_ptr(), global_max.data_ptr(), row_sum.data_ptr(),
                                         row_sum.numel(), stream), "ce_shard_rescale")
    return row_sum


def ce_shard_loss(global_max, global_sum, target_logit):
    """Per-row loss -log softmax[target] = log(sum) + max - target logit (fp32)."""
    import torch
    loss = torch.empty_like(global_max)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _ce_check(lib.b200_ce_shard_loss(loss.data_ptr(), global_max.data_ptr(), global_sum.data_ptr(),
                                      target_logit.data_ptr(), loss.numel(), stream), "ce_shard_loss")
    return loss


def ce_shard_backward(logits, targets, col0, global_max, global_sum, scale, out=None):
    """dlogits = (exp(l - max) / sum - onehot) * scale for this rank's columns; out=logits works in place."""
    import torch
    rows, cols, ld, stream = _ce_args(logits, targets)
    if out is None:  # same shape and row pitch as the input, which may be a column range of a wider matrix
        out = torch.empty_strided(logits.shape, logits.stride(), dtype=logits.dtype, device=logits.device)
    if out.shape != logits.shape or out.stride() != logits.stride() or out.dtype != logits.dtype:
        raise LinearError(1, "ce_shard_backward", "out must match logits")
    _ce_check(lib.b200_ce_shard_backward_bf16(out.data_ptr() if cols else None, logits.data_ptr() if cols else None, rows,
                                               cols, ld, targets.data_ptr(), col0, global_max.data_ptr(),
                                               global_sum.data_ptr(), float(scale), stream), "ce_shard_backward")
    return out
