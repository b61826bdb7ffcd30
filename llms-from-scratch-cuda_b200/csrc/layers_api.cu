// The callers of the linear-layer path, as drop-ins: attention (with rotary embedding and the fused
// softmax(QK^T)V core), the SwiGLU feed-forward block and the softmax cross-entropy.  Each function keeps the
// signature -- and therefore the mangled name -- that the reference declares in cuda/kernels.cuh, so that
// the reference's host code links against this library with its own cuda/attention.cu,
// cuda/flash_attention.cu, cuda/swiglu.cu, cuda/crossentropy.cu, cuda/rmsnorm.cu, cuda/residual.cu and cuda/adamw.cu left out of the build:
//
//   flash_attention_forward / _backward  kernels.cuh:316-341 (fp32), :420-437 (bf16); bodies empty upstream
//                                        (flash_attention.cu:12-17, 51-57)
//   attention_forward / _backward        kernels.cuh:156-206 (fp32), :371-388 (bf16); attention.cu:235-414, 582-700
//   swiglu_forward / _backward           kernels.cuh:211-247 (fp32), :390-396 (bf16); swiglu.cu:49-130, 157-216
//   crossentropy_forward / crossentropy_softmax_backward
//                                        kernels.cuh:260-277 (fp32), :402-404 (bf16); crossentropy.cu:66-92, 134-151
//   rmsnorm_forward / rmsnorm_backward   kernels.cuh:87-105 (fp32), :359-362 (bf16); rmsnorm.cu:75-105, 168-178
//   residual_forward / residual_backward kernels.cuh:280-289 (fp32), :407-408 (bf16); residual.cu:32-49, 68-78
//   adamw_update, scale_grads, fp32_to_bf16, compute_grad_norm_bf16
//                                        kernels.cuh:299-309, 411-418; adamw.cu:42-58, 90-99, 153-191
//
// Differences from the reference, on purpose: no [B, n_head, T, T] matrix is ever formed (the `att` argument
// of attention_forward keeps the row log-sum-exps and the attention context instead, which is what the
// backward pass needs); temporaries come from a per-device scratch that grows on demand instead of one
// cudaMalloc / cudaFree pair per temporary per call; d(input) of the three projections accumulates in the
// GEMM's beta = 1 epilogue instead of through extra buffers and element-wise adds (same two bf16 roundings).
// Everything runs on the legacy default stream, like the reference.  Head dimension 64.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "../../include/b200_layers.h"
#include "../../include/b200_linear.h"
#include "attention_simt.cuh"
#include "attention_sm100.cuh"
#include "layers.cuh"

struct cublasContext;
typedef struct cublasContext* cublasHandle_t;

using namespace b200;

namespace {

constexpr int kMaxDev = 64;
enum Slot { S_CONTEXT, S_DCONTEXT, S_DQ, S_DK, S_DV, S_DELTA, S_LSE, S_HIDDEN, S_DHIDDEN, S_DGATE, S_DUP, S_RMS_PARTIAL, S_ROPE_TABLE, S_NORM_PARTIAL, S_COUNT };
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct Scratch {
    void* ptr[S_COUNT] = {};
    size_t bytes[S_COUNT] = {};
    bool attn_configured = false;
    bool simt_attention = false;   // B200_ATTN_SIMT=1: bf16 attention on the CUDA-core kernels as well
    int rope_T = 0, rope_hd = 0;   // what the cos / sin table in S_ROPE_TABLE was built for
    float rope_theta = 0.f;
    EncodeTiledFn encode = nullptr;
};
Scratch g_scratch[kMaxDev];

// Per-device scratch buffer `slot` of at least `bytes` bytes (grown, never shrunk); nullptr on failure.
void* scratch(int slot, size_t bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
    Scratch& s = g_scratch[dev];
    if (bytes <= s.bytes[slot]) return s.ptr[slot];
    if (s.ptr[slot]) cudaFree(s.ptr[slot]);
    s.ptr[slot] = nullptr;
    s.bytes[slot] = 0;
    const size_t want = bytes + (bytes >> 3);
    if (cudaMalloc(&s.ptr[slot], want) != cudaSuccess) return nullptr;
    s.bytes[slot] = want;
    return s.ptr[slot];
}

int configure_attention() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return B200_E_NODEVICE;
    if (g_scratch[dev].attn_configured) return B200_OK;
#define ATTN_SMEM(kern, bytes) \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return B200_E_CUDA
    ATTN_SMEM(attn_fwd_simt<float>, ATTN_FWD_SMEM);
    ATTN_SMEM(attn_fwd_simt<__nv_bfloat16>, ATTN_FWD_SMEM);
    ATTN_SMEM(attn_bwd_dq_simt<float>, ATTN_DQ_SMEM);
    ATTN_SMEM(attn_bwd_dq_simt<__nv_bfloat16>, ATTN_DQ_SMEM);
    ATTN_SMEM(attn_bwd_dkv_simt<float>, ATTN_DKV_SMEM);
    ATTN_SMEM(attn_bwd_dkv_simt<__nv_bfloat16>, ATTN_DKV_SMEM);
    ATTN_SMEM((attn_fwd_sm100<2, false>), FA_SMEM_BYTES);
    ATTN_SMEM((attn_fwd_sm100<4, false>), FA_SMEM_BYTES);
    ATTN_SMEM((attn_fwd_sm100<2, true>), FA_SMEM_BYTES_TS);
    ATTN_SMEM((attn_fwd_sm100<4, true>), FA_SMEM_BYTES_TS);
    ATTN_SMEM((attn_bwd_dq_sm100<2, false>), FB_DQ_SMEM_BYTES);
    ATTN_SMEM((attn_bwd_dq_sm100<4, false>), FB_DQ_SMEM_BYTES);
    ATTN_SMEM((attn_bwd_dq_sm100<2, true>), FB_DQ_SMEM_BYTES_TS);
    ATTN_SMEM((attn_bwd_dq_sm100<4, true>), FB_DQ_SMEM_BYTES_TS);
    ATTN_SMEM((attn_bwd_dkv_sm100<2, false>), FB_DKV_SMEM_BYTES);
    ATTN_SMEM((attn_bwd_dkv_sm100<4, false>), FB_DKV_SMEM_BYTES);
    ATTN_SMEM((attn_bwd_dkv_sm100<2, true>), FB_DKV_SMEM_BYTES_KT);
    ATTN_SMEM((attn_bwd_dkv_sm100<4, true>), FB_DKV_SMEM_BYTES_KT);
#undef ATTN_SMEM
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn)
        return B200_E_CUDA;
    g_scratch[dev].encode = reinterpret_cast<EncodeTiledFn>(fn);
    if (const char* e = getenv("B200_ATTN_SIMT")) g_scratch[dev].simt_attention = atoi(e) != 0;
    g_scratch[dev].attn_configured = true;
    return B200_OK;
}

// bf16 [B, T, width] seen as {width, T, B} with a box of 64 columns x `box_rows` rows of one batch: rows beyond T read as
// zero and are not written.
bool token_map(CUtensorMap* tm, const void* ptr, int B, int Tlen, int width, int box_rows) {
    int dev = 0;
    cudaGetDevice(&dev);
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(Tlen), static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(width) * 2, static_cast<cuuint64_t>(Tlen) * width * 2};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return g_scratch[dev].encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Every kernel of this file begins with griddep_sync(): launched with programmatic stream serialization, its blocks
// may be scheduled while the previous kernel's last blocks retire, and wait there until that kernel has completed.
// B200_LINEAR_PDL=0 launches them fully serialized.
bool layers_pdl() {
    static const bool on = [] {
        const char* e = getenv("B200_LINEAR_PDL");
        return !(e && atoi(e) == 0);
    }();
    return on;
}
template <typename... Exp, typename... Act>
void launch_pdl(void (*kern)(Exp...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Act&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = layers_pdl() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kern, static_cast<Exp>(args)...);   // a failure is read back by the caller (cudaGetLastError)
}

bool use_tensor_cores(const void* a, const void* b, const void* c, const void* d) {
    int dev = 0;
    cudaGetDevice(&dev);
    return !g_scratch[dev].simt_attention &&
           ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
             reinterpret_cast<uintptr_t>(d)) & 15) == 0;
}

// The three switches below are read at every call (a getenv beside a kernel launch), so that a test can flip them.
int attn_row_threads() {   // B200_ATTN_ROW_THREADS: 0 (unset) = chosen per call
    const char* e = getenv("B200_ATTN_ROW_THREADS");
    const int n = e ? atoi(e) : 0;
    return (n == 2 || n == 4) ? n : 0;
}
// B200_ATTN_DKV_TRANSPOSED=1: the dK / dV kernel in its "keys on the lanes" form (S^T, dP^T; P^T and dS^T as
// tensor-memory operands).  Correct, but measured slower than the shared-memory form (T = 8192 backward 1013 us
// against 918 us), so it is off unless asked for.
bool attn_dkv_transposed() {
    const char* e = getenv("B200_ATTN_DKV_TRANSPOSED");
    return e && atoi(e) != 0;
}

// P (forward) and dS (dQ kernel) reach the tensor core as a tensor-memory operand; B200_ATTN_P_TMEM=0 sends them
// through shared memory instead (T = 8192 forward 361 us instead of 322 us).
bool attn_operand_in_tmem() {
    const char* e = getenv("B200_ATTN_P_TMEM");
    return !(e && atoi(e) == 0);
}

int flash_forward_tc(__nv_bfloat16* context, float* lse, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                     int B, int Tlen, int n_head, int n_kv_head, cudaStream_t stream) {
    b200_linear_ctx* ctx = b200_linear_default_ctx();
    CUtensorMap tmQ, tmK, tmV, tmO;
    if (!token_map(&tmQ, q, B, Tlen, n_head * FA_HD, FA_BQ) || !token_map(&tmK, k, B, Tlen, n_kv_head * FA_HD, FA_BKV) ||
        !token_map(&tmV, v, B, Tlen, n_kv_head * FA_HD, FA_BKV) || !token_map(&tmO, context, B, Tlen, n_head * FA_HD, FA_BQ))
        return B200_E_CUDA;
    FaParams p;
    p.B = B; p.T = Tlen; p.n_head = n_head; p.n_kv_head = n_kv_head;
    p.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(FA_HD));
    p.lse = lse;
    p.status = b200_linear_status_word(ctx);
    const dim3 grid(n_head, B, (Tlen + FA_BQ - 1) / FA_BQ);
    // Softmax threads per query row: four (16 softmax warps) pay once a block walks many key tiles (T = 8192: 361 us
    // against 395 us with two), two are quicker for short sequences (T = 512: 39.7 against 41.1 us).
    // B200_ATTN_ROW_THREADS=2|4 forces one.
    const int forced = attn_row_threads();
    const bool two = forced ? forced == 2 : Tlen < 2048;
    if (attn_operand_in_tmem()) {
        if (two) launch_pdl(attn_fwd_sm100<2, true>, grid, 128 + 2 * 128, FA_SMEM_BYTES_TS, stream, tmQ, tmK, tmV, tmO, p);
        else launch_pdl(attn_fwd_sm100<4, true>, grid, 128 + 4 * 128, FA_SMEM_BYTES_TS, stream, tmQ, tmK, tmV, tmO, p);
    } else {
        if (two) launch_pdl(attn_fwd_sm100<2, false>, grid, 128 + 2 * 128, FA_SMEM_BYTES, stream, tmQ, tmK, tmV, tmO, p);
        else launch_pdl(attn_fwd_sm100<4, false>, grid, 128 + 4 * 128, FA_SMEM_BYTES, stream, tmQ, tmK, tmV, tmO, p);
    }
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_E_CUDA;
}

int launch_ok() { return cudaGetLastError() == cudaSuccess ? B200_OK : B200_E_CUDA; }

bool attn_args_ok(int B, int T, int n_head, int n_kv_head, int head_dim) {
    return B > 0 && T > 0 && n_head > 0 && n_kv_head > 0 && n_head % n_kv_head == 0 && head_dim == AT_TILE &&
           B <= 65535 && n_head <= 65535;
}

template <typename T>
int flash_forward(T* context, float* lse, const T* q, const T* k, const T* v, int B, int Tlen, int n_head, int n_kv_head,
                  int head_dim, cudaStream_t stream) {
    if (!context || !lse || !q || !k || !v || !attn_args_ok(B, Tlen, n_head, n_kv_head, head_dim)) return B200_E_BADARG;
    int rc = configure_attention();
    if (rc) return rc;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        if (use_tensor_cores(context, q, k, v)) return flash_forward_tc(context, lse, q, k, v, B, Tlen, n_head, n_kv_head, stream);
    }
    const AttnParams p{B, Tlen, n_head, n_kv_head, 1.0f / sqrtf(static_cast<float>(head_dim))};
    const dim3 grid((Tlen + AT_TILE - 1) / AT_TILE, n_head, B);
    launch_pdl(attn_fwd_simt<T>, grid, AT_THREADS, ATTN_FWD_SMEM, stream, context, lse, q, k, v, p);
    return launch_ok();
}

int flash_backward_tc(__nv_bfloat16* dq, __nv_bfloat16* dk, __nv_bfloat16* dv, const __nv_bfloat16* dcontext,
                      const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, const float* lse, const float* delta,
                      int B, int Tlen, int n_head, int n_kv_head, cudaStream_t stream) {
    b200_linear_ctx* ctx = b200_linear_default_ctx();
    CUtensorMap tmQ, tmdO, tmK, tmV, tmdQ, tmdK, tmdV;
    const int C = n_head * FA_HD, KV = n_kv_head * FA_HD;
    if (!token_map(&tmQ, q, B, Tlen, C, FA_BQ) || !token_map(&tmdO, dcontext, B, Tlen, C, FA_BQ) ||
        !token_map(&tmK, k, B, Tlen, KV, FA_BKV) || !token_map(&tmV, v, B, Tlen, KV, FA_BKV) ||
        !token_map(&tmdQ, dq, B, Tlen, C, FA_BQ) || !token_map(&tmdK, dk, B, Tlen, KV, FA_BKV) ||
        !token_map(&tmdV, dv, B, Tlen, KV, FA_BKV))
        return B200_E_CUDA;
    FbParams p;
    p.B = B; p.T = Tlen; p.n_head = n_head; p.n_kv_head = n_kv_head;
    p.scale = 1.0f / sqrtf(static_cast<float>(FA_HD));
    p.scale_log2e = 1.4426950408889634f * p.scale;
    p.lse = lse;
    p.delta = delta;
    p.status = b200_linear_status_word(ctx);
    const int tiles = (Tlen + FA_BQ - 1) / FA_BQ;
    // two softmax threads per query row for the backward kernels (four measured 3-6 % slower at T = 512 and T = 8192)
    // unless B200_ATTN_ROW_THREADS=4 forces four
    const bool two = attn_row_threads() != 4;
    const bool ts = attn_operand_in_tmem(), kt = attn_dkv_transposed();
    if (two) {
        if (ts) launch_pdl(attn_bwd_dq_sm100<2, true>, dim3(n_head, B, tiles), 128 + 2 * 128, FB_DQ_SMEM_BYTES_TS, stream, tmQ, tmdO, tmK, tmV, tmdQ, p);
        else launch_pdl(attn_bwd_dq_sm100<2, false>, dim3(n_head, B, tiles), 128 + 2 * 128, FB_DQ_SMEM_BYTES, stream, tmQ, tmdO, tmK, tmV, tmdQ, p);
        if (kt) launch_pdl(attn_bwd_dkv_sm100<2, true>, dim3(n_kv_head, B, tiles), 128 + 2 * 128, FB_DKV_SMEM_BYTES_KT, stream, tmQ, tmdO, tmK, tmV, tmdK, tmdV, p);
        else launch_pdl(attn_bwd_dkv_sm100<2, false>, dim3(n_kv_head, B, tiles), 128 + 2 * 128, FB_DKV_SMEM_BYTES, stream, tmQ, tmdO, tmK, tmV, tmdK, tmdV, p);
    } else {
        if (ts) launch_pdl(attn_bwd_dq_sm100<4, true>, dim3(n_head, B, tiles), 128 + 4 * 128, FB_DQ_SMEM_BYTES_TS, stream, tmQ, tmdO, tmK, tmV, tmdQ, p);
        else launch_pdl(attn_bwd_dq_sm100<4, false>, dim3(n_head, B, tiles), 128 + 4 * 128, FB_DQ_SMEM_BYTES, stream, tmQ, tmdO, tmK, tmV, tmdQ, p);
        if (kt) launch_pdl(attn_bwd_dkv_sm100<4, true>, dim3(n_kv_head, B, tiles), 128 + 4 * 128, FB_DKV_SMEM_BYTES_KT, stream, tmQ, tmdO, tmK, tmV, tmdK, tmdV, p);
        else launch_pdl(attn_bwd_dkv_sm100<4, false>, dim3(n_kv_head, B, tiles), 128 + 4 * 128, FB_DKV_SMEM_BYTES, stream, tmQ, tmdO, tmK, tmV, tmdK, tmdV, p);
    }
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_E_CUDA;
}

// context == nullptr: the forward pass is run again into scratch to get it (the reference's flash API does
// not hand the context to the backward pass).
template <typename T>
int flash_backward(T* dq, T* dk, T* dv, const T* dcontext, const T* q, const T* k, const T* v, const float* lse,
                   const T* context, int B, int Tlen, int n_head, int n_kv_head, int head_dim, cudaStream_t stream) {
    if (!dq || !dk || !dv || !dcontext || !q || !k || !v || !lse || !attn_args_ok(B, Tlen, n_head, n_kv_head, head_dim))
        return B200_E_BADARG;
    int rc = configure_attention();
    if (rc) return rc;
    const AttnParams p{B, Tlen, n_head, n_kv_head, 1.0f / sqrtf(static_cast<float>(head_dim))};
    const size_t rows = static_cast<size_t>(B) * n_head * Tlen;
    float* delta = static_cast<float*>(scratch(S_DELTA, rows * sizeof(float)));
    if (!delta) return B200_E_CUDA;
    if (!context) {
        T* ctx_tmp = static_cast<T*>(scratch(S_CONTEXT, static_cast<size_t>(B) * Tlen * n_head * head_dim * sizeof(T)));
        float* lse_tmp = static_cast<float*>(scratch(S_LSE, rows * sizeof(float)));
        if (!ctx_tmp || !lse_tmp) return B200_E_CUDA;
        rc = flash_forward<T>(ctx_tmp, lse_tmp, q, k, v, B, Tlen, n_head, n_kv_head, head_dim, stream);
        if (rc) return rc;
        context = ctx_tmp;
    }
    bool delta_done = false;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        if (head_dim == 64 && ((reinterpret_cast<uintptr_t>(dcontext) | reinterpret_cast<uintptr_t>(context)) & 15) == 0) {
            const long long tokens = static_cast<long long>(B) * Tlen;
            launch_pdl(attn_delta_bf16x8, static_cast<unsigned>((tokens + 7) / 8 < 148 * 16 ? (tokens + 7) / 8 : 148 * 16), 256, 0, stream,
                       delta, reinterpret_cast<const uint4*>(dcontext), reinterpret_cast<const uint4*>(context), B, Tlen, n_head);
            delta_done = true;
        }
    }
    if (!delta_done)
        launch_pdl(attn_delta<T>, static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, stream, delta, dcontext, context, p);
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        if (use_tensor_cores(dq, dk, dv, dcontext) && use_tensor_cores(q, k, v, q))
            return flash_backward_tc(dq, dk, dv, dcontext, q, k, v, lse, delta, B, Tlen, n_head, n_kv_head, stream);
    }
    const int tiles = (Tlen + AT_TILE - 1) / AT_TILE;
    launch_pdl(attn_bwd_dq_simt<T>, dim3(tiles, n_head, B), AT_THREADS, ATTN_DQ_SMEM, stream, dq, dcontext, q, k, v, lse, delta, p);
    launch_pdl(attn_bwd_dkv_simt<T>, dim3(tiles, n_kv_head, B), AT_THREADS, ATTN_DKV_SMEM, stream, dk, dv, dcontext, q, k, v, lse,
                                                                                         delta, p);
    return launch_ok();
}

template <typename T, int DIR>
int rope(T* q, T* k, int B, int Tlen, int n_head, int n_kv_head, int head_dim, float theta, cudaStream_t stream) {
    if (!q || !k || B <= 0 || Tlen <= 0 || head_dim <= 0 || (head_dim & 1) || head_dim > 128) return B200_E_BADARG;
    const long long total = static_cast<long long>(B) * Tlen * (n_head + n_kv_head) * (head_dim / 2);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return B200_E_NODEVICE;
    Scratch& sc = g_scratch[dev];
    const int half = head_dim / 2;
    float2* table = static_cast<float2*>(scratch(S_ROPE_TABLE, static_cast<size_t>(Tlen) * half * sizeof(float2)));
    if (!table) return B200_E_CUDA;
    if (sc.rope_T != Tlen || sc.rope_hd != head_dim || sc.rope_theta != theta) {
        // Rebuilt only when the sequence length, head dimension or base changes; the host waits for it once, so that
        // calls on any other stream may use it afterwards.
        RopeFreq freqs;
        for (int i = 0; i < half; ++i)  // cuda/rope.cu:29: 1 / theta^(2i / head_dim)
            freqs.f[i] = static_cast<float>(1.0 / pow(static_cast<double>(theta), (2.0 * i) / head_dim));
        launch_pdl(rope_table_kernel, (Tlen * half + 255) / 256, 256, 0, stream, table, Tlen, half, freqs);
        if (cudaStreamSynchronize(stream) != cudaSuccess) return B200_E_CUDA;
        sc.rope_T = Tlen; sc.rope_hd = head_dim; sc.rope_theta = theta;
    }
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        if ((head_dim % 8) == 0 && ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k)) & 15) == 0) {
            const long long total_vec = total / 4;
            launch_pdl(rope_kernel_bf16x8<DIR>, static_cast<unsigned>((total_vec + 255) / 256), 256, 0, stream, reinterpret_cast<uint4*>(q), reinterpret_cast<uint4*>(k), total_vec, Tlen, n_head, n_kv_head, head_dim, table);
            return launch_ok();
        }
    }
    launch_pdl(rope_kernel<T, DIR>, static_cast<unsigned>((total + 255) / 256), 256, 0, stream, q, k, total, Tlen, n_head, n_kv_head,
                                                                                       head_dim, table);
    return launch_ok();
}

#define TRY(expr)              \
    do {                       \
        int rc__ = (expr);     \
        if (rc__) return rc__; \
    } while (0)

// GEMM dispatch by storage type.
int gemm(b200_linear_ctx* ctx, int which, int beta1, __nv_bfloat16* out, const __nv_bfloat16* x, const __nv_bfloat16* y, int M,
         int N, int K) {
    return b200_linear_gemm_bf16(ctx, which, beta1, out, x, y, M, N, K);
}
int gemm(b200_linear_ctx* ctx, int which, int beta1, float* out, const float* x, const float* y, int M, int N, int K) {
    return b200_linear_gemm_f32(ctx, which, beta1, out, x, y, M, N, K);
}
int backward(b200_linear_ctx* ctx, __nv_bfloat16* dA, __nv_bfloat16* dB, const __nv_bfloat16* dC, const __nv_bfloat16* A,
             const __nv_bfloat16* Bm, int M, int N, int K) {
    return b200_linear_backward_bf16(ctx, dA, dB, dC, A, Bm, M, N, K);
}
int backward(b200_linear_ctx* ctx, float* dA, float* dB, const float* dC, const float* A, const float* Bm, int M, int N, int K) {
    return b200_linear_backward_f32(ctx, dA, dB, dC, A, Bm, M, N, K);
}

// Several projections of one input (Q, K, V; gate, up): one launch each way for bf16 (b200_linear_gemm_bf16_grouped),
// one product at a time for fp32 or with B200_LINEAR_GROUPED=0.
bool grouped_launches() {
    static const bool on = [] {
        const char* e = getenv("B200_LINEAR_GROUPED");
        return !(e && atoi(e) == 0);
    }();
    return on;
}
bool fused_swiglu() {   // B200_LINEAR_FUSED_SWIGLU=0: gate / up GEMMs and the element-wise kernel separately
    static const bool on = [] {
        const char* e = getenv("B200_LINEAR_FUSED_SWIGLU");
        return !(e && atoi(e) == 0);
    }();
    return on;
}
template <typename T>
int forward_group(b200_linear_ctx* ctx, int count, T* const* outs, const T* x, const T* const* ws, int M, const int* Ns, int K) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        if (grouped_launches()) {
            const void* xs[3] = {x, x, x};
            return b200_linear_gemm_bf16_grouped(ctx, B200_GEMM_FWD_NN, 0, count, reinterpret_cast<void* const*>(outs), xs,
                                                 reinterpret_cast<const void* const*>(ws), M, Ns, K);
        }
    }
    for (int i = 0; i < count; ++i) TRY(gemm(ctx, B200_GEMM_FWD_NN, 0, outs[i], x, ws[i], M, Ns[i], K));
    return B200_OK;
}
// dA = sum_i dCs[i] * Bs[i]^T, dBs[i] += A^T * dCs[i]
template <typename T>
int backward_group(b200_linear_ctx* ctx, int count, T* dA, T* const* dBs, const T* const* dCs, const T* A, const T* const* Bs,
                   int M, const int* Ns, int K) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        if (grouped_launches())
            return b200_linear_backward_bf16_grouped(ctx, count, dA, 0, reinterpret_cast<void* const*>(dBs),
                                                     reinterpret_cast<const void* const*>(dCs), A,
                                                     reinterpret_cast<const void* const*>(Bs), M, Ns, K);
    }
    TRY(backward(ctx, dA, dBs[0], dCs[0], A, Bs[0], M, Ns[0], K));
    for (int i = 1; i < count; ++i) {   // the other inputs' gradients accumulate through the beta = 1 epilogue
        TRY(gemm(ctx, B200_GEMM_DGRAD_NT, 1, dA, dCs[i], Bs[i], M, Ns[i], K));
        TRY(gemm(ctx, B200_GEMM_WGRAD_TN, 1, dBs[i], A, dCs[i], M, Ns[i], K));
    }
    return B200_OK;
}

// What attention_forward leaves in the caller's `att` buffer ([B, n_head, T, T] elements of T in the reference):
// the row log-sum-exps (fp32) followed, 256-byte aligned, by the attention context [B*T, C].  It fits whenever
// T >= 68; for shorter sequences the backward pass recomputes both.
template <typename T>
struct AttStash {
    float* lse;
    T* context;
    bool fits;
    AttStash(void* att, int B, int Tlen, int C, int n_head) {
        const size_t lse_bytes = ((static_cast<size_t>(B) * n_head * Tlen * sizeof(float) + 255) / 256) * 256;
        const size_t ctx_bytes = static_cast<size_t>(B) * Tlen * C * sizeof(T);
        fits = att != nullptr && lse_bytes + ctx_bytes <= static_cast<size_t>(B) * n_head * Tlen * Tlen * sizeof(T) &&
               (reinterpret_cast<uintptr_t>(att) & 15) == 0;
        lse = static_cast<float*>(att);
        context = reinterpret_cast<T*>(static_cast<char*>(att) + lse_bytes);
    }
};

template <typename T>
int attention_fwd(b200_linear_ctx* ctx, T* out, T* q, T* k, T* v, void* att, const T* inp, const T* wq, const T* wk,
                  const T* wv, const T* wo, int B, int Tlen, int C, int n_head, int n_kv_head, float rope_theta) {
    if (!ctx || !out || !q || !k || !v || !inp || !wq || !wk || !wv || !wo || n_head <= 0 || C % n_head != 0) return B200_E_BADARG;
    const int hd = C / n_head, kv = n_kv_head * hd, BT = B * Tlen;
    if (!attn_args_ok(B, Tlen, n_head, n_kv_head, hd)) return B200_E_BADARG;
    {   // attention.cu:597-599
        T* const outs[3] = {q, k, v};
        const T* const ws[3] = {wq, wk, wv};
        const int Ns[3] = {C, kv, kv};
        TRY(forward_group<T>(ctx, 3, outs, inp, ws, BT, Ns, C));
    }
    TRY((rope<T, +1>(q, k, B, Tlen, n_head, n_kv_head, hd, rope_theta, nullptr)));
    AttStash<T> st(att, B, Tlen, C, n_head);
    T* context = st.context;
    float* lse = st.lse;
    if (!st.fits) {
        context = static_cast<T*>(scratch(S_CONTEXT, static_cast<size_t>(BT) * C * sizeof(T)));
        lse = static_cast<float*>(scratch(S_LSE, static_cast<size_t>(B) * n_head * Tlen * sizeof(float)));
        if (!context || !lse) return B200_E_CUDA;
    }
    TRY(flash_forward<T>(context, lse, q, k, v, B, Tlen, n_head, n_kv_head, hd, nullptr));
    return gemm(ctx, B200_GEMM_FWD_NN, 0, out, context, wo, BT, C, C);
}

template <typename T>
int attention_bwd(b200_linear_ctx* ctx, T* dinp, T* dwq, T* dwk, T* dwv, T* dwo, const T* dout, const T* inp, const T* q,
                  const T* k, const T* v, const void* att, const T* wq, const T* wk, const T* wv, const T* wo, int B,
                  int Tlen, int C, int n_head, int n_kv_head, float rope_theta) {
    if (!ctx || !dinp || !dwq || !dwk || !dwv || !dwo || !dout || !inp || !q || !k || !v || !wq || !wk || !wv || !wo ||
        n_head <= 0 || C % n_head != 0)
        return B200_E_BADARG;
    const int hd = C / n_head, kv = n_kv_head * hd, BT = B * Tlen;
    if (!attn_args_ok(B, Tlen, n_head, n_kv_head, hd)) return B200_E_BADARG;
    AttStash<T> st(const_cast<void*>(att), B, Tlen, C, n_head);
    const T* context = st.context;
    const float* lse = st.lse;
    if (!st.fits) {  // short sequences: nothing was kept, run the fused forward again
        T* c2 = static_cast<T*>(scratch(S_CONTEXT, static_cast<size_t>(BT) * C * sizeof(T)));
        float* l2 = static_cast<float*>(scratch(S_LSE, static_cast<size_t>(B) * n_head * Tlen * sizeof(float)));
        if (!c2 || !l2) return B200_E_CUDA;
        TRY(flash_forward<T>(c2, l2, q, k, v, B, Tlen, n_head, n_kv_head, hd, nullptr));
        context = c2;
        lse = l2;
    }
    T* dcontext = static_cast<T*>(scratch(S_DCONTEXT, static_cast<size_t>(BT) * C * sizeof(T)));
    T* dq = static_cast<T*>(scratch(S_DQ, static_cast<size_t>(BT) * C * sizeof(T)));
    T* dk = static_cast<T*>(scratch(S_DK, static_cast<size_t>(BT) * kv * sizeof(T)));
    T* dv = static_cast<T*>(scratch(S_DV, static_cast<size_t>(BT) * kv * sizeof(T)));
    if (!dcontext || !dq || !dk || !dv) return B200_E_CUDA;
    TRY(backward(ctx, dcontext, dwo, dout, context, wo, BT, C, C));                       // attention.cu:640
    TRY(flash_backward<T>(dq, dk, dv, dcontext, q, k, v, lse, context, B, Tlen, n_head, n_kv_head, hd, nullptr));
    TRY((rope<T, -1>(dq, dk, B, Tlen, n_head, n_kv_head, hd, rope_theta, nullptr)));          // attention.cu:669
    // attention.cu:671-688: the three projections' weight gradients, and d(input) = the sum of their input gradients
    T* const dws[3] = {dwq, dwk, dwv};
    const T* const dcs[3] = {dq, dk, dv};
    const T* const ws[3] = {wq, wk, wv};
    const int Ns[3] = {C, kv, kv};
    return backward_group<T>(ctx, 3, dinp, dws, dcs, inp, ws, BT, Ns, C);
}

template <typename T>
int swiglu_gate(T* hidden, const T* gate, const T* up, long long n) {
    const bool vec = sizeof(T) == 2 && (n % 8) == 0 &&
                     ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up)) & 15) == 0;
    if (vec) {
        const long long n8 = n / 8;
        launch_pdl(swiglu_gate_kernel_bf16x8, static_cast<unsigned>((n8 + 255) / 256 < 65535 * 16 ? (n8 + 255) / 256 : 65535 * 16), 256, 0, nullptr, reinterpret_cast<uint4*>(hidden), reinterpret_cast<const uint4*>(gate), reinterpret_cast<const uint4*>(up), n8);
    } else {
        launch_pdl(swiglu_gate_kernel<T>, static_cast<unsigned>((n + 255) / 256 < 65535 * 16 ? (n + 255) / 256 : 65535 * 16), 256, 0, nullptr, hidden, gate, up, n);
    }
    return launch_ok();
}

template <typename T>
int swiglu_fwd(b200_linear_ctx* ctx, T* out, T* gate, T* up, T* hidden, const T* inp, const T* w_gate, const T* w_up,
               const T* w_down, int BT, int C, int ff) {
    if (!ctx || !out || !gate || !up || !hidden || !inp || !w_gate || !w_up || !w_down || BT <= 0 || C <= 0 || ff <= 0)
        return B200_E_BADARG;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        // gate, up and hidden from one launch (SiLU(gate) * up in the GEMM's epilogue) where the shapes allow
        if (grouped_launches() && fused_swiglu()) {
            const int rc = b200_linear_swiglu_forward_bf16(ctx, gate, up, hidden, inp, w_gate, w_up, BT, ff, C);
            if (rc == B200_OK) return gemm(ctx, B200_GEMM_FWD_NN, 0, out, hidden, w_down, BT, C, ff);
            if (rc != B200_E_BADARG) return rc;
        }
    }
    {   // swiglu.cu:161-162
        T* const outs[2] = {gate, up};
        const T* const ws[2] = {w_gate, w_up};
        const int Ns[2] = {ff, ff};
        TRY(forward_group<T>(ctx, 2, outs, inp, ws, BT, Ns, C));
    }
    TRY(swiglu_gate<T>(hidden, gate, up, static_cast<long long>(BT) * ff));
    return gemm(ctx, B200_GEMM_FWD_NN, 0, out, hidden, w_down, BT, C, ff);
}

template <typename T>
int swiglu_bwd(b200_linear_ctx* ctx, T* dinp, T* dw_gate, T* dw_up, T* dw_down, const T* dout, const T* inp, const T* gate,
               const T* up, const T* w_gate, const T* w_up, const T* w_down, int BT, int C, int ff) {
    if (!ctx || !dinp || !dw_gate || !dw_up || !dw_down || !dout || !inp || !gate || !up || !w_gate || !w_up || !w_down ||
        BT <= 0 || C <= 0 || ff <= 0)
        return B200_E_BADARG;
    const long long n = static_cast<long long>(BT) * ff;
    T* hidden = static_cast<T*>(scratch(S_HIDDEN, n * sizeof(T)));
    T* dhidden = static_cast<T*>(scratch(S_DHIDDEN, n * sizeof(T)));
    T* dgate = static_cast<T*>(scratch(S_DGATE, n * sizeof(T)));
    T* dup = static_cast<T*>(scratch(S_DUP, n * sizeof(T)));
    if (!hidden || !dhidden || !dgate || !dup) return B200_E_CUDA;
    TRY(swiglu_gate<T>(hidden, gate, up, n));                                              // swiglu.cu:184
    TRY(backward(ctx, dhidden, dw_down, dout, hidden, w_down, BT, C, ff));                 // swiglu.cu:192
    const bool vec = sizeof(T) == 2 && (n % 8) == 0;
    const unsigned blocks = static_cast<unsigned>(((vec ? n / 8 : n) + 255) / 256 < 65535 * 16 ? ((vec ? n / 8 : n) + 255) / 256 : 65535 * 16);
    if (vec)
        launch_pdl(swiglu_gate_backward_kernel_bf16x8, blocks, 256, 0, nullptr, reinterpret_cast<uint4*>(dgate), reinterpret_cast<uint4*>(dup),
                                                            reinterpret_cast<const uint4*>(dhidden),
                                                            reinterpret_cast<const uint4*>(gate),
                                                            reinterpret_cast<const uint4*>(up), n / 8);
    else
        launch_pdl(swiglu_gate_backward_kernel<T>, blocks, 256, 0, nullptr, dgate, dup, dhidden, gate, up, n);
    TRY(launch_ok());
    // swiglu.cu:197-208: both projections' weight gradients, and d(input) = the sum of their input gradients
    T* const dws[2] = {dw_gate, dw_up};
    const T* const dcs[2] = {dgate, dup};
    const T* const ws[2] = {w_gate, w_up};
    const int Ns[2] = {ff, ff};
    return backward_group<T>(ctx, 2, dinp, dws, dcs, inp, ws, BT, Ns, C);
}

template <typename T>
int ce_forward(float* losses, T* logits_probs, const int* targets, int B, int Tlen, int V) {
    if (!losses || !logits_probs || !targets || B <= 0 || Tlen <= 0 || V <= 0) return B200_E_BADARG;
    const int rows = B * Tlen;
    // The kernel walks a row three times (maximum, exponentials, normalisation); the second and third walk are meant
    // to hit L2.  With long rows (128 256 entries = 250 KB) four resident blocks per SM keep 150 MB in flight, more
    // than the 126 MB L2 holds, and the later walks go back to HBM: an (unused) dynamic shared-memory request caps the
    // residency so that the rows in flight stay below ~96 MB.
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        return B200_E_CUDA;
    const double row_bytes = static_cast<double>(V) * sizeof(T);
    int resident = static_cast<int>(96.0e6 / row_bytes / sms);
    resident = resident < 1 ? 1 : (resident > 4 ? 4 : resident);
    size_t pad = 0;
    if (resident < 4) {
        pad = static_cast<size_t>(227 * 1024 / resident - 2048) & ~static_cast<size_t>(1023);
        static bool configured[kMaxDev][2] = {};
        if (dev < kMaxDev && !configured[dev][sizeof(T) == 2]) {
            if (cudaFuncSetAttribute(ce_row_forward<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048) != cudaSuccess)
                return B200_E_CUDA;
            configured[dev][sizeof(T) == 2] = true;
        }
    }
    launch_pdl(ce_row_forward<T>, rows, CE_ROW_THREADS, pad, nullptr, losses, logits_probs, targets, rows, V);
    return launch_ok();
}

template <typename T>
int ce_backward(T* dlogits, const T* probs, const int* targets, int B, int Tlen, int V, float scale) {
    if (!dlogits || !probs || !targets || B <= 0 || Tlen <= 0 || V <= 0) return B200_E_BADARG;
    const int rows = B * Tlen;
    const bool vec = sizeof(T) == 2 && (V % 8) == 0 &&
                     ((reinterpret_cast<uintptr_t>(dlogits) | reinterpret_cast<uintptr_t>(probs)) & 15) == 0;
    const long long n = static_cast<long long>(rows) * (vec ? V / 8 : V);
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256 < 148LL * 64 ? (n + 255) / 256 : 148LL * 64);
    if (vec)
        launch_pdl(ce_row_backward_bf16x8, blocks, 256, 0, nullptr, reinterpret_cast<uint4*>(dlogits), reinterpret_cast<const uint4*>(probs),
                                                targets, scale, rows, V / 8);
    else
        launch_pdl(ce_row_backward<T>, blocks, 256, 0, nullptr, dlogits, probs, targets, scale, rows, V);
    return launch_ok();
}

template <typename T>
int rmsnorm_fwd(T* out, float* rrms, const T* inp, const T* weight, float eps, int rows, int C) {
    if (!out || !rrms || !inp || !weight || rows <= 0 || C <= 0) return B200_E_BADARG;
    const int blocks = (rows + 7) / 8 < 148 * 8 ? (rows + 7) / 8 : 148 * 8;   // 8 warps per CTA, one row per warp at a time
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        if ((C % 8) == 0 && C <= 32 * 8 * RMS_VEC_MAX &&
            ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(inp) | reinterpret_cast<uintptr_t>(weight)) & 15) == 0) {
            launch_pdl(rmsnorm_fwd_bf16x8, blocks, 256, 0, nullptr, reinterpret_cast<uint4*>(out), rrms, reinterpret_cast<const uint4*>(inp),
                                                reinterpret_cast<const uint4*>(weight), eps, rows, C);
            return launch_ok();
        }
    }
    launch_pdl(rmsnorm_fwd_kernel<T>, blocks, 256, 0, nullptr, out, rrms, inp, weight, eps, rows, C);
    return launch_ok();
}

template <typename T>
int rmsnorm_bwd(T* dinp, T* dweight, const T* dout, const T* inp, const T* weight, const float* rrms, int rows, int C) {
    if (!dinp || !dweight || !dout || !inp || !weight || !rrms || rows <= 0 || C <= 0) return B200_E_BADARG;
    const int blocks = (rows + 7) / 8 < 148 * 8 ? (rows + 7) / 8 : 148 * 8;
    const int rows_per_chunk = rows >= 4096 ? 64 : 16;
    const int chunks = (rows + rows_per_chunk - 1) / rows_per_chunk;
    constexpr int kFusedBlocks = 148 * 2;
    const size_t partial_rows = chunks > kFusedBlocks ? chunks : kFusedBlocks;
    float* partial = static_cast<float*>(scratch(S_RMS_PARTIAL, partial_rows * C * sizeof(float)));
    if (!partial) return B200_E_CUDA;
    bool vec = false;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        vec = (C % 8) == 0 && C <= 32 * 8 * RMS_VEC_MAX &&
              ((reinterpret_cast<uintptr_t>(dinp) | reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(inp) |
                reinterpret_cast<uintptr_t>(weight)) & 15) == 0;
        if (vec && C <= 1024) {
            // one pass: d(input) and the per-block partial sums of d(weight), then the fixed-order reduction
            const int fb = (rows + 7) / 8 < kFusedBlocks ? (rows + 7) / 8 : kFusedBlocks;
            auto args = [&](auto kern) {
                launch_pdl(kern, fb, 256, 0, nullptr, reinterpret_cast<uint4*>(dinp), partial, reinterpret_cast<const uint4*>(dout),
                           reinterpret_cast<const uint4*>(inp), reinterpret_cast<const uint4*>(weight), rrms, rows, C);
            };
            if (C <= 256) args(rmsnorm_bwd_fused_bf16x8<1>);
            else if (C <= 512) args(rmsnorm_bwd_fused_bf16x8<2>);
            else if (C <= 768) args(rmsnorm_bwd_fused_bf16x8<3>);
            else args(rmsnorm_bwd_fused_bf16x8<4>);
            launch_pdl(rmsnorm_bwd_dw_reduce<T>, (C + 31) / 32, 256, 0, nullptr, dweight, partial, fb, C);
            return launch_ok();
        }
        if (vec)
            launch_pdl(rmsnorm_bwd_dinp_bf16x8, blocks, 256, 0, nullptr, reinterpret_cast<uint4*>(dinp), reinterpret_cast<const uint4*>(dout),
                                                     reinterpret_cast<const uint4*>(inp), reinterpret_cast<const uint4*>(weight),
                                                     rrms, rows, C);
    }
    if (!vec) launch_pdl(rmsnorm_bwd_dinp_kernel<T>, blocks, 256, 0, nullptr, dinp, dout, inp, weight, rrms, rows, C);
    launch_pdl(rmsnorm_bwd_dw_partial_kernel<T>, dim3((C + 255) / 256, chunks), 256, 0, nullptr, partial, dout, inp, rrms, rows, C, rows_per_chunk);
    launch_pdl(rmsnorm_bwd_dw_reduce<T>, (C + 31) / 32, 256, 0, nullptr, dweight, partial, chunks, C);
    return launch_ok();
}

template <typename T>
int residual_fwd(T* out, const T* a, const T* b, long long n) {
    if (!out || !a || !b || n <= 0) return B200_E_BADARG;
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
    const long long nvec = aligned ? n / VEC : 0;
    if (nvec > 0) {
        const long long blocks = (nvec + 255) / 256;
        launch_pdl(residual_forward_vec<T>, static_cast<unsigned>(blocks < 148 * 32 ? blocks : 148 * 32), 256, 0, nullptr, reinterpret_cast<uint4*>(out), reinterpret_cast<const uint4*>(a), reinterpret_cast<const uint4*>(b), nvec);
    }
    const long long done = nvec * VEC;
    if (done < n) launch_pdl(residual_forward_scalar<T>, static_cast<unsigned>((n - done + 255) / 256), 256, 0, nullptr, out, a, b, done, n);
    return launch_ok();
}

template <typename T>
int residual_bwd(T* da, T* db, const T* dout, long long n) {
    if (!da || !db || !dout || n <= 0) return B200_E_BADARG;
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = ((reinterpret_cast<uintptr_t>(da) | reinterpret_cast<uintptr_t>(db) | reinterpret_cast<uintptr_t>(dout)) & 15) == 0;
    const long long nvec = aligned ? n / VEC : 0;
    if (nvec > 0) {
        const long long blocks = (nvec + 255) / 256;
        launch_pdl(residual_backward_vec<T>, static_cast<unsigned>(blocks < 148 * 32 ? blocks : 148 * 32), 256, 0, nullptr, reinterpret_cast<uint4*>(da), reinterpret_cast<uint4*>(db), reinterpret_cast<const uint4*>(dout), nvec);
    }
    const long long done = nvec * VEC;
    if (done < n) launch_pdl(residual_backward_scalar<T>, static_cast<unsigned>((n - done + 255) / 256), 256, 0, nullptr, da, db, dout, done, n);
    return launch_ok();
}

// the reference's error convention for the void overloads (cuda/tensor.h:10-29)
void check(int rc, const char* what) {
    if (rc == B200_OK) return;
    fprintf(stderr, "b200_layers error %s: %s (cuda: %s)\n", what, b200_linear_strerror(rc), cudaGetErrorString(cudaGetLastError()));
    exit(EXIT_FAILURE);
}

}  // namespace

// ------------------------------------------------------------------------------------------ C entry points
extern "C" {

int b200_flash_attention_forward_bf16(void* context, float* lse, const void* q, const void* k, const void* v, int B, int T,
                                      int n_head, int n_kv_head, int head_dim, void* cuda_stream) {
    typedef __nv_bfloat16 bf;
    return flash_forward<bf>(static_cast<bf*>(context), lse, static_cast<const bf*>(q), static_cast<const bf*>(k),
                             static_cast<const bf*>(v), B, T, n_head, n_kv_head, head_dim, static_cast<cudaStream_t>(cuda_stream));
}
int b200_flash_attention_forward_f32(float* context, float* lse, const float* q, const float* k, const float* v, int B, int T,
                                     int n_head, int n_kv_head, int head_dim, void* cuda_stream) {
    return flash_forward<float>(context, lse, q, k, v, B, T, n_head, n_kv_head, head_dim, static_cast<cudaStream_t>(cuda_stream));
}
int b200_flash_attention_backward_bf16(void* dq, void* dk, void* dv, const void* dcontext, const void* q, const void* k,
                                       const void* v, const float* lse, const void* context, int B, int T, int n_head,
                                       int n_kv_head, int head_dim, void* cuda_stream) {
    typedef __nv_bfloat16 bf;
    return flash_backward<bf>(static_cast<bf*>(dq), static_cast<bf*>(dk), static_cast<bf*>(dv), static_cast<const bf*>(dcontext),
                              static_cast<const bf*>(q), static_cast<const bf*>(k), static_cast<const bf*>(v), lse,
                              static_cast<const bf*>(context), B, T, n_head, n_kv_head, head_dim,
                              static_cast<cudaStream_t>(cuda_stream));
}
int b200_flash_attention_backward_f32(float* dq, float* dk, float* dv, const float* dcontext, const float* q, const float* k,
                                      const float* v, const float* lse, const float* context, int B, int T, int n_head,
                                      int n_kv_head, int head_dim, void* cuda_stream) {
    return flash_backward<float>(dq, dk, dv, dcontext, q, k, v, lse, context, B, T, n_head, n_kv_head, head_dim,
                                 static_cast<cudaStream_t>(cuda_stream));
}
int b200_rope_bf16(void* q, void* k, int B, int T, int n_head, int n_kv_head, int head_dim, float theta, int backward,
                   void* cuda_stream) {
    typedef __nv_bfloat16 bf;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    return backward ? rope<bf, -1>(static_cast<bf*>(q), static_cast<bf*>(k), B, T, n_head, n_kv_head, head_dim, theta, s)
                    : rope<bf, +1>(static_cast<bf*>(q), static_cast<bf*>(k), B, T, n_head, n_kv_head, head_dim, theta, s);
}

int b200_attention_forward_bf16(b200_linear_ctx* ctx, void* out, void* q, void* k, void* v, void* att, const void* inp,
                                const void* wq, const void* wk, const void* wv, const void* wo, int B, int T, int C, int n_head,
                                int n_kv_head, float rope_theta) {
    typedef __nv_bfloat16 bf;
    return attention_fwd<bf>(ctx, static_cast<bf*>(out), static_cast<bf*>(q), static_cast<bf*>(k), static_cast<bf*>(v), att,
                             static_cast<const bf*>(inp), static_cast<const bf*>(wq), static_cast<const bf*>(wk),
                             static_cast<const bf*>(wv), static_cast<const bf*>(wo), B, T, C, n_head, n_kv_head, rope_theta);
}
int b200_attention_backward_bf16(b200_linear_ctx* ctx, void* dinp, void* dwq, void* dwk, void* dwv, void* dwo, const void* dout,
                                 const void* inp, const void* q, const void* k, const void* v, const void* att, const void* wq,
                                 const void* wk, const void* wv, const void* wo, int B, int T, int C, int n_head, int n_kv_head,
                                 float rope_theta) {
    typedef __nv_bfloat16 bf;
    return attention_bwd<bf>(ctx, static_cast<bf*>(dinp), static_cast<bf*>(dwq), static_cast<bf*>(dwk), static_cast<bf*>(dwv),
                             static_cast<bf*>(dwo), static_cast<const bf*>(dout), static_cast<const bf*>(inp),
                             static_cast<const bf*>(q), static_cast<const bf*>(k), static_cast<const bf*>(v), att,
                             static_cast<const bf*>(wq), static_cast<const bf*>(wk), static_cast<const bf*>(wv),
                             static_cast<const bf*>(wo), B, T, C, n_head, n_kv_head, rope_theta);
}
int b200_attention_forward_f32(b200_linear_ctx* ctx, float* out, float* q, float* k, float* v, float* att, const float* inp,
                               const float* wq, const float* wk, const float* wv, const float* wo, int B, int T, int C,
                               int n_head, int n_kv_head, float rope_theta) {
    return attention_fwd<float>(ctx, out, q, k, v, att, inp, wq, wk, wv, wo, B, T, C, n_head, n_kv_head, rope_theta);
}
int b200_attention_backward_f32(b200_linear_ctx* ctx, float* dinp, float* dwq, float* dwk, float* dwv, float* dwo,
                                const float* dout, const float* inp, const float* q, const float* k, const float* v,
                                const float* att, const float* wq, const float* wk, const float* wv, const float* wo, int B, int T,
                                int C, int n_head, int n_kv_head, float rope_theta) {
    return attention_bwd<float>(ctx, dinp, dwq, dwk, dwv, dwo, dout, inp, q, k, v, att, wq, wk, wv, wo, B, T, C, n_head,
                                n_kv_head, rope_theta);
}

int b200_swiglu_forward_bf16(b200_linear_ctx* ctx, void* out, void* gate, void* up, void* hidden, const void* inp,
                             const void* w_gate, const void* w_up, const void* w_down, int BT, int C, int ffn_hidden) {
    typedef __nv_bfloat16 bf;
    return swiglu_fwd<bf>(ctx, static_cast<bf*>(out), static_cast<bf*>(gate), static_cast<bf*>(up), static_cast<bf*>(hidden),
                          static_cast<const bf*>(inp), static_cast<const bf*>(w_gate), static_cast<const bf*>(w_up),
                          static_cast<const bf*>(w_down), BT, C, ffn_hidden);
}
int b200_swiglu_backward_bf16(b200_linear_ctx* ctx, void* dinp, void* dw_gate, void* dw_up, void* dw_down, const void* dout,
                              const void* inp, const void* gate, const void* up, const void* w_gate, const void* w_up,
                              const void* w_down, int BT, int C, int ffn_hidden) {
    typedef __nv_bfloat16 bf;
    return swiglu_bwd<bf>(ctx, static_cast<bf*>(dinp), static_cast<bf*>(dw_gate), static_cast<bf*>(dw_up), static_cast<bf*>(dw_down),
                          static_cast<const bf*>(dout), static_cast<const bf*>(inp), static_cast<const bf*>(gate),
                          static_cast<const bf*>(up), static_cast<const bf*>(w_gate), static_cast<const bf*>(w_up),
                          static_cast<const bf*>(w_down), BT, C, ffn_hidden);
}
int b200_swiglu_forward_f32(b200_linear_ctx* ctx, float* out, float* gate, float* up, float* hidden, const float* inp,
                            const float* w_gate, const float* w_up, const float* w_down, int BT, int C, int ffn_hidden) {
    return swiglu_fwd<float>(ctx, out, gate, up, hidden, inp, w_gate, w_up, w_down, BT, C, ffn_hidden);
}
int b200_swiglu_backward_f32(b200_linear_ctx* ctx, float* dinp, float* dw_gate, float* dw_up, float* dw_down, const float* dout,
                             const float* inp, const float* gate, const float* up, const float* w_gate, const float* w_up,
                             const float* w_down, int BT, int C, int ffn_hidden) {
    return swiglu_bwd<float>(ctx, dinp, dw_gate, dw_up, dw_down, dout, inp, gate, up, w_gate, w_up, w_down, BT, C, ffn_hidden);
}

int b200_crossentropy_forward_bf16(float* losses, void* logits_probs, const int* targets, int B, int T, int V) {
    return ce_forward<__nv_bfloat16>(losses, static_cast<__nv_bfloat16*>(logits_probs), targets, B, T, V);
}
int b200_crossentropy_forward_f32(float* losses, float* logits_probs, const int* targets, int B, int T, int V) {
    return ce_forward<float>(losses, logits_probs, targets, B, T, V);
}
int b200_crossentropy_backward_bf16(void* dlogits, const void* probs, const int* targets, int B, int T, int V, float loss_scale) {
    if (B <= 0 || T <= 0) return B200_E_BADARG;
    return ce_backward<__nv_bfloat16>(static_cast<__nv_bfloat16*>(dlogits), static_cast<const __nv_bfloat16*>(probs), targets, B, T,
                                      V, loss_scale / static_cast<float>(B * T));
}
int b200_crossentropy_backward_f32(float* dlogits, const float* probs, const int* targets, int B, int T, int V) {
    if (B <= 0 || T <= 0) return B200_E_BADARG;
    return ce_backward<float>(dlogits, probs, targets, B, T, V, 1.0f / static_cast<float>(B * T));
}

int b200_residual_forward_bf16(void* out, const void* a, const void* b, long long n) {
    typedef __nv_bfloat16 bf;
    return residual_fwd<bf>(static_cast<bf*>(out), static_cast<const bf*>(a), static_cast<const bf*>(b), n);
}
int b200_residual_forward_f32(float* out, const float* a, const float* b, long long n) { return residual_fwd<float>(out, a, b, n); }
int b200_residual_backward_bf16(void* da, void* db, const void* dout, long long n) {
    typedef __nv_bfloat16 bf;
    return residual_bwd<bf>(static_cast<bf*>(da), static_cast<bf*>(db), static_cast<const bf*>(dout), n);
}
int b200_residual_backward_f32(float* da, float* db, const float* dout, long long n) { return residual_bwd<float>(da, db, dout, n); }

int b200_rmsnorm_forward_bf16(void* out, float* rrms, const void* inp, const void* weight, float eps, int BT, int C) {
    typedef __nv_bfloat16 bf;
    return rmsnorm_fwd<bf>(static_cast<bf*>(out), rrms, static_cast<const bf*>(inp), static_cast<const bf*>(weight), eps, BT, C);
}
int b200_rmsnorm_forward_f32(float* out, float* rrms, const float* inp, const float* weight, float eps, int BT, int C) {
    return rmsnorm_fwd<float>(out, rrms, inp, weight, eps, BT, C);
}
int b200_rmsnorm_backward_bf16(void* dinp, void* dweight, const void* dout, const void* inp, const void* weight,
                               const float* rrms, int BT, int C) {
    typedef __nv_bfloat16 bf;
    return rmsnorm_bwd<bf>(static_cast<bf*>(dinp), static_cast<bf*>(dweight), static_cast<const bf*>(dout),
                           static_cast<const bf*>(inp), static_cast<const bf*>(weight), rrms, BT, C);
}
int b200_rmsnorm_backward_f32(float* dinp, float* dweight, const float* dout, const float* inp, const float* weight,
                              const float* rrms, int BT, int C) {
    return rmsnorm_bwd<float>(dinp, dweight, dout, inp, weight, rrms, BT, C);
}

// adamw_update / scale_grads / fp32_to_bf16 / compute_grad_norm_bf16, cuda/adamw.cu:42-58, 90-99, 153-191.
int b200_adamw_update_f32(float* params, const float* grads, float* m, float* v, float lr, float beta1, float beta2, float eps,
                          float weight_decay, int t, long long n) {
    if (!params || !grads || !m || !v || n <= 0 || t <= 0) return B200_E_BADARG;
    launch_pdl(adamw_kernel_f32, static_cast<unsigned>((n + 255) / 256), 256, 0, nullptr, params, grads, m, v, lr, beta1, beta2, eps, weight_decay,
                                                                      1.0f - powf(beta1, static_cast<float>(t)),
                                                                      1.0f - powf(beta2, static_cast<float>(t)), n);
    return launch_ok();
}
int b200_adamw_update_bf16(void* params, float* master, const void* grads, float* m, float* v, float lr, float beta1, float beta2,
                           float eps, float weight_decay, float grad_scale, int t, long long n) {
    if (!params || !master || !grads || !m || !v || n <= 0 || t <= 0) return B200_E_BADARG;
    launch_pdl(adamw_kernel_bf16, static_cast<unsigned>((n + 255) / 256), 256, 0, nullptr, static_cast<__nv_bfloat16*>(params), master, static_cast<const __nv_bfloat16*>(grads), m, v, lr, beta1, beta2, eps,
        weight_decay, grad_scale, 1.0f - powf(beta1, static_cast<float>(t)), 1.0f - powf(beta2, static_cast<float>(t)), n);
    return launch_ok();
}
int b200_scale_f32(float* data, float scale, long long n) {
    if (!data || n <= 0) return B200_E_BADARG;
    launch_pdl(scale_kernel_f32, static_cast<unsigned>((n + 255) / 256), 256, 0, nullptr, data, scale, n);
    return launch_ok();
}
int b200_f32_to_bf16(const float* src, void* dst, long long n) {
    if (!src || !dst || n <= 0) return B200_E_BADARG;
    launch_pdl(f32_to_bf16_kernel, static_cast<unsigned>((n + 255) / 256), 256, 0, nullptr, src, static_cast<__nv_bfloat16*>(dst), n);
    return launch_ok();
}
// *norm = sqrt(sum (g / loss_scale)^2) over the fp32 embedding gradient and the bf16 rest; non-finite bf16 entries
// are zeroed in place.  Synchronises (the result is a host value), like the reference's.
int b200_grad_norm_bf16(float* norm, const float* dwte_fp32, long long emb_n, void* grads_bf16, long long rest_n, float loss_scale) {
    if (!norm || !dwte_fp32 || !grads_bf16 || emb_n <= 0 || rest_n <= 0 || loss_scale == 0.f) return B200_E_BADARG;
    constexpr int kBlocks = 148 * 8;
    float* partial = static_cast<float*>(scratch(S_NORM_PARTIAL, (2 * kBlocks + 1) * sizeof(float)));
    if (!partial) return B200_E_CUDA;
    const float scale = 1.0f / loss_scale;
    launch_pdl(sumsq_partial_f32, kBlocks, 256, 0, nullptr, partial, dwte_fp32, scale, emb_n);
    launch_pdl(sumsq_sanitize_partial_bf16, kBlocks, 256, 0, nullptr, partial + kBlocks, static_cast<__nv_bfloat16*>(grads_bf16), scale, rest_n);
    launch_pdl(sum_partials, 1, 256, 0, nullptr, partial + 2 * kBlocks, partial, 2 * kBlocks);
    float h = 0.f;
    if (cudaMemcpy(&h, partial + 2 * kBlocks, sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) return B200_E_CUDA;
    *norm = sqrtf(h);
    return B200_OK;
}

}  // extern "C"

// ------------------------------------------------- the reference's C++ overloads (exact mangled names)
void adamw_update(float* params, const float* grads, float* m, float* v, float lr, float beta1, float beta2, float eps,
                  float weight_decay, int t, int N) {
    check(b200_adamw_update_f32(params, grads, m, v, lr, beta1, beta2, eps, weight_decay, t, N), "adamw_update(fp32)");
}
void adamw_update(__nv_bfloat16* params, float* master_params, const __nv_bfloat16* grads, float* m, float* v, float lr, float beta1,
                  float beta2, float eps, float weight_decay, float grad_scale, int t, int N) {
    check(b200_adamw_update_bf16(params, master_params, grads, m, v, lr, beta1, beta2, eps, weight_decay, grad_scale, t, N),
          "adamw_update(bf16)");
}
void scale_grads(float* data, float scale, int N) { check(b200_scale_f32(data, scale, N), "scale_grads"); }
void fp32_to_bf16(const float* src, __nv_bfloat16* dst, int N) { check(b200_f32_to_bf16(src, dst, N), "fp32_to_bf16"); }
float compute_grad_norm_bf16(float* dwte_fp32, int emb_N, __nv_bfloat16* grads_bf16, int rest_N, float loss_scale) {
    float norm = 0.f;
    check(b200_grad_norm_bf16(&norm, dwte_fp32, emb_N, grads_bf16, rest_N, loss_scale), "compute_grad_norm_bf16");
    return norm;
}

void residual_forward(float* out, const float* a, const float* b, int N) {
    check(b200_residual_forward_f32(out, a, b, N), "residual_forward(fp32)");
}
void residual_backward(float* da, float* db, const float* dout, int N) {
    check(b200_residual_backward_f32(da, db, dout, N), "residual_backward(fp32)");
}
void residual_forward(__nv_bfloat16* out, const __nv_bfloat16* a, const __nv_bfloat16* b, int N) {
    check(b200_residual_forward_bf16(out, a, b, N), "residual_forward(bf16)");
}
void residual_backward(__nv_bfloat16* da, __nv_bfloat16* db, const __nv_bfloat16* dout, int N) {
    check(b200_residual_backward_bf16(da, db, dout, N), "residual_backward(bf16)");
}
void rmsnorm_forward(float* out, float* rrms, const float* inp, const float* weight, float eps, int B_T, int C) {
    check(b200_rmsnorm_forward_f32(out, rrms, inp, weight, eps, B_T, C), "rmsnorm_forward(fp32)");
}
void rmsnorm_backward(float* dinp, float* dweight, const float* dout, const float* inp, const float* weight, const float* rrms,
                      int B_T, int C) {
    check(b200_rmsnorm_backward_f32(dinp, dweight, dout, inp, weight, rrms, B_T, C), "rmsnorm_backward(fp32)");
}
void rmsnorm_forward(__nv_bfloat16* out, float* rrms, const __nv_bfloat16* inp, const __nv_bfloat16* weight, float eps, int B_T,
                     int C) {
    check(b200_rmsnorm_forward_bf16(out, rrms, inp, weight, eps, B_T, C), "rmsnorm_forward(bf16)");
}
void rmsnorm_backward(__nv_bfloat16* dinp, __nv_bfloat16* dweight, const __nv_bfloat16* dout, const __nv_bfloat16* inp,
                      const __nv_bfloat16* weight, const float* rrms, int B_T, int C) {
    check(b200_rmsnorm_backward_bf16(dinp, dweight, dout, inp, weight, rrms, B_T, C), "rmsnorm_backward(bf16)");
}

void flash_attention_forward(float* context, float* lse, const float* q, const float* k, const float* v, int B, int T, int n_head,
                             int n_kv_head, int head_dim) {
    check(b200_flash_attention_forward_f32(context, lse, q, k, v, B, T, n_head, n_kv_head, head_dim, nullptr), "flash_attention_forward(fp32)");
}
void flash_attention_forward(__nv_bfloat16* context, float* lse, const __nv_bfloat16* q, const __nv_bfloat16* k,
                             const __nv_bfloat16* v, int B, int T, int n_head, int n_kv_head, int head_dim) {
    check(b200_flash_attention_forward_bf16(context, lse, q, k, v, B, T, n_head, n_kv_head, head_dim, nullptr), "flash_attention_forward(bf16)");
}
void flash_attention_backward(float* dq, float* dk, float* dv, const float* dcontext, const float* q, const float* k,
                              const float* v, const float* lse, int B, int T, int n_head, int n_kv_head, int head_dim) {
    check(b200_flash_attention_backward_f32(dq, dk, dv, dcontext, q, k, v, lse, nullptr, B, T, n_head, n_kv_head, head_dim, nullptr),
          "flash_attention_backward(fp32)");
}
void flash_attention_backward(__nv_bfloat16* dq, __nv_bfloat16* dk, __nv_bfloat16* dv, const __nv_bfloat16* dcontext,
                              const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, const float* lse, int B,
                              int T, int n_head, int n_kv_head, int head_dim) {
    check(b200_flash_attention_backward_bf16(dq, dk, dv, dcontext, q, k, v, lse, nullptr, B, T, n_head, n_kv_head, head_dim, nullptr),
          "flash_attention_backward(bf16)");
}

void attention_forward(float* out, float* q, float* k, float* v, float* att_or_lse, const float* inp, const float* wq,
                       const float* wk, const float* wv, const float* wo, int B, int T, int C, int n_head, int n_kv_head,
                       float rope_theta, cublasHandle_t) {
    check(b200_attention_forward_f32(b200_linear_default_ctx(), out, q, k, v, att_or_lse, inp, wq, wk, wv, wo, B, T, C, n_head,
                                     n_kv_head, rope_theta), "attention_forward(fp32)");
}
void attention_backward(float* dinp, float* dwq, float* dwk, float* dwv, float* dwo, const float* dout, const float* inp,
                        const float* q, const float* k, const float* v, const float* att_or_lse, const float* wq, const float* wk,
                        const float* wv, const float* wo, int B, int T, int C, int n_head, int n_kv_head, float rope_theta,
                        cublasHandle_t) {
    check(b200_attention_backward_f32(b200_linear_default_ctx(), dinp, dwq, dwk, dwv, dwo, dout, inp, q, k, v, att_or_lse, wq, wk,
                                      wv, wo, B, T, C, n_head, n_kv_head, rope_theta), "attention_backward(fp32)");
}
void attention_forward(__nv_bfloat16* out, __nv_bfloat16* q, __nv_bfloat16* k, __nv_bfloat16* v, __nv_bfloat16* att,
                       const __nv_bfloat16* inp, const __nv_bfloat16* wq, const __nv_bfloat16* wk, const __nv_bfloat16* wv,
                       const __nv_bfloat16* wo, int B, int T, int C, int n_head, int n_kv_head, float rope_theta, cublasHandle_t) {
    check(b200_attention_forward_bf16(b200_linear_default_ctx(), out, q, k, v, att, inp, wq, wk, wv, wo, B, T, C, n_head, n_kv_head,
                                      rope_theta), "attention_forward(bf16)");
}
void attention_backward(__nv_bfloat16* dinp, __nv_bfloat16* dwq, __nv_bfloat16* dwk, __nv_bfloat16* dwv, __nv_bfloat16* dwo,
                        const __nv_bfloat16* dout, const __nv_bfloat16* inp, const __nv_bfloat16* q, const __nv_bfloat16* k,
                        const __nv_bfloat16* v, const __nv_bfloat16* att, const __nv_bfloat16* wq, const __nv_bfloat16* wk,
                        const __nv_bfloat16* wv, const __nv_bfloat16* wo, int B, int T, int C, int n_head, int n_kv_head,
                        float rope_theta, cublasHandle_t) {
    check(b200_attention_backward_bf16(b200_linear_default_ctx(), dinp, dwq, dwk, dwv, dwo, dout, inp, q, k, v, att, wq, wk, wv, wo,
                                       B, T, C, n_head, n_kv_head, rope_theta), "attention_backward(bf16)");
}

void swiglu_forward(float* out, float* gate, float* up, float* hidden, const float* inp, const float* w_gate, const float* w_up,
                    const float* w_down, int B_T, int C, int ffn_hidden, cublasHandle_t) {
    check(b200_swiglu_forward_f32(b200_linear_default_ctx(), out, gate, up, hidden, inp, w_gate, w_up, w_down, B_T, C, ffn_hidden),
          "swiglu_forward(fp32)");
}
void swiglu_backward(float* dinp, float* dw_gate, float* dw_up, float* dw_down, const float* dout, const float* inp,
                     const float* gate, const float* up, const float* w_gate, const float* w_up, const float* w_down, int B_T,
                     int C, int ffn_hidden, cublasHandle_t) {
    check(b200_swiglu_backward_f32(b200_linear_default_ctx(), dinp, dw_gate, dw_up, dw_down, dout, inp, gate, up, w_gate, w_up,
                                   w_down, B_T, C, ffn_hidden), "swiglu_backward(fp32)");
}
void swiglu_forward(__nv_bfloat16* out, __nv_bfloat16* gate, __nv_bfloat16* up, __nv_bfloat16* hidden, const __nv_bfloat16* inp,
                    const __nv_bfloat16* w_gate, const __nv_bfloat16* w_up, const __nv_bfloat16* w_down, int B_T, int C,
                    int ffn_hidden, cublasHandle_t) {
    check(b200_swiglu_forward_bf16(b200_linear_default_ctx(), out, gate, up, hidden, inp, w_gate, w_up, w_down, B_T, C, ffn_hidden),
          "swiglu_forward(bf16)");
}
void swiglu_backward(__nv_bfloat16* dinp, __nv_bfloat16* dw_gate, __nv_bfloat16* dw_up, __nv_bfloat16* dw_down,
                     const __nv_bfloat16* dout, const __nv_bfloat16* inp, const __nv_bfloat16* gate, const __nv_bfloat16* up,
                     const __nv_bfloat16* w_gate, const __nv_bfloat16* w_up, const __nv_bfloat16* w_down, int B_T, int C,
                     int ffn_hidden, cublasHandle_t) {
    check(b200_swiglu_backward_bf16(b200_linear_default_ctx(), dinp, dw_gate, dw_up, dw_down, dout, inp, gate, up, w_gate, w_up,
                                    w_down, B_T, C, ffn_hidden), "swiglu_backward(bf16)");
}

void crossentropy_forward(float* losses, const float* logits, const int* targets, int B, int T, int V) {
    check(b200_crossentropy_forward_f32(losses, const_cast<float*>(logits), targets, B, T, V), "crossentropy_forward(fp32)");
}
void crossentropy_softmax_backward(float* dlogits, const float* probs, const int* targets, int B, int T, int V) {
    check(b200_crossentropy_backward_f32(dlogits, probs, targets, B, T, V), "crossentropy_softmax_backward(fp32)");
}
void crossentropy_forward(float* losses, const __nv_bfloat16* logits, const int* targets, int B, int T, int V) {
    check(b200_crossentropy_forward_bf16(losses, const_cast<__nv_bfloat16*>(logits), targets, B, T, V), "crossentropy_forward(bf16)");
}
void crossentropy_softmax_backward(__nv_bfloat16* dlogits, const __nv_bfloat16* probs, const int* targets, int B, int T, int V,
                                   float loss_scale) {
    check(b200_crossentropy_backward_bf16(dlogits, probs, targets, B, T, V, loss_scale), "crossentropy_softmax_backward(bf16)");
}
