// The four C++ overloads that the reference's host code links against, with exactly the
// signatures (and therefore the Itanium-mangled names) of the reference's cuda/kernels.cuh:
//   cuda/kernels.cuh:47-52   void matmul_forward (cublasHandle_t, float*, const float*, const float*, int,int,int)
//   cuda/kernels.cuh:56-65   void matmul_backward(cublasHandle_t, float*, float*, const float*, const float*, const float*, int,int,int)
//   cuda/kernels.cuh:348     void matmul_forward (cublasHandle_t, __nv_bfloat16*, const __nv_bfloat16*, const __nv_bfloat16*, int,int,int)
//   cuda/kernels.cuh:350     void matmul_backward(cublasHandle_t, __nv_bfloat16*, __nv_bfloat16*, const __nv_bfloat16*, ...)
// Linking this library in place of the object built from the reference's cuda/matmul.cu swaps
// the GEMM leaf under attention_forward/backward, swiglu_forward/backward and the LM head
// without touching any caller.
//
// The cublasHandle_t argument is accepted and ignored: cuBLAS' handle type is opaque, so the
// library keeps its own context per device, created on first use.  Work is enqueued on the
// legacy default stream, which is where the reference's callers expect it (they cudaFree
// operands right after these calls return).  Errors follow the reference's convention
// (cuda/tensor.h:10-29): a message on stderr, then exit(EXIT_FAILURE).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "../../include/b200_linear.h"

struct cublasContext;
typedef struct cublasContext* cublasHandle_t;

namespace {

constexpr int kMaxDevices = 64;
b200_linear_ctx* g_ctx[kMaxDevices] = {};

b200_linear_ctx* device_ctx() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        fprintf(stderr, "b200_linear error %s:%d: no current CUDA device\n", __FILE__, __LINE__);
        exit(EXIT_FAILURE);
    }
    if (!g_ctx[dev]) {
        int rc = b200_linear_create(&g_ctx[dev]);
        if (rc != B200_OK) {
            fprintf(stderr, "b200_linear error %s:%d: context creation failed: %s\n", __FILE__, __LINE__,
                    b200_linear_strerror(rc));
            exit(EXIT_FAILURE);
        }
    }
    return g_ctx[dev];
}

void check(int rc, b200_linear_ctx* ctx, const char* what, int line) {
    if (rc == B200_OK) return;
    fprintf(stderr, "b200_linear error %s:%d: %s: %s (cuda %d)\n", __FILE__, line, what, b200_linear_strerror(rc),
            b200_linear_last_cuda_error(ctx));
    exit(EXIT_FAILURE);
}

}  // namespace

void matmul_forward(cublasHandle_t, float* C, const float* A, const float* B, int M, int N, int K) {
    b200_linear_ctx* ctx = device_ctx();
    check(b200_linear_forward_f32(ctx, C, A, B, M, N, K), ctx, "matmul_forward(fp32)", __LINE__);
}

void matmul_backward(cublasHandle_t, float* dA, float* dB, const float* dC, const float* A, const float* B,
                     int M, int N, int K) {
    b200_linear_ctx* ctx = device_ctx();
    check(b200_linear_backward_f32(ctx, dA, dB, dC, A, B, M, N, K), ctx, "matmul_backward(fp32)", __LINE__);
}

void matmul_forward(cublasHandle_t, __nv_bfloat16* C, const __nv_bfloat16* A, const __nv_bfloat16* B, int M,
                    int N, int K) {
    b200_linear_ctx* ctx = device_ctx();
    check(b200_linear_forward_bf16(ctx, C, A, B, M, N, K), ctx, "matmul_forward(bf16)", __LINE__);
}

void matmul_backward(cublasHandle_t, __nv_bfloat16* dA, __nv_bfloat16* dB, const __nv_bfloat16* dC,
                     const __nv_bfloat16* A, const __nv_bfloat16* B, int M, int N, int K) {
    b200_linear_ctx* ctx = device_ctx();
    check(b200_linear_backward_bf16(ctx, dA, dB, dC, A, B, M, N, K), ctx, "matmul_backward(bf16)", __LINE__);
}
