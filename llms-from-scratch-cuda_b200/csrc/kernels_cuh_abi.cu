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

void poll_all_at_exit();

b200_linear_ctx* device_ctx() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        fprintf(stderr, "b200_linear error %s:%d: no current CUDA device\n", __FILE__, __LINE__);
        exit(EXIT_FAILURE);
    }
    if (!g_ctx[dev]) {
        static bool registered = false;
        if (!registered) {
            registered = true;
            atexit(poll_all_at_exit);
        }
        int rc = b200_linear_create(&g_ctx[dev]);
        if (rc != B200_OK) {
            fprintf(stderr, "b200_linear error %s:%d: context creation failed: %s\n", __FILE__, __LINE__,
                    b200_linear_strerror(rc));
            exit(EXIT_FAILURE);
        }
    }
    return g_ctx[dev];
}

void fail(int rc, b200_linear_ctx* ctx, const char* what, int line) {
    fprintf(stderr, "b200_linear error %s:%d: %s: %s (cuda %d)\n", __FILE__, line, what, b200_linear_strerror(rc),
            b200_linear_last_cuda_error(ctx));
    exit(EXIT_FAILURE);
}

// A kernel whose bounded wait ran out has left its output partly written; the void signatures of the
// reference have no way to say so.  Every kPollEvery-th call therefore reads the context's device status
// word (a stream synchronisation and a 4-byte copy; the reference's callers synchronise the device several
// times per layer themselves, with their cudaFree of temporaries) and ends the program the way the
// reference ends on any CUDA error.  A process that exits normally is checked once more on the way out.
constexpr long long kPollEvery = 1024;
long long g_calls = 0;

void poll_status(b200_linear_ctx* ctx, const char* what, int line) {
    int code = 0;
    const int rc = b200_linear_sync(ctx, &code);
    if (rc == B200_OK) return;
    fprintf(stderr, "b200_linear: device code %d\n", code);
    fail(rc, ctx, what, line);
}

void poll_all_at_exit() {
    int current = 0;
    if (cudaGetDevice(&current) != cudaSuccess) return;
    for (int dev = 0; dev < kMaxDevices; ++dev) {
        if (!g_ctx[dev]) continue;
        if (cudaSetDevice(dev) != cudaSuccess) continue;
        int code = 0;
        if (b200_linear_sync(g_ctx[dev], &code) == B200_E_DEVICE_WAIT)
            fprintf(stderr, "b200_linear: a kernel on device %d gave up on a bounded wait (device code %d): "
                            "results of this run are not to be trusted\n", dev, code);
    }
    cudaSetDevice(current);
}

}  // namespace

extern "C" b200_linear_ctx* b200_linear_default_ctx(void) { return device_ctx(); }

namespace {

void check(int rc, b200_linear_ctx* ctx, const char* what, int line) {
    if (rc != B200_OK) fail(rc, ctx, what, line);
    if (++g_calls % kPollEvery == 0) poll_status(ctx, what, line);
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
