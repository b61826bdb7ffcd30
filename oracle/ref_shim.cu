// TEST INFRASTRUCTURE — not part of the product.
//
// extern "C" doorway onto the reference's own, unmodified cuda/matmul.cu (cuBLAS) and
// cuda/crossentropy.cu, so that Python tests and bench.py can call them through ctypes.
// oracle/build.py compiles this file together with those two sources, taken from where the
// reference checkout lies, into oracle/_ref/libref_matmul.so.  Nothing of the reference is copied into this
// repository: its header is only included at build time.
#include "kernels.cuh"  // the reference's cuda/kernels.cuh (via -I at build time)

extern "C" {

int ref_create(void** handle) {
    cublasHandle_t h = nullptr;
    if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) return 1;
    // llama2-mistral/src/model.cpp:405 of the reference: the bf16 model enables tensor-op math.
    cublasSetMathMode(h, CUBLAS_TENSOR_OP_MATH);
    *handle = h;
    return 0;
}
int ref_create_fp32(void** handle) {  // llama2-mistral/src/model.cpp:11: default math mode
    cublasHandle_t h = nullptr;
    if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) return 1;
    *handle = h;
    return 0;
}
int ref_destroy(void* handle) { return cublasDestroy((cublasHandle_t)handle) != CUBLAS_STATUS_SUCCESS; }
int ref_set_stream(void* handle, void* stream) {
    return cublasSetStream((cublasHandle_t)handle, (cudaStream_t)stream) != CUBLAS_STATUS_SUCCESS;
}

void ref_matmul_forward_bf16(void* h, void* C, const void* A, const void* B, int M, int N, int K) {
    matmul_forward((cublasHandle_t)h, (__nv_bfloat16*)C, (const __nv_bfloat16*)A, (const __nv_bfloat16*)B, M, N, K);
}
void ref_matmul_backward_bf16(void* h, void* dA, void* dB, const void* dC, const void* A, const void* B, int M,
                              int N, int K) {
    matmul_backward((cublasHandle_t)h, (__nv_bfloat16*)dA, (__nv_bfloat16*)dB, (const __nv_bfloat16*)dC,
                    (const __nv_bfloat16*)A, (const __nv_bfloat16*)B, M, N, K);
}
void ref_matmul_forward_f32(void* h, float* C, const float* A, const float* B, int M, int N, int K) {
    matmul_forward((cublasHandle_t)h, C, A, B, M, N, K);
}
void ref_matmul_backward_f32(void* h, float* dA, float* dB, const float* dC, const float* A, const float* B,
                             int M, int N, int K) {
    matmul_backward((cublasHandle_t)h, dA, dB, dC, A, B, M, N, K);
}

// cuda/crossentropy.cu, bf16 overloads (declared cuda/kernels.cuh:402-403): probabilities are written in place
// of the logits; the backward reads them and writes dlogits (the reference passes the same buffer for both).
void ref_crossentropy_forward_bf16(float* losses, const void* logits, const int* targets, int B, int T, int V) {
    crossentropy_forward(losses, (const __nv_bfloat16*)logits, targets, B, T, V);
}
void ref_crossentropy_backward_bf16(void* dlogits, const void* probs, const int* targets, int B, int T, int V,
                                    float loss_scale) {
    crossentropy_softmax_backward((__nv_bfloat16*)dlogits, (const __nv_bfloat16*)probs, targets, B, T, V, loss_scale);
}

}  // extern "C"
