// TEST INFRASTRUCTURE — not part of the product.
//
// extern "C" doorway onto the reference's own, unmodified cuda/matmul.cu (cuBLAS), cuda/crossentropy.cu,
// cuda/attention.cu, cuda/swiglu.cu and cuda/rope.cu, so that Python tests and bench.py can call them through
// ctypes.  oracle/build.py compiles this file together with those sources, taken from where the
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

// cuda/attention.cu, cuda/swiglu.cu, cuda/rope.cu (with cuda/softmax.cu and cuda/residual.cu, which they call):
// the reference's own layer code on the reference's own cuBLAS GEMMs, as the checker of the library's layer drop-ins.
void ref_attention_forward_bf16(void* h, void* out, void* q, void* k, void* v, void* att, const void* inp, const void* wq,
                                const void* wk, const void* wv, const void* wo, int B, int T, int C, int n_head, int n_kv_head,
                                float rope_theta) {
    typedef __nv_bfloat16 bf;
    attention_forward((bf*)out, (bf*)q, (bf*)k, (bf*)v, (bf*)att, (const bf*)inp, (const bf*)wq, (const bf*)wk, (const bf*)wv,
                      (const bf*)wo, B, T, C, n_head, n_kv_head, rope_theta, (cublasHandle_t)h);
}
void ref_attention_backward_bf16(void* h, void* dinp, void* dwq, void* dwk, void* dwv, void* dwo, const void* dout,
                                 const void* inp, const void* q, const void* k, const void* v, const void* att, const void* wq,
                                 const void* wk, const void* wv, const void* wo, int B, int T, int C, int n_head, int n_kv_head,
                                 float rope_theta) {
    typedef __nv_bfloat16 bf;
    attention_backward((bf*)dinp, (bf*)dwq, (bf*)dwk, (bf*)dwv, (bf*)dwo, (const bf*)dout, (const bf*)inp, (const bf*)q,
                       (const bf*)k, (const bf*)v, (const bf*)att, (const bf*)wq, (const bf*)wk, (const bf*)wv, (const bf*)wo, B, T,
                       C, n_head, n_kv_head, rope_theta, (cublasHandle_t)h);
}
void ref_attention_forward_f32(void* h, float* out, float* q, float* k, float* v, float* att, const float* inp, const float* wq,
                               const float* wk, const float* wv, const float* wo, int B, int T, int C, int n_head, int n_kv_head,
                               float rope_theta) {
    attention_forward(out, q, k, v, att, inp, wq, wk, wv, wo, B, T, C, n_head, n_kv_head, rope_theta, (cublasHandle_t)h);
}
void ref_attention_backward_f32(void* h, float* dinp, float* dwq, float* dwk, float* dwv, float* dwo, const float* dout,
                                const float* inp, const float* q, const float* k, const float* v, const float* att,
                                const float* wq, const float* wk, const float* wv, const float* wo, int B, int T, int C,
                                int n_head, int n_kv_head, float rope_theta) {
    attention_backward(dinp, dwq, dwk, dwv, dwo, dout, inp, q, k, v, att, wq, wk, wv, wo, B, T, C, n_head, n_kv_head, rope_theta,
                       (cublasHandle_t)h);
}
void ref_swiglu_forward_bf16(void* h, void* out, void* gate, void* up, void* hidden, const void* inp, const void* w_gate,
                             const void* w_up, const void* w_down, int BT, int C, int ff) {
    typedef __nv_bfloat16 bf;
    swiglu_forward((bf*)out, (bf*)gate, (bf*)up, (bf*)hidden, (const bf*)inp, (const bf*)w_gate, (const bf*)w_up, (const bf*)w_down,
                   BT, C, ff, (cublasHandle_t)h);
}
void ref_swiglu_backward_bf16(void* h, void* dinp, void* dw_gate, void* dw_up, void* dw_down, const void* dout, const void* inp,
                              const void* gate, const void* up, const void* w_gate, const void* w_up, const void* w_down, int BT,
                              int C, int ff) {
    typedef __nv_bfloat16 bf;
    swiglu_backward((bf*)dinp, (bf*)dw_gate, (bf*)dw_up, (bf*)dw_down, (const bf*)dout, (const bf*)inp, (const bf*)gate,
                    (const bf*)up, (const bf*)w_gate, (const bf*)w_up, (const bf*)w_down, BT, C, ff, (cublasHandle_t)h);
}
void ref_rope_forward_bf16(void* q, void* k, int B, int T, int n_head, int n_kv_head, int head_dim, float theta) {
    rope_forward((__nv_bfloat16*)q, (__nv_bfloat16*)k, B, T, n_head, n_kv_head, head_dim, theta);
}

// cuda/adamw.cu: the optimizer step and the global gradient norm, as the reference's main.cpp calls them
void ref_adamw_update_bf16(void* params, float* master, const void* grads, float* m, float* v, float lr, float beta1, float beta2,
                           float eps, float weight_decay, float grad_scale, int t, int N) {
    adamw_update((__nv_bfloat16*)params, master, (const __nv_bfloat16*)grads, m, v, lr, beta1, beta2, eps, weight_decay, grad_scale, t, N);
}
void ref_adamw_update_f32(float* params, const float* grads, float* m, float* v, float lr, float beta1, float beta2, float eps,
                          float weight_decay, int t, int N) {
    adamw_update(params, grads, m, v, lr, beta1, beta2, eps, weight_decay, t, N);
}
float ref_grad_norm_bf16(float* dwte, int emb_N, void* grads, int rest_N, float loss_scale) {
    return compute_grad_norm_bf16(dwte, emb_N, (__nv_bfloat16*)grads, rest_N, loss_scale);
}

}  // extern "C"
