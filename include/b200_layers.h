/* C ABI of the layer-level entry points of libb200_linear.so: the callers of the linear-layer GEMMs in
 * chriskuchar/llms-from-scratch-cuda, each with the argument list of the reference function it replaces
 * (cuda/kernels.cuh) plus, where the reference passes a cublasHandle_t, a b200_linear_ctx.  The same library
 * also exports the reference's C++ overloads themselves (same mangled names), so that its host code links
 * unchanged with cuda/attention.cu, cuda/flash_attention.cu, cuda/swiglu.cu, cuda/crossentropy.cu, cuda/rmsnorm.cu,
 * cuda/residual.cu and cuda/adamw.cu left out.
 *
 * Layouts are the reference's: activations [B*T, C] row-major, weights [in, out], q / context [B*T, n_head*hd],
 * k / v [B*T, n_kv_head*hd] with query head h reading KV head h / (n_head / n_kv_head); lse [B, n_head, T] fp32.
 * Head dimension 64 only (both model families); anything else returns B200_E_BADARG.  All calls are
 * asynchronous; functions with a `cuda_stream` argument run there (NULL = legacy default stream), the
 * others on the legacy default stream, which is where the reference's callers expect them.
 * Return values are the B200_* codes of b200_linear.h.  Temporaries live in a per-device scratch that grows on
 * demand (cudaMalloc on first use of a larger shape, never per call). */
#ifndef B200_LAYERS_H
#define B200_LAYERS_H

#include "b200_linear.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Fused causal grouped-query attention core: context = softmax(q k^T / sqrt(hd), causal) v, lse = row
 * log-sum-exp of the scaled scores; no [B, n_head, T, T] matrix exists at any time.  q and k already carry
 * the rotary embedding.  Fills the signatures the reference declares and leaves empty:
 * flash_attention_forward, cuda/flash_attention.cu:12-49, cuda/kernels.cuh:316-326 (fp32), :420-427 (bf16). */
int b200_flash_attention_forward_bf16(void* context, float* lse, const void* q, const void* k, const void* v, int B,
                                      int T, int n_head, int n_kv_head, int head_dim, void* cuda_stream);
int b200_flash_attention_forward_f32(float* context, float* lse, const float* q, const float* k, const float* v, int B,
                                     int T, int n_head, int n_kv_head, int head_dim, void* cuda_stream);
/* flash_attention_backward, cuda/flash_attention.cu:51-98, cuda/kernels.cuh:328-341, :428-437.  dk and dv are
 * overwritten (the reference's contract asks the caller to zero them for its atomics; zeroing is harmless).
 * `context` is the forward output; NULL (the reference's argument list has none) makes the call recompute it.
 * No atomics: results are the same from run to run. */
int b200_flash_attention_backward_bf16(void* dq, void* dk, void* dv, const void* dcontext, const void* q, const void* k,
                                       const void* v, const float* lse, const void* context, int B, int T, int n_head,
                                       int n_kv_head, int head_dim, void* cuda_stream);
int b200_flash_attention_backward_f32(float* dq, float* dk, float* dv, const float* dcontext, const float* q,
                                      const float* k, const float* v, const float* lse, const float* context, int B, int T,
                                      int n_head, int n_kv_head, int head_dim, void* cuda_stream);
/* rope_forward / rope_backward (backward != 0), cuda/rope.cu:95-109, in place on q [B*T, n_head*hd] and k. */
int b200_rope_bf16(void* q, void* k, int B, int T, int n_head, int n_kv_head, int head_dim, float theta, int backward,
                   void* cuda_stream);

/* attention_forward, cuda/attention.cu:582-618 (bf16), :235-292 (fp32): q, k, v projections, rotary embedding,
 * attention core, output projection.  `att` is the reference's [B, n_head, T, T] score buffer; here it receives
 * the row log-sum-exps and the attention context (what the backward pass needs) and nothing else of it is touched. */
int b200_attention_forward_bf16(b200_linear_ctx* ctx, void* out, void* q, void* k, void* v, void* att, const void* inp,
                                const void* wq, const void* wk, const void* wv, const void* wo, int B, int T, int C,
                                int n_head, int n_kv_head, float rope_theta);
int b200_attention_forward_f32(b200_linear_ctx* ctx, float* out, float* q, float* k, float* v, float* att, const float* inp,
                               const float* wq, const float* wk, const float* wv, const float* wo, int B, int T, int C,
                               int n_head, int n_kv_head, float rope_theta);
/* attention_backward, cuda/attention.cu:621-700 (bf16), :294-414 (fp32).  `att` must be the buffer the matching
 * attention_forward call wrote.  dinp is overwritten; dwq, dwk, dwv, dwo accumulate (beta = 1). */
int b200_attention_backward_bf16(b200_linear_ctx* ctx, void* dinp, void* dwq, void* dwk, void* dwv, void* dwo,
                                 const void* dout, const void* inp, const void* q, const void* k, const void* v,
                                 const void* att, const void* wq, const void* wk, const void* wv, const void* wo, int B, int T,
                                 int C, int n_head, int n_kv_head, float rope_theta);
int b200_attention_backward_f32(b200_linear_ctx* ctx, float* dinp, float* dwq, float* dwk, float* dwv, float* dwo,
                                const float* dout, const float* inp, const float* q, const float* k, const float* v,
                                const float* att, const float* wq, const float* wk, const float* wv, const float* wo, int B,
                                int T, int C, int n_head, int n_kv_head, float rope_theta);

/* swiglu_forward, cuda/swiglu.cu:157-170 (bf16), :49-70 (fp32): out = (SiLU(inp w_gate) * (inp w_up)) w_down;
 * gate, up and hidden are written as the reference writes them. */
int b200_swiglu_forward_bf16(b200_linear_ctx* ctx, void* out, void* gate, void* up, void* hidden, const void* inp,
                             const void* w_gate, const void* w_up, const void* w_down, int BT, int C, int ffn_hidden);
int b200_swiglu_forward_f32(b200_linear_ctx* ctx, float* out, float* gate, float* up, float* hidden, const float* inp,
                            const float* w_gate, const float* w_up, const float* w_down, int BT, int C, int ffn_hidden);
/* swiglu_backward, cuda/swiglu.cu:172-216 (bf16), :72-130 (fp32).  dinp overwritten; the three dW accumulate. */
int b200_swiglu_backward_bf16(b200_linear_ctx* ctx, void* dinp, void* dw_gate, void* dw_up, void* dw_down, const void* dout,
                              const void* inp, const void* gate, const void* up, const void* w_gate, const void* w_up,
                              const void* w_down, int BT, int C, int ffn_hidden);
int b200_swiglu_backward_f32(b200_linear_ctx* ctx, float* dinp, float* dw_gate, float* dw_up, float* dw_down,
                             const float* dout, const float* inp, const float* gate, const float* up, const float* w_gate,
                             const float* w_up, const float* w_down, int BT, int C, int ffn_hidden);

/* crossentropy_forward, cuda/crossentropy.cu:134-140 (bf16), :66-76 (fp32): per-row loss; the probabilities
 * replace the logits in place, with the reference's rounding points (the exponential is stored in the storage
 * type, then divided by the sum of the unrounded exponentials, then stored again).  One CTA per row instead
 * of one thread per row. */
int b200_crossentropy_forward_bf16(float* losses, void* logits_probs, const int* targets, int B, int T, int V);
int b200_crossentropy_forward_f32(float* losses, float* logits_probs, const int* targets, int B, int T, int V);
/* crossentropy_softmax_backward, cuda/crossentropy.cu:142-151 (bf16: scale = loss_scale / (B*T)), :78-92 (fp32). */
int b200_crossentropy_backward_bf16(void* dlogits, const void* probs, const int* targets, int B, int T, int V,
                                    float loss_scale);
int b200_crossentropy_backward_f32(float* dlogits, const float* probs, const int* targets, int B, int T, int V);

/* rmsnorm_forward, cuda/rmsnorm.cu:75-85 (fp32), :168-172 (bf16): out = inp * rsqrt(mean(inp^2) + eps) * weight per row,
 * rrms [BT] = the rsqrt, kept for the backward pass. */
int b200_rmsnorm_forward_bf16(void* out, float* rrms, const void* inp, const void* weight, float eps, int BT, int C);
int b200_rmsnorm_forward_f32(float* out, float* rrms, const float* inp, const float* weight, float eps, int BT, int C);
/* rmsnorm_backward, cuda/rmsnorm.cu:88-105 (fp32), :174-178 (bf16): dinp overwritten, dweight accumulated.  The
 * reference adds to dweight with one atomic per element and row (on bf16: a compare-and-swap loop with a rounding
 * per addition); here the rows are summed in fp32 in a fixed order and added to the stored gradient once. */
int b200_rmsnorm_backward_bf16(void* dinp, void* dweight, const void* dout, const void* inp, const void* weight,
                               const float* rrms, int BT, int C);
int b200_rmsnorm_backward_f32(float* dinp, float* dweight, const float* dout, const float* inp, const float* weight,
                              const float* rrms, int BT, int C);

/* residual_forward (out = a + b, out may be a) and residual_backward (da += dout, db += dout),
 * cuda/residual.cu:32-49 (fp32), :68-78 (bf16); n elements. */
int b200_residual_forward_bf16(void* out, const void* a, const void* b, long long n);
int b200_residual_forward_f32(float* out, const float* a, const float* b, long long n);
int b200_residual_backward_bf16(void* da, void* db, const void* dout, long long n);
int b200_residual_backward_f32(float* da, float* db, const float* dout, long long n);

/* adamw_update (cuda/adamw.cu:42-58 fp32; :90-99 mixed precision: bf16 weights and gradients, fp32 master weights and
 * moments), scale_grads (:153-157), fp32_to_bf16 (:165-169): the reference's arithmetic, one element per thread. */
int b200_adamw_update_f32(float* params, const float* grads, float* m, float* v, float lr, float beta1, float beta2, float eps,
                          float weight_decay, int t, long long n);
int b200_adamw_update_bf16(void* params, float* master, const void* grads, float* m, float* v, float lr, float beta1,
                           float beta2, float eps, float weight_decay, float grad_scale, int t, long long n);
int b200_scale_f32(float* data, float scale, long long n);
int b200_f32_to_bf16(const float* src, void* dst, long long n);
/* compute_grad_norm_bf16, cuda/adamw.cu:171-191: *norm = the global L2 norm of (gradient / loss_scale) over the fp32
 * embedding gradient and the bf16 rest, whose non-finite or > 65000 entries are zeroed in place.  Two-stage sum in a
 * fixed order instead of one atomic per 256 elements; synchronises, like the reference's (the result is a host value). */
int b200_grad_norm_bf16(float* norm, const float* dwte_fp32, long long emb_n, void* grads_bf16, long long rest_n,
                        float loss_scale);

#ifdef __cplusplus
}
#endif
#endif /* B200_LAYERS_H */
