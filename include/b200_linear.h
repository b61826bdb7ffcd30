/* C ABI of libb200_linear.so: the linear-layer GEMMs of chriskuchar/llms-from-scratch-cuda
 * (its cuda/matmul.cu) as hand-written sm_100a kernels.
 *
 * All matrices are dense row-major with the inner extent as leading dimension, exactly as
 * the reference passes them (cuda/kernels.cuh:46-65):
 *     A [M,K]   left input / saved activation
 *     B [K,N]   weight, stored [in, out]
 *     C [M,N]   output;  dC [M,N] upstream gradient;  dA [M,K];  dB [K,N]
 * Every pointer is a device pointer on the context's device.  Calls are asynchronous on the
 * context's stream (default: the legacy default stream, which is what the reference uses).
 * Every function returns 0 on success or a B200_E_* code; nothing here calls exit().
 */
#ifndef B200_LINEAR_H
#define B200_LINEAR_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_linear_ctx b200_linear_ctx;

enum {
    B200_OK = 0,
    B200_E_BADARG = 1,       /* null pointer, non-positive dimension, unknown enum */
    B200_E_CUDA = 2,         /* a CUDA runtime/driver call failed (see b200_linear_last_cuda_error) */
    B200_E_NODEVICE = 3,     /* no sm_100 device is current */
    B200_E_DEVICE_WAIT = 4,  /* a kernel gave up on a bounded wait (see b200_linear_sync) */
    B200_E_TOOBIG = 5        /* size beyond a stated limit */
};

/* GEMM selector for b200_linear_gemm_*: the three products of the linear layer. */
enum {
    B200_GEMM_FWD_NN = 0,    /* out[M,N]  = A[M,K] * B[K,N]             (cuda/matmul.cu:10,61)  */
    B200_GEMM_DGRAD_NT = 1,  /* out[M,K]  = dC[M,N] * B[K,N]^T          (cuda/matmul.cu:30,82)  */
    B200_GEMM_WGRAD_TN = 2   /* out[K,N] (+)= A[M,K]^T * dC[M,N]        (cuda/matmul.cu:40,94)  */
};

/* Context = what the reference keeps in its cublasHandle_t (cublasCreate / cublasDestroy in
 * llama2-mistral/src/model.cpp:11,372,404,709): stream, SM count, tensor-map cache, split-K
 * workspace and the device status word.  One per process and GPU. */
int b200_linear_create(b200_linear_ctx** out);
int b200_linear_destroy(b200_linear_ctx* ctx);
/* The context that the reference's C++ overloads exported by this library (matmul_forward and the other
 * kernels.cuh signatures, which carry no context of ours) use on the current device: created on first use,
 * on the legacy default stream, destroyed never.  NULL if it cannot be created. */
b200_linear_ctx* b200_linear_default_ctx(void);
/* cudaStream_t passed as void*; replaces cublasSetStream (never called by the reference,
 * which stays on the legacy default stream). */
int b200_linear_set_stream(b200_linear_ctx* ctx, void* cuda_stream);
/* Synchronise the context's stream and return B200_E_DEVICE_WAIT if any kernel since the last
 * call recorded a timed-out wait (the raw device code is stored in *device_code if non-null). */
int b200_linear_sync(b200_linear_ctx* ctx, int* device_code);
/* Self-test of the error path above, with no counterpart in the reference: launches one warp that waits
 * (at most limit_cycles SM clocks, at most about a second) on a barrier that nothing completes.  The wait
 * gives up, the kernel records its code and returns; the next b200_linear_sync reports
 * B200_E_DEVICE_WAIT and clears it, and the context stays usable.  Nothing faults or hangs. */
int b200_linear_selftest_wait_timeout(b200_linear_ctx* ctx, long long limit_cycles);
/* Device address of the context's status word (what b200_linear_sync reads): for kernels of this library that
 * are launched outside the context's own entry points and report their bounded waits through it. */
int* b200_linear_status_word(b200_linear_ctx* ctx);
/* Number of kernels this library has launched on this context so far. */
long long b200_linear_launch_count(const b200_linear_ctx* ctx);
int b200_linear_last_cuda_error(const b200_linear_ctx* ctx);
const char* b200_linear_strerror(int code);

/* bf16 storage, fp32 accumulate.  Replaces
 *   matmul_forward(cublasHandle_t, __nv_bfloat16* C, const __nv_bfloat16* A, const __nv_bfloat16* B, M,N,K)
 *   cuda/matmul.cu:55-71, declared cuda/kernels.cuh:348.   C = bf16_rn(A*B). */
int b200_linear_forward_bf16(b200_linear_ctx* ctx, void* C, const void* A, const void* B, int M, int N,
                             int K);
/* Replaces matmul_backward(handle, dA, dB, dC, A, B, M,N,K), cuda/matmul.cu:73-104, declared
 * cuda/kernels.cuh:350.  dA = bf16_rn(dC*B^T);  dB = bf16_rn(bf16_rn(A^T*dC) + float(dB))  (beta = 1,
 * the product rounded to bf16 before the old gradient is added, exactly as the reference's cuBLAS does).
 * dA or dB may be NULL to skip that product. */
int b200_linear_backward_bf16(b200_linear_ctx* ctx, void* dA, void* dB, const void* dC, const void* A,
                              const void* B, int M, int N, int K);
/* True-fp32 twins.  Replace matmul_forward / matmul_backward on float*, cuda/matmul.cu:4-48,
 * declared cuda/kernels.cuh:47-65 (cublasSgemm, default math mode). */
int b200_linear_forward_f32(b200_linear_ctx* ctx, float* C, const float* A, const float* B, int M, int N,
                            int K);
int b200_linear_backward_f32(b200_linear_ctx* ctx, float* dA, float* dB, const float* dC, const float* A,
                             const float* B, int M, int N, int K);

/* One product at a time, with beta in {0,1} selectable for every layout (the shape/layout/beta
 * sweep).  `which` is a B200_GEMM_* value; M,N,K keep the meaning above for every `which`;
 * x, y are the two inputs in the order of the formulas above (A,B / dC,B / A,dC). */
int b200_linear_gemm_bf16(b200_linear_ctx* ctx, int which, int beta1, void* out, const void* x,
                          const void* y, int M, int N, int K);
int b200_linear_gemm_f32(b200_linear_ctx* ctx, int which, int beta1, float* out, const float* x,
                         const float* y, int M, int N, int K);
/* The bf16 product on operands that are column ranges of wider row-major matrices: ld_out, ld_x, ld_y are
 * the row pitches in elements (0 = dense).  This is how one rank multiplies by its vocabulary shard of the
 * LM head w_out[K, V] (llama2-mistral/src/model.cpp:612,635) where it lies: y = w_out + col0, ld_y = V,
 * N = the shard's width; likewise out = dw_out + col0 for the weight gradient.  Pitches must be multiples
 * of 8 elements, pointers 16-byte aligned and N, K multiples of 8 (B200_E_BADARG otherwise: the CUDA-core
 * kernel behind the dense entry points takes dense operands only). */
int b200_linear_gemm_bf16_ld(b200_linear_ctx* ctx, int which, int beta1, void* out, long long ld_out,
                             const void* x, long long ld_x, const void* y, long long ld_y, int M, int N, int K);

/* Up to three bf16 products that share an operand, in ONE launch (count = 1..3; dense operands).  This is how the
 * callers of matmul_forward / matmul_backward that issue several GEMMs on one input are served: the Q, K, V
 * projections of cuda/attention.cu:597-599 (forward) and :671-688 (backward), gate and up of cuda/swiglu.cu:161-162
 * and :192-202.
 *   B200_GEMM_FWD_NN    outs[i][M, Ns[i]]   = xs[0][M, K] * ys[i][K, Ns[i]]
 *   B200_GEMM_WGRAD_TN  outs[i][K, Ns[i]] (+)= xs[0][M, K]^T * ys[i][M, Ns[i]]
 *   B200_GEMM_DGRAD_NT  outs[0][M, K]     (+)= sum_i xs[i][M, Ns[i]] * ys[i][K, Ns[i]]^T
 * The first two lay the products side by side along the output columns (a column tile belongs to one product);
 * the third runs them through one accumulator, so the sum over i is formed in fp32 and rounded to bf16 once
 * (the reference adds the three bf16 results with residual_forward: up to three roundings).  Needs Ns[i] % 64 == 0,
 * K % 8 == 0 (K % 64 == 0 for the weight gradient) and 16-byte-aligned pointers; anything else runs as `count` single
 * products with beta = 1 accumulation.  No counterpart in the reference (one cuBLAS call per product). */
int b200_linear_gemm_bf16_grouped(b200_linear_ctx* ctx, int which, int beta1, int count, void* const* outs,
                                  const void* const* xs, const void* const* ys, int M, const int* Ns, int K);
/* matmul_backward for such a group: dA (+)= sum_i dCs[i] * Bs[i]^T (beta1_dA selects +=), dBs[i] += A^T * dCs[i];
 * two launches side by side, like b200_linear_backward_bf16.  dA or dBs may be NULL. */
int b200_linear_backward_bf16_grouped(b200_linear_ctx* ctx, int count, void* dA, int beta1_dA, void* const* dBs,
                                      const void* const* dCs, const void* A, const void* const* Bs, int M,
                                      const int* Ns, int K);
/* The LM head and the first pass of its cross-entropy in one GEMM (llama2-mistral/src/model.cpp:612-613,
 * cuda/crossentropy.cu:96-110): logits[M, N] = x[M, K] w[K, N] stored as bf16 (row pitches ld_* in elements, 0 = dense:
 * a vocabulary shard of w_out where it lies) and, per row, the maximum, sum exp(l - max) and the target's logit over
 * these N columns (global columns col0 .. col0 + N - 1; row_target = 0 when the target lives elsewhere) -- the
 * outputs of b200_ce_shard_stats_bf16, formed in the GEMM's epilogue from the rounded logits while they are in
 * registers instead of by a pass over the stored matrix (one read of M x N x 2 bytes less).  Continue with
 * b200_ce_shard_rescale / _loss / _backward_bf16.  B200_E_BADARG for operands the tensor-core kernel cannot take
 * (N, K, pitches not multiples of 8, pointers not 16-byte aligned): use b200_linear_gemm_bf16_ld and
 * b200_ce_shard_stats_bf16 then.  Asynchronous on the context's stream. */
int b200_linear_forward_ce_stats_bf16(b200_linear_ctx* ctx, void* logits, long long ld_out, const void* x, long long ld_x,
                                      const void* w, long long ld_w, int M, int N, int K, const int* targets, int col0,
                                      float* row_max, float* row_sum, float* row_target);

/* The forward half of swiglu_forward (cuda/swiglu.cu:161-164) in one launch: gate[M, ff] = x[M, K] w_gate[K, ff],
 * up = x w_up, hidden = SiLU(gate) * up, the last formed in the GEMM's epilogue from the bf16-rounded gate and up (the
 * values the reference's element-wise kernel reads back from memory).  Returns B200_E_BADARG for shapes or pointers
 * this kernel does not take (ff % 128 != 0, K % 8 != 0, pointers not 16-byte aligned, fewer than two SMs); the
 * caller then uses b200_linear_gemm_bf16_grouped and its own element-wise pass. */
int b200_linear_swiglu_forward_bf16(b200_linear_ctx* ctx, void* gate, void* up, void* hidden, const void* x,
                                    const void* w_gate, const void* w_up, int M, int ff, int K);

/* Tuning / introspection.  A plan is what the dispatcher would launch for a bf16 product:
 * tile width BN (output columns per tile; 0 = CUDA-core kernel), cta_pair (1 = 256-row tiles
 * computed by a 2-CTA cluster), and the work split: of `tiles` output tiles the first `dp_tiles`
 * are computed whole, the others are each cut into `splits` ranges of the contraction
 * (`sk_items` partial work items in all).  Pure host arithmetic: usable without a GPU. */
typedef struct {
    int bn;
    int cta_pair;
    int splits;
    int m_fastest;
    int tiles;
    int waves_x100;
    int dp_tiles;
    int sk_items;
    int cluster_split;  /* > 1: every tile is shared by a cluster of this many CTAs (or CTA pairs), one
                           range of the contraction each, summed through distributed shared memory */
    int est_ns;         /* the cost model's estimate of the kernel's duration on sm_count SMs, nanoseconds */
} b200_linear_plan_t;
int b200_linear_plan_bf16(int which, int beta1, int M, int N, int K, int sm_count,
                          b200_linear_plan_t* plan);
/* The plan b200_linear_gemm_bf16_grouped would launch (host arithmetic only; usable without a GPU): the tile width
 * divides every Ns[i] for the column-concatenated products, plan->bn == 0 when the shapes run as single products. */
int b200_linear_plan_grouped_bf16(int which, int count, int M, const int* Ns, int K, int sm_count, b200_linear_plan_t* plan);
/* Force a plan for subsequent bf16 calls on this context (bn = -1 restores the heuristic).
 * splits: 0 = cut only the ragged last wave (automatic), 1 = cut nothing, >= 2 = cut every tile
 * (partials through the workspace), < 0 = share every tile among a cluster of |splits| CTAs (or
 * pairs) that sum through distributed shared memory (|splits| * (1 + cta_pair) <= 8, |splits| <= bn/32). */
int b200_linear_force_plan(b200_linear_ctx* ctx, int bn, int cta_pair, int splits);
/* b200_linear_backward_bf16 runs its two products side by side, each on its own share of the SMs, when the
 * cost model expects that to finish sooner than one after the other.  sm_dgrad > 0 fixes dgrad's share
 * (wgrad gets the rest) for subsequent calls; 0 restores the model's choice. */
int b200_linear_force_backward_split(b200_linear_ctx* ctx, int sm_dgrad);

/* Weight gradient dB[K,N] = bf16_rn(bf16_rn(A[M,K]^T * dC[M,N]) + dB) that allocates nothing.
 * This entry point has no counterpart in the reference.  It exists for hosts in which this
 * library must never allocate device memory: a trainer that gave the whole GPU to its own arena
 * at start-up (a later cudaMalloc just fails), or a step loop that cannot take the device-wide
 * stall of cudaMalloc/cudaFree when a context's workspace would have to grow.  It needs no
 * context: its split-K scratch is a fixed array of about 8 MiB inside the library image, resident on
 * every GPU that loads the library until the process exits.
 *   - Limit: ceil(K/128) * ceil(N/128) <= 128 output tiles (e.g. 768x2048 or 1024x2048; the 2048x4096
 *     of a fused gate/up gradient and the LM head do not fit); larger outputs return B200_E_TOOBIG.  N and K must be multiples of 8 and the pointers 16-byte
 *     aligned (B200_E_BADARG otherwise; there is no slower fallback behind this call).
 *   - The first call on each device looks up the array's device address and configures the
 *     kernel (under a lock, so threads may race for it); make that first call outside any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels can run at the same time
 *     (different streams) race.  Calls on one stream are safe; each clears the counters it needs.
 *   - Asynchronous on `cuda_stream` (a cudaStream_t; NULL = legacy default stream).
 *   - Its kernels' waits are bounded like all others; one that runs out leaves a code in a status word
 *     inside the same array, which stays set until b200_linear_noalloc_status reads it. */
int b200_linear_wgrad_bf16_noalloc(void* dB, const void* A, const void* dC, int M, int N, int K,
                                   void* cuda_stream);
/* Waits for `cuda_stream`, then returns B200_E_DEVICE_WAIT (raw code in *device_code, may be NULL) if a
 * kernel of b200_linear_wgrad_bf16_noalloc gave up on a wait on the current device since the last call,
 * and clears the word; B200_OK otherwise.  Allocates nothing either.  No counterpart in the reference. */
int b200_linear_noalloc_status(int* device_code, void* cuda_stream);

/* Cross-entropy when the LM head [K, V] is sharded by columns across GPUs (one process per GPU): the
 * per-shard device kernels.  They replace crossentropy_forward / crossentropy_softmax_backward
 * (cuda/crossentropy.cu:96-122,124-132; bf16 overloads declared cuda/kernels.cuh:402-403; called from
 * llama2-mistral/src/model.cpp:613-614,634) in that mode, where no rank ever holds a whole row of logits.
 * logits: [rows, ld] bf16, this rank's columns [0, cols) = global columns [col0, col0 + cols); targets:
 * global token ids [rows].  The host does the two small exchanges in between (all-reduce MAX of the row maxima,
 * all-reduce SUM of the re-based sums and target logits).  No context: asynchronous on `cuda_stream`
 * (a cudaStream_t; NULL = legacy default stream).  Same loss and gradient as the reference up to its bf16
 * rounding of the probabilities, which these kernels do not do (only dlogits is rounded, once).
 *   stats:    row_max = max_v l, row_sum = sum_v exp(l - row_max), row_target = l[target] or 0 if not owned
 *   rescale:  row_sum *= exp(local_max - global_max)
 *   loss:     loss = log(global_sum) + global_max - target_logit                  (= -log softmax[target])
 *   backward: dlogits = (exp(l - global_max) / global_sum - [column == target]) * scale   (in place allowed);
 *             the reference's scale is loss_scale / BT (cuda/crossentropy.cu:155). */
int b200_ce_shard_stats_bf16(const void* logits, int rows, int cols, long long ld, const int* targets, int col0,
                             float* row_max, float* row_sum, float* row_target, void* cuda_stream);
int b200_ce_shard_rescale(const float* local_max, const float* global_max, float* row_sum, int rows,
                          void* cuda_stream);
int b200_ce_shard_loss(float* loss, const float* global_max, const float* global_sum, const float* target_logit,
                       int rows, void* cuda_stream);
int b200_ce_shard_backward_bf16(void* dlogits, const void* logits, int rows, int cols, long long ld,
                                const int* targets, int col0, const float* global_max, const float* global_sum,
                                float scale, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_LINEAR_H */
