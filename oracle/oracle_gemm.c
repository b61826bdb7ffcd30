/* TEST INFRASTRUCTURE — not part of the product.
 *
 * CPU restatement of the linear-layer GEMMs of chriskuchar/llms-from-scratch-cuda
 * (cuda/matmul.cu).  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline /
 * reference legs may load this file; the product path never does.
 *
 * Parity status: the reference delegates the arithmetic to NVIDIA cuBLAS (a closed
 * third-party library, unpinned by the reference; cublasSgemm at cuda/matmul.cu:10,30,40 and
 * cublasGemmEx(CUDA_R_16BF, CUBLAS_COMPUTE_32F) at :61,82,94) and ships no test, golden
 * vector or fixture for this path, so there is nothing of the reference's own to pin this
 * restatement against on a CPU.  It is pinned instead (a) against numpy float64 matmul on
 * committed seeded fixtures (tests/golden/), and (b) on a GPU box against the reference's
 * unmodified matmul.cu built into oracle/_ref/ (see oracle/build.py).
 *
 * What is restated (row-major, leading dimension = inner extent, cuda/kernels.cuh:46-65):
 *   which 0  forward  C [M,N]  = A [M,K] * B[K,N]              cuda/matmul.cu:2-18, 55-71
 *   which 1  dgrad    dA[M,K]  = dC[M,N] * B[K,N]^T   beta=0   cuda/matmul.cu:19,26,29-37, 81-91
 *   which 2  wgrad    dB[K,N] += A [M,K]^T * dC[M,N]  beta=1   cuda/matmul.cu:20,27,39-47, 93-103
 * Inputs are float (bf16 values are exact in float); the fp64 functions accumulate in double.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* ---- seeded inputs: counter-based splitmix64 -> Box-Muller normal ---- */
static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

/* out[i] = mean + std * N(0,1), element i depends only on (seed, i). */
void oracle_fill_normal(float* out, size_t n, uint64_t seed, float mean, float std) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; ++i) {
        uint64_t r = splitmix64(seed * 0xD1342543DE82EF95ull + (uint64_t)i);
        double u1 = ((double)(r >> 40) + 1.0) * (1.0 / 16777217.0);   /* (0,1) */
        double u2 = (double)((r >> 8) & 0xFFFFFFull) * (1.0 / 16777216.0);
        double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
        out[i] = (float)(mean + std * z);
    }
}

/* Round to nearest-even bf16 and back, in place (what __float2bfloat16_rn does). */
void oracle_round_bf16(float* x, size_t n) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; ++i) {
        uint32_t u;
        memcpy(&u, &x[i], 4);
        if ((u & 0x7F800000u) != 0x7F800000u) {
            uint32_t lsb = (u >> 16) & 1u;
            u += 0x7FFFu + lsb;
        }
        u &= 0xFFFF0000u;
        memcpy(&x[i], &u, 4);
    }
}

/* ---- fp64 oracle.  out (double) = (old ? old : 0) + product.  Returns 0, or 1 on bad args. */
int oracle_gemm_f64(int which, double* out, const float* old, const float* x, const float* y, int M, int N,
                    int K) {
    if (!out || !x || !y || M <= 0 || N <= 0 || K <= 0) return 1;
    if (which == 0) { /* C[m,n] = sum_k A[m,k] B[k,n] */
#pragma omp parallel for schedule(static)
        for (int m = 0; m < M; ++m) {
            double* c = out + (size_t)m * N;
            for (int n = 0; n < N; ++n) c[n] = old ? (double)old[(size_t)m * N + n] : 0.0;
            for (int k = 0; k < K; ++k) {
                const double a = x[(size_t)m * K + k];
                const float* b = y + (size_t)k * N;
                for (int n = 0; n < N; ++n) c[n] += a * (double)b[n];
            }
        }
    } else if (which == 1) { /* dA[m,k] = sum_n dC[m,n] B[k,n] */
#pragma omp parallel for schedule(static)
        for (int m = 0; m < M; ++m) {
            const float* d = x + (size_t)m * N;
            for (int k = 0; k < K; ++k) {
                const float* b = y + (size_t)k * N;
                double s = 0.0;
#pragma omp simd reduction(+ : s)
                for (int n = 0; n < N; ++n) s += (double)d[n] * (double)b[n];
                out[(size_t)m * K + k] = s + (old ? (double)old[(size_t)m * K + k] : 0.0);
            }
        }
    } else if (which == 2) { /* dB[k,n] = old + sum_m A[m,k] dC[m,n] */
#pragma omp parallel for schedule(static)
        for (int k = 0; k < K; ++k) {
            double* o = out + (size_t)k * N;
            for (int n = 0; n < N; ++n) o[n] = old ? (double)old[(size_t)k * N + n] : 0.0;
            for (int m = 0; m < M; ++m) {
                const double a = x[(size_t)m * K + k];
                const float* d = y + (size_t)m * N;
                for (int n = 0; n < N; ++n) o[n] += a * (double)d[n];
            }
        }
    } else {
        return 1;
    }
    return 0;
}

/* fp64 value of `count` chosen output elements (rows[i], cols[i]) — for shapes whose full
 * fp64 product would take too long. */
int oracle_gemm_f64_samples(int which, double* out, const float* x, const float* y, int M, int N, int K,
                            const int* rows, const int* cols, int count) {
    if (!out || !x || !y || !rows || !cols || M <= 0 || N <= 0 || K <= 0) return 1;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < count; ++i) {
        const int r = rows[i], c = cols[i];
        double s = 0.0;
        if (which == 0)      for (int k = 0; k < K; ++k) s += (double)x[(size_t)r * K + k] * (double)y[(size_t)k * N + c];
        else if (which == 1) for (int n = 0; n < N; ++n) s += (double)x[(size_t)r * N + n] * (double)y[(size_t)c * N + n];
        else                 for (int m = 0; m < M; ++m) s += (double)x[(size_t)m * K + r] * (double)y[(size_t)m * N + c];
        out[i] = s;
    }
    return 0;
}

/* ---- fp32 host GEMM: the timed CPU baseline (all cores OpenMP gives it). ----
 * out = (beta1 ? out : 0) + product, fp32 throughout, like cublasSgemm's arithmetic. */
int oracle_gemm_f32(int which, int beta1, float* out, const float* x, const float* y, int M, int N, int K) {
    if (!out || !x || !y || M <= 0 || N <= 0 || K <= 0) return 1;
    if (which == 0) {
#pragma omp parallel for schedule(static)
        for (int m0 = 0; m0 < M; m0 += 4) {
            const int mr = M - m0 < 4 ? M - m0 : 4;
            for (int i = 0; i < mr; ++i) {
                float* c = out + (size_t)(m0 + i) * N;
                if (!beta1) memset(c, 0, sizeof(float) * (size_t)N);
            }
            for (int k = 0; k < K; ++k) {
                const float* b = y + (size_t)k * N;
                for (int i = 0; i < mr; ++i) {
                    const float a = x[(size_t)(m0 + i) * K + k];
                    float* c = out + (size_t)(m0 + i) * N;
#pragma omp simd
                    for (int n = 0; n < N; ++n) c[n] += a * b[n];
                }
            }
        }
    } else if (which == 1) {
#pragma omp parallel for schedule(static)
        for (int m = 0; m < M; ++m) {
            const float* d = x + (size_t)m * N;
            for (int k = 0; k < K; ++k) {
                const float* b = y + (size_t)k * N;
                float s = 0.f;
#pragma omp simd reduction(+ : s)
                for (int n = 0; n < N; ++n) s += d[n] * b[n];
                float* o = out + (size_t)m * K + k;
                *o = beta1 ? *o + s : s;
            }
        }
    } else if (which == 2) {
#pragma omp parallel for schedule(static)
        for (int k0 = 0; k0 < K; k0 += 4) {
            const int kr = K - k0 < 4 ? K - k0 : 4;
            for (int i = 0; i < kr; ++i)
                if (!beta1) memset(out + (size_t)(k0 + i) * N, 0, sizeof(float) * (size_t)N);
            for (int m = 0; m < M; ++m) {
                const float* d = y + (size_t)m * N;
                for (int i = 0; i < kr; ++i) {
                    const float a = x[(size_t)m * K + k0 + i];
                    float* o = out + (size_t)(k0 + i) * N;
#pragma omp simd
                    for (int n = 0; n < N; ++n) o[n] += a * d[n];
                }
            }
        }
    } else {
        return 1;
    }
    return 0;
}

int oracle_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    n = omp_get_max_threads();
#endif
    return n;
}
