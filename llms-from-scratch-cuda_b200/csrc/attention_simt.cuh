// Fused causal grouped-query attention on the CUDA cores (fp32 arithmetic, fp32 or bf16 storage):
// softmax(Q K^T / sqrt(d)) V without ever holding a [B, n_head, T, T] matrix, forward and backward.
//
// This is what the reference declares as flash_attention_forward / flash_attention_backward and leaves
// empty (cuda/flash_attention.cu:12-17,51-57; contract in cuda/kernels.cuh:316-341,420-437), and what
// replaces the seven kernels + three T x T buffers of its attention_forward / attention_backward
// (cuda/attention.cu:8-231 fp32, :419-580 bf16).  Layouts are the reference's: q, context [B*T, n_head*64],
// k, v [B*T, n_kv_head*64], query head h reads KV head h / (n_head / n_kv_head), lse [B, n_head, T] fp32
// = log sum_j exp(s_ij) of the scaled, causally masked scores.  Head dimension 64 (both model families).
//
// These kernels serve the fp32 overloads and are the checker-friendly form of the algorithm; the bf16
// overloads run on the tensor cores (attention_sm100.cuh) and fall back to these only for shapes the
// tensor-core kernels do not take.
//
// One tile primitive does all five products: acc[4x4 per thread] += sum_k At[k][r] * Bt[k][c] over 64 x 64
// tiles held "contraction index first" in shared memory with a row pitch of 68 floats (16-byte aligned
// float4 reads, no bank conflicts across the 16 x 16 thread grid).
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

#include "gemm_simt.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int AT_TILE = 64;       // query rows / key rows per tile, and the head dimension
constexpr int AT_PITCH = 68;      // floats per tile row in shared memory
constexpr int AT_THREADS = 256;   // 16 x 16 threads, 4 x 4 outputs each
constexpr int AT_TILE_FLOATS = AT_TILE * AT_PITCH;

struct AttnParams {
    int B, T, n_head, n_kv_head;
    float scale;  // 1 / sqrt(head_dim)
};

// acc[i][j] += sum_k At[k][r0 + i] * Bt[k][c0 + j]
__device__ __forceinline__ void at_mm(float (&acc)[4][4], const float* __restrict__ At, const float* __restrict__ Bt,
                                      int r0, int c0) {
#pragma unroll 8
    for (int k = 0; k < AT_TILE; ++k) {
        const float4 a = *reinterpret_cast<const float4*>(At + k * AT_PITCH + r0);
        const float4 b = *reinterpret_cast<const float4*>(Bt + k * AT_PITCH + c0);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
}

// 64 rows (tokens t0 .. t0+63 of batch b, zero beyond T) x 64 columns (col0 ..) of a [B*T, ld] matrix into
// shared memory, as dst[row][col] (TRANSPOSE = false) or dst[col][row] (TRANSPOSE = true).
template <typename T, bool TRANSPOSE>
__device__ __forceinline__ void at_load(float* __restrict__ dst, const T* __restrict__ src, long long ld, int b, int Tlen,
                                        int t0, int col0) {
    for (int idx = threadIdx.x; idx < AT_TILE * AT_TILE; idx += AT_THREADS) {
        const int r = idx >> 6, c = idx & 63;
        const int t = t0 + r;
        const float v = t < Tlen ? to_f32<T>(src[(static_cast<long long>(b) * Tlen + t) * ld + col0 + c]) : 0.f;
        if constexpr (TRANSPOSE) dst[c * AT_PITCH + r] = v;
        else dst[r * AT_PITCH + c] = v;
    }
}

// The thread's 4 x 4 block of a tile held in registers, written as dst[row][col] or dst[col][row].
template <bool TRANSPOSE>
__device__ __forceinline__ void at_store_block(float* __restrict__ dst, const float (&x)[4][4], int r0, int c0) {
    if constexpr (TRANSPOSE) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float4*>(dst + (c0 + j) * AT_PITCH + r0) = make_float4(x[0][j], x[1][j], x[2][j], x[3][j]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            *reinterpret_cast<float4*>(dst + (r0 + i) * AT_PITCH + c0) = make_float4(x[i][0], x[i][1], x[i][2], x[i][3]);
    }
}

__device__ __forceinline__ float at_row_max16(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float at_row_sum16(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Forward.  grid = (query tiles, n_head, B); the longest rows (last query tiles) are scheduled first.
template <typename T>
__global__ void __launch_bounds__(AT_THREADS)
attn_fwd_simt(T* __restrict__ context, float* __restrict__ lse, const T* __restrict__ q, const T* __restrict__ k,
              const T* __restrict__ v, const AttnParams p) {
    griddep_sync();
    extern __shared__ __align__(16) float at_smem[];
    float* Qt = at_smem;                    // [d][r]
    float* Kt = Qt + AT_TILE_FLOATS;        // [d][c]
    float* Vs = Kt + AT_TILE_FLOATS;        // [c][d]
    float* Pt = Vs + AT_TILE_FLOATS;        // [c][r]
    const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (p.n_head / p.n_kv_head);
    const int C = p.n_head * AT_TILE, KV = p.n_kv_head * AT_TILE;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15, r0 = ty * 4, c0 = tx * 4;
    at_load<T, true>(Qt, q, C, b, p.T, qt * AT_TILE, h * AT_TILE);
    float o[4][4] = {}, m[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { m[i] = -INFINITY; l[i] = 0.f; }
    for (int j = 0; j <= qt; ++j) {
        __syncthreads();  // the previous tile's products have read Kt, Vs, Pt
        at_load<T, true>(Kt, k, KV, b, p.T, j * AT_TILE, kvh * AT_TILE);
        at_load<T, false>(Vs, v, KV, b, p.T, j * AT_TILE, kvh * AT_TILE);
        __syncthreads();
        float s[4][4] = {};
        at_mm(s, Qt, Kt, r0, c0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = qt * AT_TILE + r0 + i;
            float mx = -INFINITY;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int col = j * AT_TILE + c0 + jj;
                s[i][jj] = (col > row || col >= p.T) ? -INFINITY : s[i][jj] * p.scale;
                mx = fmaxf(mx, s[i][jj]);
            }
            mx = at_row_max16(mx);
            const float m_new = fmaxf(m[i], mx);
            const float alpha = m[i] == -INFINITY ? 0.f : expf(m[i] - m_new);
            float sum = 0.f;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                s[i][jj] = s[i][jj] == -INFINITY ? 0.f : expf(s[i][jj] - m_new);
                sum += s[i][jj];
            }
            sum = at_row_sum16(sum);
            l[i] = l[i] * alpha + sum;
            m[i] = m_new;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) o[i][jj] *= alpha;
        }
        at_store_block<true>(Pt, s, r0, c0);
        __syncthreads();
        at_mm(o, Pt, Vs, r0, c0);  // o[r][d] += sum_c P[r][c] V[c][d]
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = qt * AT_TILE + r0 + i;
        if (row >= p.T) continue;
        const float inv = 1.0f / l[i];
        T* dst = context + (static_cast<long long>(b) * p.T + row) * C + h * AT_TILE + c0;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) dst[jj] = from_f32<T>(o[i][jj] * inv);
        if (tx == 0) lse[(static_cast<long long>(b) * p.n_head + h) * p.T + row] = m[i] + logf(l[i]);
    }
}

// delta[b, h, t] = sum_d dcontext[t, h, d] * context[t, h, d]  (= sum_j P_tj dP_tj): one warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(256)
attn_delta(float* __restrict__ delta, const T* __restrict__ dcontext, const T* __restrict__ context, const AttnParams p) {
    griddep_sync();
    const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long total = static_cast<long long>(p.B) * p.T * p.n_head;
    if (warp >= total) return;
    const int h = static_cast<int>(warp % p.n_head);
    const long long bt = warp / p.n_head;
    const long long base = (bt * p.n_head + h) * AT_TILE;
    float s = to_f32<T>(dcontext[base + lane]) * to_f32<T>(context[base + lane]) +
              to_f32<T>(dcontext[base + 32 + lane]) * to_f32<T>(context[base + 32 + lane]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        const int b = static_cast<int>(bt / p.T), t = static_cast<int>(bt % p.T);
        delta[(static_cast<long long>(b) * p.n_head + h) * p.T + t] = s;
    }
}

// P and dS of one (query tile, key tile) pair from the tiles in shared memory; rows = queries, cols = keys.
__device__ __forceinline__ void at_p_ds(float (&pv)[4][4], float (&ds)[4][4], const float* Qt, const float* Kt,
                                        const float* dOt, const float* Vt, const float* lse_s, const float* delta_s,
                                        int r0, int c0, int row_base, int col_base, int Tlen, float scale) {
    float s[4][4] = {}, dp[4][4] = {};
    at_mm(s, Qt, Kt, r0, c0);
    at_mm(dp, dOt, Vt, r0, c0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row_base + r0 + i;
        const float ls = lse_s[r0 + i], dl = delta_s[r0 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = col_base + c0 + j;
            const bool masked = col > row || col >= Tlen || row >= Tlen;
            const float pr = masked ? 0.f : expf(s[i][j] * scale - ls);
            pv[i][j] = pr;
            ds[i][j] = pr * (dp[i][j] - dl);
        }
    }
}

// dQ.  grid = (query tiles, n_head, B).  dQ_i = scale * sum_{j <= i} dS_ij K_j.
template <typename T>
__global__ void __launch_bounds__(AT_THREADS)
attn_bwd_dq_simt(T* __restrict__ dq, const T* __restrict__ dcontext, const T* __restrict__ q, const T* __restrict__ k,
                 const T* __restrict__ v, const float* __restrict__ lse, const float* __restrict__ delta,
                 const AttnParams p) {
    griddep_sync();
    extern __shared__ __align__(16) float at_smem[];
    float* Qt = at_smem;                     // [d][r]
    float* dOt = Qt + AT_TILE_FLOATS;        // [d][r]
    float* Kt = dOt + AT_TILE_FLOATS;        // [d][c]
    float* Vt = Kt + AT_TILE_FLOATS;         // [d][c]
    float* Ks = Vt + AT_TILE_FLOATS;         // [c][d]
    float* dSt = Ks + AT_TILE_FLOATS;        // [c][r]
    float* lse_s = dSt + AT_TILE_FLOATS;     // [r]
    float* delta_s = lse_s + AT_TILE;        // [r]
    const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (p.n_head / p.n_kv_head);
    const int C = p.n_head * AT_TILE, KV = p.n_kv_head * AT_TILE;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15, r0 = ty * 4, c0 = tx * 4;
    at_load<T, true>(Qt, q, C, b, p.T, qt * AT_TILE, h * AT_TILE);
    at_load<T, true>(dOt, dcontext, C, b, p.T, qt * AT_TILE, h * AT_TILE);
    if (threadIdx.x < AT_TILE) {
        const int t = qt * AT_TILE + threadIdx.x;
        const long long idx = (static_cast<long long>(b) * p.n_head + h) * p.T + t;
        lse_s[threadIdx.x] = t < p.T ? lse[idx] : 0.f;
        delta_s[threadIdx.x] = t < p.T ? delta[idx] : 0.f;
    }
    float acc[4][4] = {};
    for (int j = 0; j <= qt; ++j) {
        __syncthreads();
        at_load<T, true>(Kt, k, KV, b, p.T, j * AT_TILE, kvh * AT_TILE);
        at_load<T, true>(Vt, v, KV, b, p.T, j * AT_TILE, kvh * AT_TILE);
        at_load<T, false>(Ks, k, KV, b, p.T, j * AT_TILE, kvh * AT_TILE);
        __syncthreads();
        float pv[4][4], ds[4][4];
        at_p_ds(pv, ds, Qt, Kt, dOt, Vt, lse_s, delta_s, r0, c0, qt * AT_TILE, j * AT_TILE, p.T, p.scale);
        at_store_block<true>(dSt, ds, r0, c0);
        __syncthreads();
        at_mm(acc, dSt, Ks, r0, c0);  // dQ[r][d] += sum_c dS[r][c] K[c][d]
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = qt * AT_TILE + r0 + i;
        if (row >= p.T) continue;
        T* dst = dq + (static_cast<long long>(b) * p.T + row) * C + h * AT_TILE + c0;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) dst[jj] = from_f32<T>(acc[i][jj] * p.scale);
    }
}

// dK, dV.  grid = (key tiles, n_kv_head, B).  Every query head of the group and every query tile at or after
// the key tile contributes; the sums are formed inside the CTA in a fixed order (no atomics).
//   dV_j = sum_{h in group, i >= j} P_ij^T dO_i        dK_j = scale * sum dS_ij^T Q_i
template <typename T>
__global__ void __launch_bounds__(AT_THREADS)
attn_bwd_dkv_simt(T* __restrict__ dk, T* __restrict__ dv, const T* __restrict__ dcontext, const T* __restrict__ q,
                  const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ lse,
                  const float* __restrict__ delta, const AttnParams p) {
    griddep_sync();
    extern __shared__ __align__(16) float at_smem[];
    float* Kt = at_smem;                     // [d][c]
    float* Vt = Kt + AT_TILE_FLOATS;         // [d][c]
    float* Qt = Vt + AT_TILE_FLOATS;         // [d][r]
    float* dOt = Qt + AT_TILE_FLOATS;        // [d][r]
    float* Qs = dOt + AT_TILE_FLOATS;        // [r][d]
    float* dOs = Qs + AT_TILE_FLOATS;        // [r][d]
    float* Pn = dOs + AT_TILE_FLOATS;        // [r][c]
    float* dSn = Pn + AT_TILE_FLOATS;        // [r][c]
    float* lse_s = dSn + AT_TILE_FLOATS;
    float* delta_s = lse_s + AT_TILE;
    const int kt = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int ratio = p.n_head / p.n_kv_head;
    const int C = p.n_head * AT_TILE, KV = p.n_kv_head * AT_TILE;
    const int q_tiles = (p.T + AT_TILE - 1) / AT_TILE;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15, r0 = ty * 4, c0 = tx * 4;
    at_load<T, true>(Kt, k, KV, b, p.T, kt * AT_TILE, kvh * AT_TILE);
    at_load<T, true>(Vt, v, KV, b, p.T, kt * AT_TILE, kvh * AT_TILE);
    float dk_acc[4][4] = {}, dv_acc[4][4] = {};
    for (int hg = 0; hg < ratio; ++hg) {
        const int h = kvh * ratio + hg;
        for (int i = kt; i < q_tiles; ++i) {
            __syncthreads();
            at_load<T, true>(Qt, q, C, b, p.T, i * AT_TILE, h * AT_TILE);
            at_load<T, true>(dOt, dcontext, C, b, p.T, i * AT_TILE, h * AT_TILE);
            at_load<T, false>(Qs, q, C, b, p.T, i * AT_TILE, h * AT_TILE);
            at_load<T, false>(dOs, dcontext, C, b, p.T, i * AT_TILE, h * AT_TILE);
            if (threadIdx.x < AT_TILE) {
                const int t = i * AT_TILE + threadIdx.x;
                const long long idx = (static_cast<long long>(b) * p.n_head + h) * p.T + t;
                lse_s[threadIdx.x] = t < p.T ? lse[idx] : 0.f;
                delta_s[threadIdx.x] = t < p.T ? delta[idx] : 0.f;
            }
            __syncthreads();
            float pv[4][4], ds[4][4];
            at_p_ds(pv, ds, Qt, Kt, dOt, Vt, lse_s, delta_s, r0, c0, i * AT_TILE, kt * AT_TILE, p.T, p.scale);
            at_store_block<false>(Pn, pv, r0, c0);
            at_store_block<false>(dSn, ds, r0, c0);
            __syncthreads();
            // this thread's output block: key rows r0.., head-dimension columns c0..
            at_mm(dv_acc, Pn, dOs, r0, c0);   // dV[c][d] += sum_r P[r][c] dO[r][d]
            at_mm(dk_acc, dSn, Qs, r0, c0);   // dK[c][d] += sum_r dS[r][c] Q[r][d]
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = kt * AT_TILE + r0 + i;
        if (row >= p.T) continue;
        const long long off = (static_cast<long long>(b) * p.T + row) * KV + kvh * AT_TILE + c0;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            dk[off + jj] = from_f32<T>(dk_acc[i][jj] * p.scale);
            dv[off + jj] = from_f32<T>(dv_acc[i][jj]);
        }
    }
}

constexpr int ATTN_FWD_SMEM = 4 * AT_TILE_FLOATS * 4;
constexpr int ATTN_DQ_SMEM = (6 * AT_TILE_FLOATS + 2 * AT_TILE) * 4;
constexpr int ATTN_DKV_SMEM = (8 * AT_TILE_FLOATS + 2 * AT_TILE) * 4;

}  // namespace b200
