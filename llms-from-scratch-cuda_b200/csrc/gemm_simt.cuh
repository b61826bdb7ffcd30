// CUDA-core GEMM used for (a) the true-fp32 overloads of the reference's linear
// layer (cuda/matmul.cu:4-48 of the reference: cublasSgemm, no TF32) and (b) bf16
// shapes whose row pitch is not a multiple of 16 bytes and therefore cannot be
// described by a TMA tensor map.  Same operand model as the tensor-core kernel:
//     D[Mo, No] = sum_c P[Mo, c] * Q[No, c],  each operand K-major or MN-major.
// 128 x 128 x 16 tiles, 256 threads, 8 x 8 outputs per thread, fp32 FMA.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

namespace b200 {

constexpr int ST_BM = 128, ST_BN = 128, ST_BK = 16, ST_THREADS = 256, ST_PAD = 4;

struct SimtParams {
    int Mo, No, Kc;
    int splits, kc_per_split;  // split-K over the contraction (kc_per_split multiple of ST_BK)
    const void* P;
    const void* Q;
    void* out;                 // T [Mo,No] (splits == 1) or fp32 workspace [splits,Mo,No]
    int beta1;                 // only with splits == 1: out = acc + out
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Load one 128(row) x 16(c) operand tile into smem laid out [c][row (+pad)].
//   K-major : global element (row, c) at base[row * ld + c],  ld = Kc
//   MN-major: global element (row, c) at base[c * ld + row],  ld = number of rows
template <typename T, bool MN, bool VEC>
__device__ __forceinline__ void simt_fetch(float (&reg)[8], const T* __restrict__ base, long long ld,
                                           int row0, int nrows, int c0, int c_end) {
    const int t = threadIdx.x;
    if constexpr (MN) {
        // thread -> (c = t/32 + 8*h, 4 consecutive rows at (t%32)*4)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c = c0 + (t >> 5) + 8 * h;
            const int r = row0 + (t & 31) * 4;
            if constexpr (VEC) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < c_end && r < nrows) v = *reinterpret_cast<const float4*>(base + (long long)c * ld + r);
                reg[4 * h] = v.x; reg[4 * h + 1] = v.y; reg[4 * h + 2] = v.z; reg[4 * h + 3] = v.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    reg[4 * h + e] = (c < c_end && r + e < nrows) ? to_f32<T>(base[(long long)c * ld + r + e]) : 0.f;
            }
        }
    } else {
        // thread -> (row = t/4 + 64*h, 4 consecutive c at (t%4)*4)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = row0 + (t >> 2) + 64 * h;
            const int c = c0 + (t & 3) * 4;
            if constexpr (VEC) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < nrows && c < c_end) v = *reinterpret_cast<const float4*>(base + (long long)r * ld + c);
                reg[4 * h] = v.x; reg[4 * h + 1] = v.y; reg[4 * h + 2] = v.z; reg[4 * h + 3] = v.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    reg[4 * h + e] = (r < nrows && c + e < c_end) ? to_f32<T>(base[(long long)r * ld + c + e]) : 0.f;
            }
        }
    }
}
template <bool MN>
__device__ __forceinline__ void simt_stash(float (*s)[ST_BM + ST_PAD], const float (&reg)[8]) {
    const int t = threadIdx.x;
    if constexpr (MN) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
            *reinterpret_cast<float4*>(&s[(t >> 5) + 8 * h][(t & 31) * 4]) =
                make_float4(reg[4 * h], reg[4 * h + 1], reg[4 * h + 2], reg[4 * h + 3]);
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[(t & 3) * 4 + e][(t >> 2) + 64 * h] = reg[4 * h + e];
    }
}

// VEC requires fp32 operands whose pitches (and Kc split bounds) are multiples of 4 elements.
template <typename T, bool P_MN, bool Q_MN, bool VEC>
__global__ void __launch_bounds__(ST_THREADS)
gemm_simt(const SimtParams p) {
    __shared__ __align__(16) float sP[2][ST_BK][ST_BM + ST_PAD];
    __shared__ __align__(16) float sQ[2][ST_BK][ST_BN + ST_PAD];
    const T* P = reinterpret_cast<const T*>(p.P);
    const T* Q = reinterpret_cast<const T*>(p.Q);
    const int m0 = blockIdx.y * ST_BM, n0 = blockIdx.x * ST_BN, split = blockIdx.z;
    const int c_begin = split * p.kc_per_split;
    const int c_end = min(c_begin + p.kc_per_split, p.Kc);
    const long long ldP = P_MN ? p.Mo : p.Kc, ldQ = Q_MN ? p.No : p.Kc;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float rP[8], rQ[8];
    simt_fetch<T, P_MN, VEC>(rP, P, ldP, m0, p.Mo, c_begin, c_end);
    simt_fetch<T, Q_MN, VEC>(rQ, Q, ldQ, n0, p.No, c_begin, c_end);
    simt_stash<P_MN>(sP[0], rP);
    simt_stash<Q_MN>(sQ[0], rQ);
    __syncthreads();

    int buf = 0;
    for (int c0 = c_begin; c0 < c_end; c0 += ST_BK) {
        const bool more = c0 + ST_BK < c_end;
        if (more) {
            simt_fetch<T, P_MN, VEC>(rP, P, ldP, m0, p.Mo, c0 + ST_BK, c_end);
            simt_fetch<T, Q_MN, VEC>(rQ, Q, ldQ, n0, p.No, c0 + ST_BK, c_end);
        }
#pragma unroll
        for (int k = 0; k < ST_BK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&sP[buf][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&sP[buf][k][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&sQ[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&sQ[buf][k][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) {
            simt_stash<P_MN>(sP[buf ^ 1], rP);
            simt_stash<Q_MN>(sQ[buf ^ 1], rQ);
        }
        __syncthreads();
        buf ^= 1;
    }

    const bool partial = p.splits > 1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (row >= p.Mo) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (col >= p.No) continue;
            const size_t idx = static_cast<size_t>(row) * p.No + col;
            if (partial) {
                reinterpret_cast<float*>(p.out)[static_cast<size_t>(split) * p.Mo * p.No + idx] = acc[i][j];
            } else {
                T* o = reinterpret_cast<T*>(p.out);
                // beta = 1 rounds like the tensor-core path and the reference's cuBLAS: the product is rounded
                // to the storage type before the old value is added (a no-op for fp32)
                o[idx] = p.beta1 ? from_f32<T>(to_f32<T>(from_f32<T>(acc[i][j])) + to_f32<T>(o[idx]))
                                 : from_f32<T>(acc[i][j]);
            }
        }
    }
}

// out = (beta1 ? out : 0) + sum_s ws[s], summed in the fixed order s = 0..S-1.
template <typename T>
__global__ void splitk_reduce_generic(T* __restrict__ out, const float* __restrict__ ws, long long n,
                                      int splits, int beta1) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float a = 0.f;
        for (int s = 0; s < splits; ++s) a += ws[s * n + i];
        if (beta1) a = to_f32<T>(from_f32<T>(a)) + to_f32<T>(out[i]);  // product rounded first, as above
        out[i] = from_f32<T>(a);
    }
}

}  // namespace b200
