// Cross-entropy over a vocabulary that is split across GPUs: the per-shard kernels.
//
// The reference computes softmax cross-entropy on one GPU with one thread per row
// (cuda/crossentropy.cu:96-122: row maximum, exponentials, normalisation, -log p[target]) and its
// gradient element-wise (cuda/crossentropy.cu:124-132: (p - onehot) * scale).  When the LM head
// [K, V] is sharded by columns (llama2-mistral/src/model.cpp:612-614,634-635 are the call sites that a
// multi-GPU driver re-orchestrates), every rank holds logits[BT, V_r] for its columns only and
// the row statistics have to be combined across ranks:
//
//   1. ce_shard_stats:    per row, over this rank's columns: m_r = max, s_r = sum exp(l - m_r), and
//                         the target's logit if this rank owns the target column      (one pass over HBM)
//      all-reduce MAX of m_r -> m
//   2. ce_shard_rescale:  s_r *= exp(m_r - m)                                         ([BT] floats)
//      all-reduce SUM of (s_r, target logit) -> (s, l_t)
//   3. ce_shard_loss:     loss = log s + m - l_t                                      ([BT] floats)
//   4. ce_shard_backward: dlogits = (exp(l - m) / s - [column == target]) * scale     (read + write)
//
// All of them are bound by HBM bandwidth: 2 bytes read per logit in (1), 2 read + 2 written in (4).
// Unlike the reference, probabilities are never rounded to bf16 on the way (it stores exp(l - max) and
// p as bf16 in place of the logits and takes -log of the rounded p); only dlogits is rounded, once.
#pragma once

#include <cuda_bf16.h>
#include <cstdint>

namespace b200 {

constexpr int CE_THREADS = 256;

// A logit of -inf (a masked column) contributes nothing; without the guards below a row or a lane's share
// that is all -inf would compute exp(-inf - -inf) = exp(NaN).
__device__ __forceinline__ void ce_online_add(float& m, float& s, float x) {
    if (x == -INFINITY) return;
    if (x > m) {
        s = s * __expf(m - x) + 1.0f;  // exp(-inf) = 0 covers the first element
        m = x;
    } else {
        s += __expf(x - m);
    }
}
__device__ __forceinline__ void ce_online_merge(float& m, float& s, float m2, float s2) {
    if (m2 > m) {
        s = s * __expf(m - m2) + s2;
        m = m2;
    } else if (m2 > -INFINITY) {
        s += s2 * __expf(m2 - m);
    }
}

__device__ __forceinline__ void ce_add_vec8(float& m, float& s, const uint4& u) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float x[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        x[2 * j] = __uint_as_float(w[j] << 16);
        x[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
    // the maximum of the eight first: one re-basing of the running sum at most (rare once the running
    // maximum has settled), then eight exponentials without a branch
    const float vm = fmaxf(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])), fmaxf(fmaxf(x[4], x[5]), fmaxf(x[6], x[7])));
    if (vm > m) {
        s *= __expf(m - vm);  // exp(-inf) = 0 covers the first vector
        m = vm;
    }
    if (m == -INFINITY) return;  // everything so far is masked: nothing to add
    float add = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) add += __expf(x[j] - m);
    s += add;
}

// One warp per row (grid-stride over rows), four 16-byte loads in flight per lane; the row is reduced with
// shuffles only.  logits: [rows, ld] bf16, columns [0, cols) belong to this shard and are global columns
// [col0, col0 + cols).  Outputs per row: max, sum of exp(l - max), target logit (0 if the target column
// lives on another rank).  cols == 0 gives (-inf, 0, 0).
__global__ void __launch_bounds__(CE_THREADS)
ce_shard_stats_bf16(const __nv_bfloat16* __restrict__ logits, int rows, int cols, long long ld,
                    const int* __restrict__ targets, int col0, float* __restrict__ row_max,
                    float* __restrict__ row_sum, float* __restrict__ row_tgt) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = CE_THREADS / 32;
    for (int r = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps_per_cta) {
        const __nv_bfloat16* row = logits + static_cast<long long>(r) * ld;
        float m = -INFINITY, s = 0.f;
        // 16-byte loads where the row start allows it (ld and the base pointer multiples of 8 elements)
        int v0 = 0;
        if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
            const int nvec = cols >> 3;
            const uint4* row4 = reinterpret_cast<const uint4*>(row);
            int i = lane;
            for (; i + 96 < nvec; i += 128) {
                const uint4 u0 = __ldg(row4 + i), u1 = __ldg(row4 + i + 32), u2 = __ldg(row4 + i + 64),
                            u3 = __ldg(row4 + i + 96);
                ce_add_vec8(m, s, u0);
                ce_add_vec8(m, s, u1);
                ce_add_vec8(m, s, u2);
                ce_add_vec8(m, s, u3);
            }
            for (; i < nvec; i += 32) ce_add_vec8(m, s, __ldg(row4 + i));
            v0 = nvec << 3;
        }
        for (int v = v0 + lane; v < cols; v += 32) ce_online_add(m, s, __bfloat162float(row[v]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
            ce_online_merge(m, s, m2, s2);
        }
        if (lane == 0) {
            row_max[r] = m;
            row_sum[r] = s;
            const int t = targets[r] - col0;
            row_tgt[r] = (t >= 0 && t < cols) ? __bfloat162float(row[t]) : 0.f;
        }
    }
}

// The same three outputs from the (max, sum) pairs that the LM-head GEMM left per row and tile (gemm_sm100.cuh,
// epilogue_store_stats): one warp per row merges the row's `np` pairs; the logits are touched only for the target.
__global__ void __launch_bounds__(CE_THREADS)
ce_merge_partials(const float2* __restrict__ partials, int np, const __nv_bfloat16* __restrict__ logits, int rows, int cols,
                  long long ld, const int* __restrict__ targets, int col0, float* __restrict__ row_max,
                  float* __restrict__ row_sum, float* __restrict__ row_tgt) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = CE_THREADS / 32;
    for (int r = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps_per_cta) {
        const float2* row = partials + static_cast<long long>(r) * np;
        float m = -INFINITY, s = 0.f;
        for (int i = lane; i < np; i += 32) {
            const float2 v = row[i];
            ce_online_merge(m, s, v.x, v.y);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
            ce_online_merge(m, s, m2, s2);
        }
        if (lane == 0) {
            row_max[r] = m;
            row_sum[r] = s;
            const int t = targets[r] - col0;
            row_tgt[r] = (t >= 0 && t < cols) ? __bfloat162float(logits[static_cast<long long>(r) * ld + t]) : 0.f;
        }
    }
}

// s_r *= exp(m_r - m): this rank's sum re-based to the global maximum (an empty shard has m_r = -inf, s_r = 0).
__global__ void ce_shard_rescale(const float* __restrict__ local_max, const float* __restrict__ global_max,
                                 float* __restrict__ row_sum, int rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) {
        const float lm = local_max[r];
        row_sum[r] = lm > -INFINITY ? row_sum[r] * __expf(lm - global_max[r]) : 0.f;
    }
}

// loss = -log softmax[target] = log s + m - l_target, per row, fp32 (cuda/crossentropy.cu:121).
__global__ void ce_shard_loss(float* __restrict__ loss, const float* __restrict__ global_max,
                              const float* __restrict__ global_sum, const float* __restrict__ target_logit, int rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) loss[r] = logf(global_sum[r]) + global_max[r] - target_logit[r];
}

__device__ __forceinline__ uint4 ce_bwd_vec8(const uint4& u, float m, float inv, int t, int c0, float scale) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float a = __expf(__uint_as_float(w[j] << 16) - m) * inv;
        float b = __expf(__uint_as_float(w[j] & 0xFFFF0000u) - m) * inv;
        if (c0 + 2 * j == t) a -= 1.0f;
        if (c0 + 2 * j + 1 == t) b -= 1.0f;
        __nv_bfloat162 p = __floats2bfloat162_rn(a * scale, b * scale);
        o[j] = *reinterpret_cast<uint32_t*>(&p);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// dlogits[r, v] = (exp(l - m_r) / s_r - [col0 + v == target_r]) * scale, bf16; may run in place.
// grid = (column chunks of 8 * CE_THREADS, rows (grid-stride)); a thread owns 8 columns and walks down the rows,
// two rows per step so that two 16-byte loads are in flight.
__global__ void __launch_bounds__(CE_THREADS)
ce_shard_backward_bf16(__nv_bfloat16* dlogits, const __nv_bfloat16* logits, int rows, int cols, long long ld,
                       const int* __restrict__ targets, int col0, const float* __restrict__ global_max,
                       const float* __restrict__ global_sum, float scale) {
    const int c0 = (blockIdx.x * CE_THREADS + threadIdx.x) * 8;
    if (c0 >= cols) return;
    const bool vec = c0 + 8 <= cols && (ld & 7) == 0 &&
                     ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15) == 0;
    const int step = gridDim.y;
    int r = blockIdx.y;
    if (vec) {
        for (; r + step < rows; r += 2 * step) {
            const int r1 = r + step;
            const uint4 u0 = *reinterpret_cast<const uint4*>(logits + static_cast<long long>(r) * ld + c0);
            const uint4 u1 = *reinterpret_cast<const uint4*>(logits + static_cast<long long>(r1) * ld + c0);
            const float m0 = global_max[r], i0 = 1.0f / global_sum[r], m1 = global_max[r1], i1 = 1.0f / global_sum[r1];
            const int t0 = targets[r] - col0, t1 = targets[r1] - col0;
            *reinterpret_cast<uint4*>(dlogits + static_cast<long long>(r) * ld + c0) = ce_bwd_vec8(u0, m0, i0, t0, c0, scale);
            *reinterpret_cast<uint4*>(dlogits + static_cast<long long>(r1) * ld + c0) = ce_bwd_vec8(u1, m1, i1, t1, c0, scale);
        }
    }
    for (; r < rows; r += step) {
        const float m = global_max[r], inv = 1.0f / global_sum[r];
        const int t = targets[r] - col0;
        const __nv_bfloat16* src = logits + static_cast<long long>(r) * ld + c0;
        __nv_bfloat16* dst = dlogits + static_cast<long long>(r) * ld + c0;
        if (vec) {
            *reinterpret_cast<uint4*>(dst) = ce_bwd_vec8(*reinterpret_cast<const uint4*>(src), m, inv, t, c0, scale);
        } else {
            for (int j = 0; j < 8 && c0 + j < cols; ++j) {
                float a = __expf(__bfloat162float(src[j]) - m) * inv;
                if (c0 + j == t) a -= 1.0f;
                dst[j] = __float2bfloat16(a * scale);
            }
        }
    }
}

}  // namespace b200
