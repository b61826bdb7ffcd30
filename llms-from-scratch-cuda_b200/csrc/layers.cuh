// Element-wise and row-wise kernels around the linear layers, for the callers of the GEMM path that this
// library also replaces: rotary embedding (cuda/rope.cu of the reference), the SwiGLU gate
// (cuda/swiglu.cu:12-47,132-155) and the whole-row softmax cross-entropy (cuda/crossentropy.cu:16-64,96-132).
// All of them are HBM-bound streaming kernels: 16-byte accesses where the row pitch allows, grids sized from
// the data, fp32 arithmetic, storage type T = float or __nv_bfloat16 with the reference's rounding points.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

#include "gemm_simt.cuh"
#include "ptx.cuh"

namespace b200 {

// ------------------------------------------------------------------------------------------------ RoPE
// One thread per (token, head of q or k, rotation pair), as cuda/rope.cu:15-57 (forward) and :63-101
// (backward: the inverse rotation), with a bounds check.  DIR = +1 forward, -1 backward.
// The rotation frequencies theta^(-2i/head_dim) are formed on the host in double precision and handed over
// rounded to fp32 (at most 64 pairs, i.e. head_dim <= 128): the angle t * freq then is one fp32 product on the device,
// which a host restatement reproduces exactly.
struct RopeFreq {
    float f[64];
};
// (cos, sin) of every (position, pair): table[t * half + i].  Built once per (T, head_dim, theta) and kept; the
// rotation kernels then are pure streaming kernels (the accurate sincosf of an angle of thousands of radians is
// far more expensive than the two loads and stores of the rotation itself).
__global__ void __launch_bounds__(256)
rope_table_kernel(float2* __restrict__ table, int Tlen, int half, const RopeFreq freqs) {
    griddep_sync();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= Tlen * half) return;
    const int t = idx / half, i = idx - t * half;
    float s, c;
    sincosf(static_cast<float>(t) * freqs.f[i], &s, &c);
    table[idx] = make_float2(c, s);
}

template <typename T, int DIR>
__global__ void __launch_bounds__(256)
rope_kernel(T* __restrict__ q, T* __restrict__ k, long long total, int Tlen, int n_head, int n_kv_head, int head_dim,
            const float2* __restrict__ table) {
    griddep_sync();
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int total_heads = n_head + n_kv_head, half = head_dim / 2;
    const int i = static_cast<int>(idx % half);
    const int h = static_cast<int>((idx / half) % total_heads);
    const long long bt = idx / (static_cast<long long>(half) * total_heads);
    const int t = static_cast<int>(bt % Tlen);
    const float2 cs = __ldg(table + t * half + i);
    const float c = cs.x;
    float s = cs.y;
    if (DIR < 0) s = -s;
    T* target = h < n_head ? q : k;
    const int heads = h < n_head ? n_head : n_kv_head, hh = h < n_head ? h : h - n_head;
    T* p = target + bt * (static_cast<long long>(heads) * head_dim) + hh * head_dim + 2 * i;
    const float x0 = to_f32<T>(p[0]), x1 = to_f32<T>(p[1]);
    p[0] = from_f32<T>(x0 * c - x1 * s);
    p[1] = from_f32<T>(x0 * s + x1 * c);
}

// ---------------------------------------------------------------------------------------------- SwiGLU
__device__ __forceinline__ float sigmoid_f(float g) { return 1.0f / (1.0f + __expf(-g)); }

// hidden = SiLU(gate) * up   (cuda/swiglu.cu:12-24, 132-140)
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_gate_kernel(T* __restrict__ hidden, const T* __restrict__ gate, const T* __restrict__ up, long long n) {
    griddep_sync();
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float g = to_f32<T>(gate[i]);
        hidden[i] = from_f32<T>(g * sigmoid_f(g) * to_f32<T>(up[i]));
    }
}
// dup = dhidden * SiLU(gate);  dgate = dhidden * up * SiLU'(gate)   (cuda/swiglu.cu:27-47, 142-155)
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_gate_backward_kernel(T* __restrict__ dgate, T* __restrict__ dup, const T* __restrict__ dhidden,
                            const T* __restrict__ gate, const T* __restrict__ up, long long n) {
    griddep_sync();
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float g = to_f32<T>(gate[i]), u = to_f32<T>(up[i]), dh = to_f32<T>(dhidden[i]);
        const float sig = sigmoid_f(g);
        dup[i] = from_f32<T>(dh * (g * sig));
        dgate[i] = from_f32<T>(dh * u * (sig * (1.0f + g * (1.0f - sig))));
    }
}
// Eight bf16 values per thread: 16-byte loads and stores (n a multiple of 8, pointers 16-byte aligned).
__global__ void __launch_bounds__(256)
swiglu_gate_kernel_bf16x8(uint4* __restrict__ hidden, const uint4* __restrict__ gate, const uint4* __restrict__ up,
                          long long n8) {
    griddep_sync();
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const uint4 gv = gate[i], uv = up[i];
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xFFFF0000u);
            const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xFFFF0000u);
            __nv_bfloat162 r = __floats2bfloat162_rn(g0 * sigmoid_f(g0) * u0, g1 * sigmoid_f(g1) * u1);
            o[j] = *reinterpret_cast<uint32_t*>(&r);
        }
        hidden[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}
__global__ void __launch_bounds__(256)
swiglu_gate_backward_kernel_bf16x8(uint4* __restrict__ dgate, uint4* __restrict__ dup, const uint4* __restrict__ dhidden,
                                   const uint4* __restrict__ gate, const uint4* __restrict__ up, long long n8) {
    griddep_sync();
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const uint4 gv = gate[i], uv = up[i], dv = dhidden[i];
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w}, dw[4] = {dv.x, dv.y, dv.z, dv.w};
        uint32_t og[4], ou[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float g[2] = {__uint_as_float(gw[j] << 16), __uint_as_float(gw[j] & 0xFFFF0000u)};
            float u[2] = {__uint_as_float(uw[j] << 16), __uint_as_float(uw[j] & 0xFFFF0000u)};
            float d[2] = {__uint_as_float(dw[j] << 16), __uint_as_float(dw[j] & 0xFFFF0000u)};
            float rg[2], ru[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float sig = sigmoid_f(g[e]);
                ru[e] = d[e] * (g[e] * sig);
                rg[e] = d[e] * u[e] * (sig * (1.0f + g[e] * (1.0f - sig)));
            }
            __nv_bfloat162 a = __floats2bfloat162_rn(rg[0], rg[1]), b = __floats2bfloat162_rn(ru[0], ru[1]);
            og[j] = *reinterpret_cast<uint32_t*>(&a);
            ou[j] = *reinterpret_cast<uint32_t*>(&b);
        }
        dgate[i] = make_uint4(og[0], og[1], og[2], og[3]);
        dup[i] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
    }
}

// ------------------------------------------------------------------------------- whole-row cross-entropy
// One CTA per row (grid-stride over rows).  Same arithmetic and rounding points as the reference's
// one-thread-per-row kernels (cuda/crossentropy.cu:16-46 fp32, :96-122 bf16): maximum; e = exp(l - max)
// stored in place in the storage type while the sum adds the unrounded e; p = stored e / sum, stored in
// place; loss = -log(stored p[target]).  Only the order of the fp32 additions differs (a tree instead of a
// serial loop).  The row is read from HBM once and written once; the second and third passes hit L2.
constexpr int CE_ROW_THREADS = 512;

// fp32 storage: the accurate exponential; bf16 storage: the fast one (its error is far below a bf16 ulp)
template <typename T> __device__ __forceinline__ float ce_exp(float x) { return sizeof(T) == 4 ? expf(x) : __expf(x); }

__device__ __forceinline__ float ce_block_reduce(float v, float* sh, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, w) : v + w;
    }
    __syncthreads();  // sh may still be read from the previous reduction
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    v = threadIdx.x < (CE_ROW_THREADS / 32) ? sh[threadIdx.x] : (is_max ? -INFINITY : 0.f);
    if (warp == 0) {
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            const float w = __shfl_xor_sync(0xffffffffu, v, o);
            v = is_max ? fmaxf(v, w) : v + w;
        }
        if (lane == 0) sh[0] = v;
    }
    __syncthreads();
    return sh[0];
}

template <typename T>
__global__ void __launch_bounds__(CE_ROW_THREADS)
ce_row_forward(float* __restrict__ losses, T* probs, const int* __restrict__ targets, int rows, long long V) {
    griddep_sync();
    __shared__ float sh[CE_ROW_THREADS / 32];
    constexpr int VEC = 16 / sizeof(T);  // elements per 16-byte access
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        T* row = probs + static_cast<long long>(r) * V;
        const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
        const long long nvec = vec ? V / VEC : 0;
        uint4* row4 = reinterpret_cast<uint4*>(row);
        auto unpack = [](const uint4& u, float (&x)[VEC]) {
            if constexpr (sizeof(T) == 2) {
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    x[2 * j] = __uint_as_float(w[j] << 16);
                    x[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
                }
            } else {
                x[0] = __uint_as_float(u.x); x[1] = __uint_as_float(u.y); x[2] = __uint_as_float(u.z); x[3] = __uint_as_float(u.w);
            }
        };
        auto pack = [](const float (&x)[VEC]) {
            if constexpr (sizeof(T) == 2) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 p = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
                    w[j] = *reinterpret_cast<uint32_t*>(&p);
                }
                return make_uint4(w[0], w[1], w[2], w[3]);
            } else {
                return make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3]));
            }
        };
        // pass 1: maximum
        float m = -INFINITY;
        for (long long i = threadIdx.x; i < nvec; i += CE_ROW_THREADS) {
            float x[VEC];
            unpack(row4[i], x);
#pragma unroll
            for (int j = 0; j < VEC; ++j) m = fmaxf(m, x[j]);
        }
        for (long long v = nvec * VEC + threadIdx.x; v < V; v += CE_ROW_THREADS) m = fmaxf(m, to_f32<T>(row[v]));
        m = ce_block_reduce(m, sh, true);
        // pass 2: exponentials, stored in place in the storage type; the sum takes them unrounded
        float s = 0.f;
        for (long long i = threadIdx.x; i < nvec; i += CE_ROW_THREADS) {
            float x[VEC];
            unpack(row4[i], x);
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                x[j] = ce_exp<T>(x[j] - m);
                s += x[j];
            }
            row4[i] = pack(x);
        }
        for (long long v = nvec * VEC + threadIdx.x; v < V; v += CE_ROW_THREADS) {
            const float e = ce_exp<T>(to_f32<T>(row[v]) - m);
            row[v] = from_f32<T>(e);
            s += e;
        }
        s = ce_block_reduce(s, sh, false);  // its barriers also order pass 2's stores before pass 3's loads
        // pass 3: normalise the stored values
        for (long long i = threadIdx.x; i < nvec; i += CE_ROW_THREADS) {
            float x[VEC];
            unpack(row4[i], x);
#pragma unroll
            for (int j = 0; j < VEC; ++j) x[j] = x[j] / s;
            row4[i] = pack(x);
        }
        for (long long v = nvec * VEC + threadIdx.x; v < V; v += CE_ROW_THREADS) row[v] = from_f32<T>(to_f32<T>(row[v]) / s);
        __syncthreads();
        if (threadIdx.x == 0) losses[r] = sizeof(T) == 4 ? -logf(to_f32<T>(row[targets[r]])) : -__logf(to_f32<T>(row[targets[r]]));
    }
}

// dlogits = (probs - onehot) * scale   (cuda/crossentropy.cu:50-64, 124-132); may run in place.
template <typename T>
__global__ void __launch_bounds__(256)
ce_row_backward(T* dlogits, const T* probs, const int* __restrict__ targets, float scale, int rows, long long V) {
    griddep_sync();
    const long long n = static_cast<long long>(rows) * V;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long r = i / V;
        const int v = static_cast<int>(i - r * V);
        dlogits[i] = from_f32<T>((to_f32<T>(probs[i]) - (v == targets[r] ? 1.0f : 0.0f)) * scale);
    }
}
// bf16, V a multiple of 8, 16-byte aligned: eight columns per thread.
__global__ void __launch_bounds__(256)
ce_row_backward_bf16x8(uint4* dlogits, const uint4* probs, const int* __restrict__ targets, float scale, int rows,
                       long long V8) {
    griddep_sync();
    const long long n = static_cast<long long>(rows) * V8;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long r = i / V8;
        const int c0 = static_cast<int>(i - r * V8) * 8;
        const int t = targets[r] - c0;
        const uint4 u = probs[i];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float a = __uint_as_float(w[j] << 16), b = __uint_as_float(w[j] & 0xFFFF0000u);
            if (t == 2 * j) a -= 1.0f;
            if (t == 2 * j + 1) b -= 1.0f;
            __nv_bfloat162 p = __floats2bfloat162_rn(a * scale, b * scale);
            o[j] = *reinterpret_cast<uint32_t*>(&p);
        }
        dlogits[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace b200

namespace b200 {

// ---------------------------------------------------------------------------------------------- RMSNorm
// out = x * rsqrt(mean(x^2) + eps) * weight, rrms = the rsqrt (cuda/rmsnorm.cu:5-35, 107-133): one warp per row.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(T* __restrict__ out, float* __restrict__ rrms, const T* __restrict__ inp, const T* __restrict__ weight,
                   float eps, int rows, int C) {
    griddep_sync();
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const T* x = inp + static_cast<long long>(r) * C;
        float ss = 0.f;
        for (int j = lane; j < C; j += 32) {
            const float v = to_f32<T>(x[j]);
            ss = fmaf(v, v, ss);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss / static_cast<float>(C) + eps);
        if (lane == 0) rrms[r] = inv;
        T* y = out + static_cast<long long>(r) * C;
        for (int j = lane; j < C; j += 32) y[j] = from_f32<T>(to_f32<T>(x[j]) * inv * to_f32<T>(weight[j]));
    }
}

// dinp = rrms * (w dy - x rrms^2 sum_j(dy_j w_j x_j) / C)   (cuda/rmsnorm.cu:37-73, 135-166): one warp per row.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dinp_kernel(T* __restrict__ dinp, const T* __restrict__ dout, const T* __restrict__ inp,
                        const T* __restrict__ weight, const float* __restrict__ rrms, int rows, int C) {
    griddep_sync();
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const T* x = inp + static_cast<long long>(r) * C;
        const T* dy = dout + static_cast<long long>(r) * C;
        float s = 0.f;
        for (int j = lane; j < C; j += 32) s += to_f32<T>(dy[j]) * to_f32<T>(weight[j]) * to_f32<T>(x[j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float inv = rrms[r];
        const float k = inv * inv * s / static_cast<float>(C);
        T* dx = dinp + static_cast<long long>(r) * C;
        for (int j = lane; j < C; j += 32)
            dx[j] = from_f32<T>(inv * (to_f32<T>(dy[j]) * to_f32<T>(weight[j]) - to_f32<T>(x[j]) * k));
    }
}

// dweight_j += sum_rows dy_j x_j rrms: the reference adds row by row with one atomic per element (a compare-and-swap
// loop on bf16, 8192 contenders per word).  Here: partial[chunk][j] = the sum over one chunk of rows (a thread per
// column, coalesced over j), then rmsnorm_bwd_dw_reduce adds the chunks in a fixed order onto the stored gradient, rounding once.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dw_partial_kernel(float* __restrict__ partial, const T* __restrict__ dout, const T* __restrict__ inp,
                              const float* __restrict__ rrms, int rows, int C, int rows_per_chunk) {
    griddep_sync();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= C) return;
    const int r0 = blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
    float s = 0.f;
    for (int r = r0; r < r1; ++r)
        s += to_f32<T>(dout[static_cast<long long>(r) * C + j]) * to_f32<T>(inp[static_cast<long long>(r) * C + j]) * rrms[r];
    partial[static_cast<long long>(blockIdx.y) * C + j] = s;
}

}  // namespace b200

namespace b200 {

// --------------------------------------------------------------------------------------- residual add
// out = a + b (cuda/residual.cu:9-16, 52-57; out may alias a) and da += dout, db += dout (:22-29, 59-66), 16 bytes per
// thread and array where the length and the pointers allow, one element per thread otherwise.
__device__ __forceinline__ uint4 bf16x8_add(const uint4& x, const uint4& y) {
    const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 r = __floats2bfloat162_rn(__uint_as_float(xw[j] << 16) + __uint_as_float(yw[j] << 16),
                                                 __uint_as_float(xw[j] & 0xFFFF0000u) + __uint_as_float(yw[j] & 0xFFFF0000u));
        o[j] = *reinterpret_cast<uint32_t*>(&r);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
__device__ __forceinline__ uint4 f32x4_add(const uint4& x, const uint4& y) {
    return make_uint4(__float_as_uint(__uint_as_float(x.x) + __uint_as_float(y.x)), __float_as_uint(__uint_as_float(x.y) + __uint_as_float(y.y)),
                      __float_as_uint(__uint_as_float(x.z) + __uint_as_float(y.z)), __float_as_uint(__uint_as_float(x.w) + __uint_as_float(y.w)));
}
template <typename T>
__global__ void __launch_bounds__(256)
residual_forward_vec(uint4* out, const uint4* a, const uint4* b, long long nvec) {
    griddep_sync();
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride)
        out[i] = sizeof(T) == 2 ? bf16x8_add(a[i], b[i]) : f32x4_add(a[i], b[i]);
}
template <typename T>
__global__ void __launch_bounds__(256)
residual_backward_vec(uint4* da, uint4* db, const uint4* dout, long long nvec) {
    griddep_sync();
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 d = dout[i];
        da[i] = sizeof(T) == 2 ? bf16x8_add(da[i], d) : f32x4_add(da[i], d);
        db[i] = sizeof(T) == 2 ? bf16x8_add(db[i], d) : f32x4_add(db[i], d);
    }
}
template <typename T>
__global__ void __launch_bounds__(256)
residual_forward_scalar(T* out, const T* a, const T* b, long long n0, long long n) {
    griddep_sync();
    const long long i = n0 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(to_f32<T>(a[i]) + to_f32<T>(b[i]));
}
template <typename T>
__global__ void __launch_bounds__(256)
residual_backward_scalar(T* da, T* db, const T* dout, long long n0, long long n) {
    griddep_sync();
    const long long i = n0 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) {
        const float d = to_f32<T>(dout[i]);
        da[i] = from_f32<T>(to_f32<T>(da[i]) + d);
        db[i] = from_f32<T>(to_f32<T>(db[i]) + d);
    }
}

// RoPE on bf16, eight elements (four rotation pairs) per thread; head_dim a multiple of 8, 16-byte aligned rows.
template <int DIR>
__global__ void __launch_bounds__(256)
rope_kernel_bf16x8(uint4* __restrict__ q, uint4* __restrict__ k, long long total_vec, int Tlen, int n_head, int n_kv_head,
                   int head_dim, const float2* __restrict__ table) {
    griddep_sync();
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_vec) return;
    const int vec_per_head = head_dim / 8, total_heads = n_head + n_kv_head, half = head_dim / 2;
    const int vi = static_cast<int>(idx % vec_per_head);
    const int h = static_cast<int>((idx / vec_per_head) % total_heads);
    const long long bt = idx / (static_cast<long long>(vec_per_head) * total_heads);
    const int t = static_cast<int>(bt % Tlen);
    uint4* target = h < n_head ? q : k;
    const int heads = h < n_head ? n_head : n_kv_head, hh = h < n_head ? h : h - n_head;
    uint4* p = target + (bt * heads + hh) * vec_per_head + vi;
    const uint4 u = *p;
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 cs = __ldg(table + t * half + vi * 4 + j);
        const float c = cs.x, s = DIR < 0 ? -cs.y : cs.y;
        const float x0 = __uint_as_float(w[j] << 16), x1 = __uint_as_float(w[j] & 0xFFFF0000u);
        __nv_bfloat162 r = __floats2bfloat162_rn(x0 * c - x1 * s, x0 * s + x1 * c);
        o[j] = *reinterpret_cast<uint32_t*>(&r);
    }
    *p = make_uint4(o[0], o[1], o[2], o[3]);
}

// RMSNorm on bf16 with 16-byte accesses (C a multiple of 8, 16-byte aligned rows): one warp per row, the row kept in
// registers between the reduction and the output (up to 32 * 8 * RMS_VEC_MAX = 2048 columns; wider rows take the
// generic kernels).
constexpr int RMS_VEC_MAX = 8;
__device__ __forceinline__ void bf16x8_unpack(const uint4& u, float (&x)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        x[2 * j] = __uint_as_float(w[j] << 16);
        x[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint4 bf16x8_pack(const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 r = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&r);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
__global__ void __launch_bounds__(256)
rmsnorm_fwd_bf16x8(uint4* __restrict__ out, float* __restrict__ rrms, const uint4* __restrict__ inp,
                   const uint4* __restrict__ weight, float eps, int rows, int C) {
    griddep_sync();
    const int lane = threadIdx.x & 31, nvec = C / 8;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const uint4* x4 = inp + static_cast<long long>(r) * nvec;
        uint4 xv[RMS_VEC_MAX];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < RMS_VEC_MAX; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                xv[i] = x4[v];
                float x[8];
                bf16x8_unpack(xv[i], x);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss / static_cast<float>(C) + eps);
        if (lane == 0) rrms[r] = inv;
        uint4* y4 = out + static_cast<long long>(r) * nvec;
#pragma unroll
        for (int i = 0; i < RMS_VEC_MAX; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                float x[8], w[8];
                bf16x8_unpack(xv[i], x);
                bf16x8_unpack(__ldg(weight + v), w);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = x[e] * inv * w[e];
                y4[v] = bf16x8_pack(x);
            }
        }
    }
}
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dinp_bf16x8(uint4* __restrict__ dinp, const uint4* __restrict__ dout, const uint4* __restrict__ inp,
                        const uint4* __restrict__ weight, const float* __restrict__ rrms, int rows, int C) {
    griddep_sync();
    const int lane = threadIdx.x & 31, nvec = C / 8;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const uint4* x4 = inp + static_cast<long long>(r) * nvec;
        const uint4* d4 = dout + static_cast<long long>(r) * nvec;
        uint4 xv[RMS_VEC_MAX], dv[RMS_VEC_MAX];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < RMS_VEC_MAX; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                xv[i] = x4[v];
                dv[i] = d4[v];
                float x[8], d[8], w[8];
                bf16x8_unpack(xv[i], x);
                bf16x8_unpack(dv[i], d);
                bf16x8_unpack(__ldg(weight + v), w);
#pragma unroll
                for (int e = 0; e < 8; ++e) s += d[e] * w[e] * x[e];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float inv = rrms[r];
        const float kk = inv * inv * s / static_cast<float>(C);
        uint4* o4 = dinp + static_cast<long long>(r) * nvec;
#pragma unroll
        for (int i = 0; i < RMS_VEC_MAX; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                float x[8], d[8], w[8];
                bf16x8_unpack(xv[i], x);
                bf16x8_unpack(dv[i], d);
                bf16x8_unpack(__ldg(weight + v), w);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = inv * (d[e] * w[e] - x[e] * kk);
                o4[v] = bf16x8_pack(x);
            }
        }
    }
}


// dinp and this block's share of dweight in one pass over dout and inp (bf16, 16-byte accesses): every warp walks its
// rows, keeps sum_rows dy_j x_j rrms for its own columns in registers, the block's eight warps add theirs up in shared
// memory in warp order, and partial[block][j] goes to rmsnorm_bwd_dw_reduce (fixed order: run-to-run identical).
template <int NV>   // 16-byte vectors per lane: C <= NV * 256
__global__ void __launch_bounds__(256)
rmsnorm_bwd_fused_bf16x8(uint4* __restrict__ dinp, float* __restrict__ partial, const uint4* __restrict__ dout,
                         const uint4* __restrict__ inp, const uint4* __restrict__ weight, const float* __restrict__ rrms,
                         int rows, int C) {
    griddep_sync();
    __shared__ float sh[NV * 256];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nvec = C / 8;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    float dw[NV][8];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) dw[i][e] = 0.f;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const uint4* x4 = inp + static_cast<long long>(r) * nvec;
        const uint4* d4 = dout + static_cast<long long>(r) * nvec;
        uint4 xv[NV], dv[NV];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                xv[i] = x4[v];
                dv[i] = d4[v];
                float x[8], d[8], w[8];
                bf16x8_unpack(xv[i], x);
                bf16x8_unpack(dv[i], d);
                bf16x8_unpack(__ldg(weight + v), w);
#pragma unroll
                for (int e = 0; e < 8; ++e) s += d[e] * w[e] * x[e];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float inv = rrms[r];
        const float kk = inv * inv * s / static_cast<float>(C);
        uint4* o4 = dinp + static_cast<long long>(r) * nvec;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                float x[8], d[8], w[8];
                bf16x8_unpack(xv[i], x);
                bf16x8_unpack(dv[i], d);
                bf16x8_unpack(__ldg(weight + v), w);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    dw[i][e] = fmaf(d[e] * x[e], inv, dw[i][e]);
                    x[e] = inv * (d[e] * w[e] - x[e] * kk);
                }
                o4[v] = bf16x8_pack(x);
            }
        }
    }
    for (int turn = 0; turn < 8; ++turn) {
        if (wid == turn) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int v = lane + 32 * i;
                if (v < nvec) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) sh[v * 8 + e] = (turn == 0 ? 0.f : sh[v * 8 + e]) + dw[i][e];
                }
            }
        }
        __syncthreads();
    }
    for (int j = threadIdx.x; j < C; j += 256) partial[static_cast<long long>(blockIdx.x) * C + j] = sh[j];
}
// dweight_j += sum over `chunks` partial rows, in the order 0, 8, 16, ... | 1, 9, ... per warp and then warp 0..7: a block
// per 32 columns, lane = column.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dw_reduce(T* __restrict__ dweight, const float* __restrict__ partial, int chunks, int C) {
    griddep_sync();
    __shared__ float sh[8][32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int j = blockIdx.x * 32 + lane;
    float s = 0.f;
    if (j < C)
        for (int c = wid; c < chunks; c += 8) s += partial[static_cast<long long>(c) * C + j];
    sh[wid][lane] = s;
    __syncthreads();
    if (wid == 0 && j < C) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += sh[w][lane];
        dweight[j] = from_f32<T>(to_f32<T>(dweight[j]) + t);
    }
}

// delta[b, h, t] = sum_d dcontext[t, h, d] * context[t, h, d] for head dimension 64, bf16, 16 bytes per lane: a warp
// covers four heads of one token per pass (eight lanes per head).
__global__ void __launch_bounds__(256)
attn_delta_bf16x8(float* __restrict__ delta, const uint4* __restrict__ dcontext, const uint4* __restrict__ context, int B,
                  int Tlen, int n_head) {
    griddep_sync();
    const int lane = threadIdx.x & 31;
    const long long rows = static_cast<long long>(B) * Tlen;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    const int nvec = n_head * 8;   // 16-byte vectors per token
    for (long long bt = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; bt < rows; bt += warps) {
        const int b = static_cast<int>(bt / Tlen), t = static_cast<int>(bt % Tlen);
        for (int v0 = 0; v0 < nvec; v0 += 32) {
            const int v = v0 + lane;
            float s = 0.f;
            if (v < nvec) {
                float x[8], y[8];
                bf16x8_unpack(dcontext[bt * nvec + v], x);
                bf16x8_unpack(context[bt * nvec + v], y);
#pragma unroll
                for (int e = 0; e < 8; ++e) s = fmaf(x[e], y[e], s);
            }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            const int h = v >> 3;
            if ((lane & 7) == 0 && v < nvec) delta[(static_cast<long long>(b) * n_head + h) * Tlen + t] = s;
        }
    }
}

}  // namespace b200

namespace b200 {

// ------------------------------------------------------------------------------ optimizer (cuda/adamw.cu)
// AdamW exactly as the reference writes it (adamw.cu:12-40 fp32, :63-88 mixed precision), one element per thread;
// it is already at the HBM roof.  The gradient norm (adamw.cu:101-191) is where the reference loses time: one
// atomicAdd per 256-element block onto a single word.  Here: per-CTA partial sums, then one CTA adds them in a fixed
// order.  The bf16 variant zeroes non-finite and > 65000 entries in place, as the reference does.
__global__ void __launch_bounds__(256)
adamw_kernel_f32(float* params, const float* grads, float* m, float* v, float lr, float beta1, float beta2, float eps,
                 float weight_decay, float bc1, float bc2, long long n) {
    griddep_sync();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = grads[i], p = params[i];
    const float mi = beta1 * m[i] + (1.0f - beta1) * g;
    const float vi = beta2 * v[i] + (1.0f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    params[i] = p - lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + weight_decay * p);
}
__global__ void __launch_bounds__(256)
adamw_kernel_bf16(__nv_bfloat16* params, float* master, const __nv_bfloat16* grads, float* m, float* v, float lr, float beta1,
                  float beta2, float eps, float weight_decay, float grad_scale, float bc1, float bc2, long long n) {
    griddep_sync();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = __bfloat162float(grads[i]) * grad_scale;
    float p = master[i];
    const float mi = beta1 * m[i] + (1.0f - beta1) * g;
    const float vi = beta2 * v[i] + (1.0f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p -= lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + weight_decay * p);
    master[i] = p;
    params[i] = __float2bfloat16(p);
}
__global__ void __launch_bounds__(256) scale_kernel_f32(float* data, float scale, long long n) {
    griddep_sync();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) data[i] *= scale;
}
__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* src, __nv_bfloat16* dst, long long n) {
    griddep_sync();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __float2bfloat16(src[i]);
}

__device__ __forceinline__ float block_sum_256(float v, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    v = threadIdx.x < 8 ? sh[threadIdx.x] : 0.f;
    if (threadIdx.x < 32) {
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;  // valid in thread 0
}
// partial[blockIdx.x] = sum over this CTA's grid-stride share of (g * scale)^2
__global__ void __launch_bounds__(256)
sumsq_partial_f32(float* __restrict__ partial, const float* __restrict__ g, float scale, long long n) {
    griddep_sync();
    __shared__ float sh[8];
    float s = 0.f;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float x = g[i] * scale;
        s = fmaf(x, x, s);
    }
    s = block_sum_256(s, sh);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void __launch_bounds__(256)
sumsq_sanitize_partial_bf16(float* __restrict__ partial, __nv_bfloat16* g, float scale, long long n) {
    griddep_sync();
    __shared__ float sh[8];
    float s = 0.f;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float x = __bfloat162float(g[i]) * scale;
        if (x != x || fabsf(x) > 65000.0f) g[i] = __float2bfloat16(0.0f);   // adamw.cu:133-135
        else s = fmaf(x, x, s);
    }
    s = block_sum_256(s, sh);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// out[0] = sum of the n partial sums, in order
__global__ void __launch_bounds__(256) sum_partials(float* __restrict__ out, const float* __restrict__ partial, int n) {
    griddep_sync();
    __shared__ float sh[8];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) s += partial[i];
    s = block_sum_256(s, sh);
    if (threadIdx.x == 0) out[0] = s;
}

}  // namespace b200
