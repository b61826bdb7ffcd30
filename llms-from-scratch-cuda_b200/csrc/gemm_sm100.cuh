// Persistent, warp-specialised bf16 GEMM for sm_100a:
//   TMA -> 128B-swizzled shared-memory ring -> tcgen05.mma (fp32 accumulators in
//   TMEM, double-buffered) -> epilogue warps (tcgen05.ld, fused beta=1 add and
//   bf16 down-cast, or fp32 split-K partials).
//
// One kernel template covers the three GEMMs of the reference's linear layer
// (cuda/matmul.cu:55-104 of the reference) by describing every product as
//     D[Mo, No] = sum_c  P[Mo, c] * Q[No, c]
// where each operand is either "K-major" (the contraction index c is the
// contiguous one in global memory) or "MN-major" (the output index is):
//     forward  C  = A  * B     : P = A  (K-major),  Q = B  (MN-major)   "NN"
//     dgrad    dA = dC * B^T   : P = dC (K-major),  Q = B  (K-major)    "NT"
//     wgrad    dB += A^T * dC  : P = A  (MN-major), Q = dC (MN-major)   "TN"
//
// CTAS = 1: one CTA per 128 x BN tile.
// CTAS = 2: a cluster of two CTAs per 256 x BN tile (tcgen05 cta_group::2).  Each CTA
//           loads its own 128 rows of P and its own BN/2 rows of Q (no multicast), the
//           even CTA issues the MMAs for both, each CTA drains its own 128 x BN
//           accumulator from its own TMEM.
#pragma once
#include <cuda_bf16.h>
#include "ptx.cuh"

namespace b200 {

constexpr int BM = 128;        // output rows per CTA = TMEM lanes
constexpr int BK = 64;         // contraction elements per stage = one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;     // contraction elements per tcgen05.mma (bf16)
constexpr int GEMM_THREADS = 256;
constexpr int SMEM_BUDGET = 227 * 1024;

enum EpilogueKind : int {
    EPI_BF16 = 0,        // out_bf16 = rn(acc)
    EPI_BF16_BETA1 = 1,  // out_bf16 = rn(acc + float(out_bf16))
    EPI_F32_PARTIAL = 2  // workspace_f32[split] = acc   (split-K; reduced by a second kernel)
};

struct GemmParams {
    int Mo, No, Kc;          // output rows, output cols, contraction length
    int m_tiles, n_tiles;    // ceil(Mo/(BM*CTAS)), ceil(No/BN)
    int splits;              // split-K factor (1 = none)
    int kb_total;            // ceil(Kc/BK)
    int kb_per_split;        // ceil(kb_total/splits); every split owns >= 1 block
    int m_fastest;           // tile raster: 1 = consecutive tiles walk down the rows
    void* out;               // bf16 [Mo,No] or fp32 workspace [splits,Mo,No]
    int* status;             // device status word (0 = ok)
};

template <int BN, int CTAS>
struct TileCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_ROWS = BN / CTAS;           // rows of Q this CTA loads
    static constexpr int B_BYTES = B_ROWS * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int CTRL_BYTES = 1024;
    static constexpr int STAGES_RAW = (SMEM_BUDGET - CTRL_BYTES - 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + CTRL_BYTES + 1024;  // +1024: manual alignment
    static constexpr int ACC_STRIDE = BN <= 64 ? 64 : (BN <= 128 ? 128 : 256);   // TMEM columns per accumulator
    static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "tile width");
    static_assert(CTAS == 1 || (CTAS == 2 && B_ROWS % 64 == 0), "pair tiles split Q in 64-row panels");
    static_assert(STAGES >= 3, "pipeline too shallow");
};

struct TileCoord {
    int m_blk, n_blk, split;
};
__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int t) {
    TileCoord c;
    const int per_split = p.m_tiles * p.n_tiles;
    c.split = t / per_split;
    const int r = t - c.split * per_split;
    if (p.m_fastest) {
        c.n_blk = r / p.m_tiles;
        c.m_blk = r - c.n_blk * p.m_tiles;
    } else {
        c.m_blk = r / p.n_tiles;
        c.n_blk = r - c.m_blk * p.n_tiles;
    }
    return c;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Control block at the start of the (1024-byte aligned) dynamic shared memory.
struct alignas(8) GemmCtrl {
    unsigned long long full[8];        // TMA -> MMA: stage filled (pair: the even CTA's counts both CTAs' bytes)
    unsigned long long empty[8];       // MMA -> TMA: stage consumed
    unsigned long long tmem_full[2];   // MMA -> epilogue: accumulator finished
    unsigned long long tmem_empty[2];  // epilogue -> MMA: accumulator drained (pair: lives in the even CTA)
    uint32_t tmem_base;
    int abort_flag;
};

// Drain one 128 x BN fp32 accumulator (this warp's 32 lanes) to global memory.
template <int BN, int EPI>
__device__ __forceinline__ void epilogue_store(const GemmParams& p, uint32_t taddr, int row, int n0,
                                               int split) {
    const bool row_ok = row < p.Mo;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if constexpr (EPI == EPI_F32_PARTIAL) {
            float* dst = reinterpret_cast<float*>(p.out) + (static_cast<size_t>(split) * p.Mo + row) * p.No + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (row_ok && col0 + 4 * j < p.No)
                    *reinterpret_cast<uint4*>(dst + 4 * j) =
                        make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.No + col0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (row_ok && col0 + 8 * j < p.No) {
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[8 * j + e]);
                    if constexpr (EPI == EPI_BF16_BETA1) {
                        const uint4 o = *reinterpret_cast<const uint4*>(dst + 8 * j);
                        v[0] += bf16_lo(o.x); v[1] += bf16_hi(o.x);
                        v[2] += bf16_lo(o.y); v[3] += bf16_hi(o.y);
                        v[4] += bf16_lo(o.z); v[5] += bf16_hi(o.z);
                        v[6] += bf16_lo(o.w); v[7] += bf16_hi(o.w);
                    }
                    *reinterpret_cast<uint4*>(dst + 8 * j) =
                        make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                   pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
                }
            }
        }
    }
}

// Warp roles: 0 = TMA producer, 1 = MMA issuer (even CTA only in a pair), 2 = TMEM allocator,
// 3 = idle, 4..7 = epilogue (warp w owns TMEM lanes 32*(w-4) .. +31).
template <int BN, bool P_MN, bool Q_MN, int EPI, int CTAS>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_sm100(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                const GemmParams p) {
    using Cfg = TileCfg<BN, CTAS>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr bool PAIR = CTAS == 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    GemmCtrl* ctrl = reinterpret_cast<GemmCtrl*>(smem);
    uint8_t* tiles = smem + Cfg::CTRL_BYTES;  // stage s: [P tile | Q tile]
    volatile int* abort_flag = &ctrl->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // position in the CTA pair
    const int total_tiles = p.m_tiles * p.n_tiles * p.splits;
    const int first_tile = blockIdx.x / CTAS, tile_step = gridDim.x / CTAS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->full[s]), 1);
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctrl->tmem_full[a]), 1);
            mbar_init(smem_u32(&ctrl->tmem_empty[a]), 4 * CTAS);
        }
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmP);
        tma_prefetch_desc(&tmQ);
    }
    if (warp == 2) {
        tmem_alloc<CTAS>(smem_u32(&ctrl->tmem_base), Cfg::TMEM_COLS);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) {  // the partner's barriers must exist before anything signals them
        cluster_arrive_release();
        cluster_wait_acquire();
    }
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t issued = 0;  // number of stage fills issued so far
            bool ok = true;
            for (int t = first_tile; t < total_tiles && ok; t += tile_step) {
                const TileCoord tc = decode_tile(p, t);
                const int kb0 = tc.split * p.kb_per_split;
                const int kb1 = min(kb0 + p.kb_per_split, p.kb_total);
                const int m0 = (tc.m_blk * CTAS + static_cast<int>(rank)) * BM;
                const int n0 = tc.n_blk * BN + static_cast<int>(rank) * Cfg::B_ROWS;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_flag, p.status,
                                   DEV_TIMEOUT_EMPTY)) {
                        ok = false;
                        break;
                    }
                    const uint32_t local_bar = smem_u32(&ctrl->full[stage]);
                    const uint32_t bar = PAIR ? map_to_cta(local_bar, 0) : local_bar;
                    const uint32_t sP = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
                    const uint32_t sQ = sP + Cfg::A_BYTES;
                    if (rank == 0) mbar_arrive_expect_tx(local_bar, CTAS * Cfg::STAGE_BYTES);
                    const int c0 = kb * BK;
                    auto load = [&](uint32_t dst, const CUtensorMap* tm, int x, int y) {
                        if constexpr (PAIR) tma_load_2d_pair(dst, tm, bar, x, y);
                        else tma_load_2d(dst, tm, bar, x, y);
                    };
                    if constexpr (P_MN) {  // global [Kc][Mo]: box = 64 output rows x BK contraction rows
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) load(sP + j * (64 * BK * 2), &tmP, m0 + 64 * j, c0);
                    } else {               // global [Mo][Kc]: box = BK contraction x BM rows
                        load(sP, &tmP, c0, m0);
                    }
                    if constexpr (Q_MN) {
#pragma unroll
                        for (int j = 0; j < Cfg::B_ROWS / 64; ++j) load(sQ + j * (64 * BK * 2), &tmQ, n0 + 64 * j, c0);
                    } else {
                        load(sQ, &tmQ, c0, n0);
                    }
                    ++issued;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok && rank == 0) {
                // Abort path: let every copy counted on this CTA's barriers land before exit.
                const uint32_t n_back = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
                uint32_t s = stage, ph = phase;
                for (uint32_t i = 0; i < n_back; ++i) {
                    if (s == 0) { s = STAGES; ph ^= 1; }
                    --s;
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&ctrl->full[s]), ph)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES / 8) {
                            atomicCAS(p.status, 0, DEV_TIMEOUT_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc(1, BM * CTAS, BN, P_MN ? 1 : 0, Q_MN ? 1 : 0);
            // K-major tile: rows of 128 B, 8-row groups 1024 B apart; +32 B per UMMA_K step.
            // MN-major tile: 64-wide column panels of BK rows x 128 B (LBO = panel pitch),
            //                8-row groups 1024 B apart (SBO); +16 rows = 2048 B per UMMA_K step.
            constexpr uint32_t P_LBO = P_MN ? 64 * BK * 2 : 16, P_STEP = P_MN ? UMMA_K * 128 : UMMA_K * 2;
            constexpr uint32_t Q_LBO = Q_MN ? 64 * BK * 2 : 16, Q_STEP = Q_MN ? UMMA_K * 128 : UMMA_K * 2;
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            for (int t = first_tile; t < total_tiles && ok; t += tile_step, ++it) {
                const TileCoord tc = decode_tile(p, t);
                const int kb0 = tc.split * p.kb_per_split;
                const int kb1 = min(kb0 + p.kb_per_split, p.kb_total);
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                if (!mbar_wait<PAIR>(smem_u32(&ctrl->tmem_empty[acc]), acc_phase ^ 1, abort_flag, p.status,
                                     DEV_TIMEOUT_TMEM_E)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&ctrl->full[stage]), phase, abort_flag, p.status,
                                   DEV_TIMEOUT_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sP = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
                    const uint32_t sQ = sP + Cfg::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t dP = umma_smem_desc(sP + k * P_STEP, P_LBO, 1024);
                        const uint64_t dQ = umma_smem_desc(sQ + k * Q_STEP, Q_LBO, 1024);
                        umma_f16<CTAS>(d_tmem, dP, dQ, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    // frees the stage (in both CTAs of a pair) when the MMAs retire
                    if constexpr (PAIR) umma_commit_2cta(smem_u32(&ctrl->empty[stage]), 3);
                    else umma_commit(smem_u32(&ctrl->empty[stage]));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) {
                    if constexpr (PAIR) umma_commit_2cta(smem_u32(&ctrl->tmem_full[acc]), 3);
                    else umma_commit(smem_u32(&ctrl->tmem_full[acc]));
                }
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------- epilogue
        const int q = warp - 4;  // TMEM lane quarter
        uint32_t it = 0;
        bool ok = true;
        for (int t = first_tile; t < total_tiles && ok; t += tile_step, ++it) {
            const TileCoord tc = decode_tile(p, t);
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            ok = mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, abort_flag, p.status,
                           DEV_TIMEOUT_TMEM_F);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = (tc.m_blk * CTAS + static_cast<int>(rank)) * BM + q * 32 + lane;
            const uint32_t taddr = tmem_base + acc * Cfg::ACC_STRIDE + (static_cast<uint32_t>(q * 32) << 16);
            epilogue_store<BN, EPI>(p, taddr, row, tc.n_blk * BN, tc.split);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(smem_u32(&ctrl->tmem_empty[acc]), 0);
                else mbar_arrive(smem_u32(&ctrl->tmem_empty[acc]));
            }
        }
    }

    // ------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) {  // neither CTA may leave while the other can still touch its smem/TMEM
        cluster_arrive_release();
        cluster_wait_acquire();
    }
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<CTAS>(tmem_base, Cfg::TMEM_COLS);
    }
}

// Split-K reduction: out = rn( sum_s ws[s] (+ float(out) when beta1) ), fixed order s = 0..S-1.
// n = Mo*No, a multiple of 8.
template <bool BETA1>
__global__ void splitk_reduce_bf16(__nv_bfloat16* __restrict__ out, const float* __restrict__ ws,
                                   long long n, int splits) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
    for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n;
         i += stride) {
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < splits; ++s) {
            const float4 x = *reinterpret_cast<const float4*>(ws + s * n + i);
            const float4 y = *reinterpret_cast<const float4*>(ws + s * n + i + 4);
            a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w;
            a[4] += y.x; a[5] += y.y; a[6] += y.z; a[7] += y.w;
        }
        if constexpr (BETA1) {
            const uint4 o = *reinterpret_cast<const uint4*>(out + i);
            a[0] += bf16_lo(o.x); a[1] += bf16_hi(o.x); a[2] += bf16_lo(o.y); a[3] += bf16_hi(o.y);
            a[4] += bf16_lo(o.z); a[5] += bf16_hi(o.z); a[6] += bf16_lo(o.w); a[7] += bf16_hi(o.w);
        }
        *reinterpret_cast<uint4*>(out + i) =
            make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]),
                       pack_bf16x2(a[6], a[7]));
    }
}

}  // namespace b200
