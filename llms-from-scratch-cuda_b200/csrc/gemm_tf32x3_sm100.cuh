// fp32 GEMM on the sm_100a tensor cores with fp32-grade accuracy ("3xTF32").
//
// The reference's fp32 path is cublasSgemm in default math mode (cuda/matmul.cu:4-48 of the
// reference): true fp32.  A single tf32 tensor-core product keeps 10 mantissa bits of each operand and
// misses the 1e-5 tolerance, so every operand x is split as x = hi + lo with hi = x truncated to
// tf32 (what the tensor core reads from an fp32 word anyway) and lo = x - hi (exact in fp32), and
//     P*Q  ~=  P_hi*Q_hi + P_hi*Q_lo + P_lo*Q_hi           (fp32 accumulate in TMEM)
// which drops only the lo*lo term (~2^-22 relative).  The lo tiles are made inside the kernel: four
// converter warps rewrite each landed stage element by element (the swizzled layout does not matter for
// an element-wise pass), so global memory holds plain fp32 matrices and nothing is repacked.
//
// The tensor core adds each MMA's result into the TMEM accumulator with truncation, which biases a long
// accumulation chain (error ~ 6e-8 per MMA, i.e. 2.5e-4 after a 32000-long contraction).  So TMEM only
// accumulates T32_CHUNK stages (256 contraction elements); the epilogue warps drain every chunk and keep
// the running sum in registers with ordinary rounded fp32 adds (two accumulator buffers: the next chunk
// is computed while the previous one is drained).
//
// MN-major 32-bit operands exist in one shared-memory layout only: 128-byte rows swizzled in 32-byte
// units, 4 contraction rows per swizzle atom (TMA: SWIZZLE_128B_ATOM_32B; descriptor layout type 1).
//
// Same operand model, tile raster and persistent schedule as the bf16 kernel; 128 x BN tiles, BK = 32
// fp32 elements (one 128-byte swizzle row), single CTA per tile, whole tiles only (no split).
#pragma once
#include "gemm_sm100.cuh"

namespace b200 {

constexpr int T32_THREADS = 512;  // warps: 0 P loads, 3 Q loads, 1 MMA, 2 TMEM, 4-11 epilogue, 12-15 converters
constexpr int T32_BK = 32;        // fp32 elements per stage row (128 bytes)
constexpr int T32_UMMA_K = 8;     // contraction elements per tcgen05.mma.kind::tf32
constexpr int T32_CHUNK = 8;      // stages accumulated in TMEM before the sum moves to registers

template <int BN>
struct T32Cfg {
    static constexpr int A_BYTES = BM * 128;
    static constexpr int B_BYTES = BN * 128;
    static constexpr int HI_BYTES = A_BYTES + B_BYTES;   // [P | Q] as loaded
    static constexpr int STAGE_BYTES = 2 * HI_BYTES;     // followed by [P_lo | Q_lo]
    static constexpr int CTRL_BYTES = 1024;
    static constexpr int EPI_BYTES = EPI_WARPS * EPI_BUF_BYTES;
    static constexpr int STAGES_RAW = (SMEM_BUDGET - CTRL_BYTES - EPI_BYTES - 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + CTRL_BYTES + EPI_BYTES + 1024;
    static constexpr int ACC_STRIDE = BN <= 64 ? 64 : 128;
    static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
    static_assert(BN == 64 || BN == 128, "tile width");
    static_assert(STAGES >= 3, "pipeline too shallow");
};

struct alignas(8) T32Ctrl {
    unsigned long long full[6];        // TMA -> converters and MMA: fp32 stage landed
    unsigned long long conv[6];        // converters -> MMA: lo tiles written
    unsigned long long empty[6];       // MMA -> TMA: stage consumed
    unsigned long long tmem_full[2];
    unsigned long long tmem_empty[2];
    unsigned long long old_bar[8];
    uint32_t tmem_base;
    int abort_flag;
};

template <int BN, bool P_MN, bool Q_MN, bool BETA1>
__global__ void __launch_bounds__(T32_THREADS, 1)
gemm_tf32x3_sm100(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                  const __grid_constant__ CUtensorMap tmD, const GemmParams p) {
    using Cfg = T32Cfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    T32Ctrl* ctrl = reinterpret_cast<T32Ctrl*>(smem);
    uint8_t* tiles = smem + Cfg::CTRL_BYTES;
    uint8_t* epi_bufs = tiles + STAGES * Cfg::STAGE_BYTES;
    volatile int* abort_flag = &ctrl->abort_flag;
    // the warp index is read through a shuffle so that the compiler knows it is uniform across the warp
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int slot = blockIdx.x, nslots = gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->full[s]), 2);   // one arrival (+ bytes) per producer thread
            mbar_init(smem_u32(&ctrl->conv[s]), 4);   // one arrival per converter warp
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctrl->tmem_full[a]), 1);
            mbar_init(smem_u32(&ctrl->tmem_empty[a]), EPI_WARPS);
        }
        for (int w8 = 0; w8 < EPI_WARPS; ++w8) mbar_init(smem_u32(&ctrl->old_bar[w8]), 1);
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmP);
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmD);
    }
    if (warp == 2) {
        tmem_alloc<1>(smem_u32(&ctrl->tmem_base), Cfg::TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;
    griddep_wait();
    griddep_launch_dependents();
    // The issuing roles run with their warp converged and one elected lane issuing (uniform operands).

    if (warp == 0 || warp == 3) {
        // ------------------------------------------------------------ TMA producers (P: warp 0, Q: warp 3)
        {
            const bool is_q = warp == 3;
            const CUtensorMap* tm = is_q ? &tmQ : &tmP;
            const bool mn = is_q ? Q_MN : P_MN;
            const bool as3d = is_q ? (p.q_3d != 0) : (p.p_3d != 0);
            const int panels = is_q ? BN / 32 : BM / 32;
            const uint32_t my_bytes = is_q ? Cfg::B_BYTES : Cfg::A_BYTES;
            const uint32_t my_off = is_q ? Cfg::A_BYTES : 0;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            WorkItem w;
            for (int i = 0; ok && get_work(p, slot, nslots, i, w); ++i) {
                const int r0 = is_q ? w.n_blk * BN : w.m_blk * BM;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    ok = mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    const uint32_t bar = smem_u32(&ctrl->full[stage]);
                    const uint32_t dst = smem_u32(tiles + stage * Cfg::STAGE_BYTES) + my_off;
                    const int c0 = kb * T32_BK;
                    if (elect_one()) {
                        mbar_arrive_expect_tx(bar, my_bytes);
                        if (!mn) {
                            tma_load_2d(dst, tm, bar, c0, r0);                 // [rows][Kc]: box 32 x rows
                        } else if (as3d) {
                            tma_load_3d(dst, tm, bar, 0, c0, r0 >> 5);         // [Kc][rows]: all 32-wide panels
                        } else {
                            for (int j = 0; j < panels; ++j)
                                tma_load_2d(dst + j * (32 * 128), tm, bar, r0 + 32 * j, c0);
                        }
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp >= 12) {
        // ------------------------------------------------------------ converters: lo = x - tf32_trunc(x)
        const int t = threadIdx.x - 12 * 32;  // 0..127
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        WorkItem w;
        for (int i = 0; ok && get_work(p, slot, nslots, i, w); ++i) {
            for (int kb = w.kb0; kb < w.kb1; ++kb) {
                ok = mbar_wait(smem_u32(&ctrl->full[stage]), phase, abort_flag, p.status, DEV_TIMEOUT_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint4* src = reinterpret_cast<const uint4*>(tiles + stage * Cfg::STAGE_BYTES);
                uint4* dst = reinterpret_cast<uint4*>(tiles + stage * Cfg::STAGE_BYTES + Cfg::HI_BYTES);
#pragma unroll 4
                for (int v = t; v < Cfg::HI_BYTES / 16; v += 128) {
                    const uint4 x = src[v];
                    uint4 y;
                    y.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(x.x & 0xFFFFE000u));
                    y.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(x.y & 0xFFFFE000u));
                    y.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(x.z & 0xFFFFE000u));
                    y.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(x.w & 0xFFFFE000u));
                    dst[v] = y;
                }
                fence_proxy_async_smem();  // generic writes -> visible to the tensor core's reads
                __syncwarp();
                if (elect_one()) mbar_arrive(smem_u32(&ctrl->conv[stage]));
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        {
            constexpr uint32_t idesc = umma_idesc(2, BM, BN, P_MN ? 1 : 0, Q_MN ? 1 : 0);
            // K-major: 128-byte swizzle, +32 B per UMMA_K (8 fp32).  MN-major: 32-wide panels of BK rows x
            // 128 B (LBO = panel pitch 4096 B), 4-row swizzle atoms 512 B apart (SBO), layout type 1;
            // +8 rows = 1024 B per UMMA_K.
            constexpr uint32_t P_LBO = P_MN ? 32 * 128 : 16, P_SBO = P_MN ? 512 : 1024, P_LT = P_MN ? 1 : 2;
            constexpr uint32_t Q_LBO = Q_MN ? 32 * 128 : 16, Q_SBO = Q_MN ? 512 : 1024, Q_LT = Q_MN ? 1 : 2;
            constexpr uint32_t P_STEP = P_MN ? T32_UMMA_K * 128 : T32_UMMA_K * 4;
            constexpr uint32_t Q_STEP = Q_MN ? T32_UMMA_K * 128 : T32_UMMA_K * 4;
            const uint64_t descP0 = umma_smem_desc(smem_u32(tiles), P_LBO, P_SBO, P_LT);
            const uint64_t descQ0 = umma_smem_desc(smem_u32(tiles) + Cfg::A_BYTES, Q_LBO, Q_SBO, Q_LT);
            constexpr uint32_t LO = Cfg::HI_BYTES >> 4;  // descriptor offset of the lo copy of a tile
            uint32_t stage = 0, phase = 0, cc = 0;       // cc: chunks issued so far (selects the TMEM buffer)
            bool ok = true;
            WorkItem w;
            for (int i = 0; ok && get_work(p, slot, nslots, i, w); ++i) {
                for (int kc = w.kb0; ok && kc < w.kb1; kc += T32_CHUNK, ++cc) {
                    const uint32_t acc = cc & 1, acc_phase = (cc >> 1) & 1;
                    ok = mbar_wait(smem_u32(&ctrl->tmem_empty[acc]), acc_phase ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_E);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
                    const int kend = min(kc + T32_CHUNK, w.kb1);
                    for (int kb = kc; kb < kend; ++kb) {
                        const uint32_t st_off = (stage * Cfg::STAGE_BYTES) >> 4;
                        ok = mbar_wait(smem_u32(&ctrl->full[stage]), phase, abort_flag, p.status, DEV_TIMEOUT_FULL);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tc_fence_after();
                        if (elect_one()) {
#pragma unroll
                            for (int k = 0; k < T32_BK / T32_UMMA_K; ++k)  // hi * hi, as soon as the stage has landed
                                umma_tf32<1>(d_tmem, descP0 + (st_off + ((k * P_STEP) >> 4)),
                                             descQ0 + (st_off + ((k * Q_STEP) >> 4)), idesc, (kb > kc || k > 0) ? 1u : 0u);
                        }
                        __syncwarp();
                        ok = mbar_wait(smem_u32(&ctrl->conv[stage]), phase, abort_flag, p.status, DEV_TIMEOUT_FULL);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tc_fence_after();
                        if (elect_one()) {
#pragma unroll
                            for (int k = 0; k < T32_BK / T32_UMMA_K; ++k) {
                                const uint64_t dP = descP0 + (st_off + ((k * P_STEP) >> 4));
                                const uint64_t dQ = descQ0 + (st_off + ((k * Q_STEP) >> 4));
                                umma_tf32<1>(d_tmem, dP + LO, dQ, idesc, 1u);  // lo * hi
                                umma_tf32<1>(d_tmem, dP, dQ + LO, idesc, 1u);  // hi * lo
                            }
                            umma_commit(smem_u32(&ctrl->empty[stage]));
                            if (kb == kend - 1) umma_commit(smem_u32(&ctrl->tmem_full[acc]));
                        }
                        __syncwarp();
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    }
                }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------ epilogue
        // warp (q, hsel): rows 32q..32q+31, columns hsel*BN/2 .. +BN/2; running fp32 sum in registers
        const int q = warp & 3, hsel = (warp - 4) >> 2;
        constexpr int HALF = BN / 2;
        const uint32_t old_bar = smem_u32(&ctrl->old_bar[warp - 4]);
        uint8_t* buf = epi_bufs + (warp - 4) * EPI_BUF_BYTES;
        uint32_t old_phase = 0, cc = 0;
        bool ok = true;
        WorkItem w;
        for (int i = 0; ok && get_work(p, slot, nslots, i, w); ++i) {
            float sum[HALF];
#pragma unroll
            for (int e = 0; e < HALF; ++e) sum[e] = 0.f;
            for (int kc = w.kb0; ok && kc < w.kb1; kc += T32_CHUNK, ++cc) {
                const uint32_t acc = cc & 1, acc_phase = (cc >> 1) & 1;
                ok = mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, abort_flag, p.status, DEV_TIMEOUT_TMEM_F);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + acc * Cfg::ACC_STRIDE + hsel * HALF + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
                for (int g = 0; g < HALF / 32; ++g) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + g * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) sum[g * 32 + e] += __uint_as_float(r[e]);
                }
                tc_fence_before();
                __syncwarp();
                if (elect_one()) mbar_arrive(smem_u32(&ctrl->tmem_empty[acc]));
            }
            if (!ok) break;
            const int row0 = w.m_blk * BM + q * 32;
#pragma unroll
            for (int g = 0; g < HALF / 32; ++g) {
                const int col0 = w.n_blk * BN + hsel * HALF + g * 32;
                if (col0 >= p.No) break;
                if (elect_one()) {
                    tma_store_wait_read<0>();
                    if constexpr (BETA1) {
                        mbar_arrive_expect_tx(old_bar, EPI_BUF_BYTES);
                        tma_load_2d(smem_u32(buf), &tmD, old_bar, col0, row0);
                    }
                }
                if constexpr (BETA1) {
                    ok = mbar_wait(old_bar, old_phase, abort_flag, p.status, DEV_TIMEOUT_DRAIN);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    old_phase ^= 1;
                } else {
                    __syncwarp();
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint4* slot16 = reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4));
                    float4 v = make_float4(sum[g * 32 + 4 * j], sum[g * 32 + 4 * j + 1], sum[g * 32 + 4 * j + 2],
                                           sum[g * 32 + 4 * j + 3]);
                    if constexpr (BETA1) {
                        const float4 o = *reinterpret_cast<const float4*>(slot16);
                        v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                    }
                    *reinterpret_cast<float4*>(slot16) = v;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (row0 < p.Mo && elect_one()) {
                    tma_store_2d(&tmD, smem_u32(buf), col0, row0);
                    tma_store_commit();
                }
            }
        }
        if (elect_one()) tma_store_wait_read<0>();  // staging buffers read; the grid's end completes the writes
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace b200
