// Fused causal grouped-query attention forward on the sm_100a tensor cores (bf16 in, fp32 accumulate):
//   context = softmax(Q K^T / sqrt(64), causal) V,   lse = row log-sum-exp of the scaled scores,
// for q, context [B, T, n_head*64], k, v [B, T, n_kv_head*64] -- the contract the reference declares for
// flash_attention_forward (cuda/kernels.cuh:420-427) and leaves empty (cuda/flash_attention.cu:12-17), and the
// core of its attention_forward (cuda/attention.cu:419-461,603-615).  No [B, n_head, T, T] matrix exists.
//
// One CTA per (batch, query head, 128 query rows); blocks are dispatched longest first (the last query tile of every
// head before anybody's first).  Per 128-row key/value tile:
//   S    = Q K^T            tcgen05.mma 128 x 128 x 64, both operands K-major from 128B-swizzled TMA tiles, S in TMEM
//   P_h  = exp2(S_h - m_h)  h = the NS (4, or 2) parts of the tile's 128 key columns, each a softmax of its own: thread
//                           (row, h) owns that part of a row of S (TMEM lane = query row), its reference maximum m_h and
//                           its row sum, so nothing is exchanged between threads per tile; P goes to shared memory as
//                           bf16 in the K-major swizzled layout the tensor core reads (two 64-column panels)
//   O_h += P_h V_h          tcgen05.mma 128 x 64 x (128 / NS), V as an MN-major operand (its rows are the contraction),
//                           accumulating in TMEM over all tiles (NS accumulators of 64 columns beside the two of S)
// m_h follows the true maximum lazily: it moves, and O_h is rescaled in TMEM (tcgen05.ld, multiply, tcgen05.st), only
// when the maximum has grown by more than 2^FA_RESCALE_STEP, so P stays below 2^8 and after the first tiles of a row the
// rescale is rare.  After the last tile the parts are combined: O = sum_h w_h O_h / sum_h w_h l_h with
// w_h = 2^(m_h - max_h m_h).  S is double-buffered in TMEM and P, K/V in shared memory, so the tensor core computes
// the next tile's S and this tile's products while the softmax warps work.
// Warp roles: 0 = TMA producer, 1 = MMA issuer, 2 = TMEM allocator, 4 .. 4 + 4 NS - 1 = softmax + epilogue: warps w,
// w + 4, ... share a TMEM lane quarter (32 query rows) and take one part each (and, in the epilogue, 64 / NS of the 64
// output columns), so that every scheduler has NS softmax warps to interleave.
// Every wait is bounded (ptx.cuh): on expiry the CTA records a code in *status and leaves.
#pragma once
#include <cuda_bf16.h>

#include "gemm_sm100.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int FA_BQ = 128;        // query rows per CTA = TMEM lanes
constexpr int FA_BKV = 128;       // key/value rows per tile
constexpr int FA_HD = 64;         // head dimension
// threads per CTA: 128 + 128 NS: warps 0-3 = producer, MMA issuer, TMEM allocator, idle; then 4 NS softmax / epilogue warps
constexpr int FA_TILE_BYTES = 128 * 64 * 2;                 // one 128 x 64 bf16 tile, 128-byte rows
constexpr int FA_KV_STAGES = 3;      // K/V tiles in flight: a stage is free again only after its P V product
constexpr int FA_KV_STAGES_TS = 5;   // ... when P / dS go through tensor memory and their shared-memory buffers are stages instead
constexpr int FA_KV_STAGES_MAX = 5;
constexpr int FA_SMEM_BYTES = 5120 /*control*/ + FA_TILE_BYTES /*Q*/ + FA_KV_STAGES * 2 * FA_TILE_BYTES /*K,V stages*/ +
                              2 * 2 * FA_TILE_BYTES /*P x 2: two 64-column panels each*/ + 1024 /*alignment*/;
// P through tensor memory: five K/V stages, one tile of output staging where the P buffers were
constexpr int FA_SMEM_BYTES_TS = 5120 + FA_TILE_BYTES + FA_KV_STAGES_TS * 2 * FA_TILE_BYTES + FA_TILE_BYTES + 1024;
constexpr int FA_TMEM_COLS = 512;  // S: 2 x 128 columns, O: 2 x 64 columns (forward), dP / dQ / dK / dV (backward)
constexpr float FA_RESCALE_STEP = 8.0f;   // a row's reference maximum moves only when the true maximum has grown by 2^8

struct FaParams {
    int B, T, n_head, n_kv_head;
    float scale_log2e;   // log2(e) / sqrt(head_dim)
    float* lse;          // [B, n_head, T]
    int* status;         // device status word (0 = ok)
};

struct alignas(8) FaCtrl {
    unsigned long long q_full;
    unsigned long long kv_full[FA_KV_STAGES_MAX], kv_empty[FA_KV_STAGES_MAX];
    unsigned long long s_full[2], s_empty[2];
    unsigned long long p_full[2], p_empty[2];
    unsigned long long pv_done;        // the P V products of one more key tile have retired (one phase per tile)
    unsigned long long lsum;           // the two halves of every row have published their maximum and row sum (once, at the end)
    uint32_t tmem_base;
    int abort_flag;
    float mpart[4][FA_BQ];             // [part][row]: reference maximum of that part of the row
    float lpart[4][FA_BQ];             // [part][row]: its row sum, in units of 2^-maximum
};
constexpr int FA_CTRL_BYTES = 5120;   // a multiple of 1024: the tiles behind it stay 1024-byte aligned
static_assert(sizeof(FaCtrl) <= FA_CTRL_BYTES, "control block");

__device__ __forceinline__ float fa_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));   // pure: the compiler may reorder and interleave these
    return y;
}

// tmQ / tmO: {n_head*64, T, B} bf16, box {64, 128, 1};  tmK / tmV: {n_kv_head*64, T, B}, box {64, 128, 1};
// all 128-byte swizzled.  Rows beyond T read as zero and are not written.
// NS = softmax threads per query row (2 or 4): each takes 128 / NS key columns of a tile as a softmax of its own, with
// its own accumulator O_part (64 TMEM columns each: S 2 x 128 + O NS x 64 <= 512), and 4 NS softmax warps run beside
// the four role warps (384 or 640 threads).
// P_TMEM: P goes back to tensor memory as bf16 (over the first half of each 32-column group of the S buffer it came
// from) and the tensor core reads it from there as the left operand of P V, instead of through shared memory.
template <int NS, bool P_TMEM>
__global__ void __launch_bounds__(128 + NS * 128, 1)
attn_fwd_sm100(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const FaParams p) {
    constexpr int STAGES = P_TMEM ? FA_KV_STAGES_TS : FA_KV_STAGES;
    extern __shared__ uint8_t fa_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    FaCtrl* ctrl = reinterpret_cast<FaCtrl*>(smem);
    uint8_t* sQ = smem + FA_CTRL_BYTES;
    uint8_t* sKV = sQ + FA_TILE_BYTES;            // stage s: [K tile | V tile]
    uint8_t* sP = sKV + STAGES * 2 * FA_TILE_BYTES;   // buffer b: [columns 0..63 | columns 64..127]
    volatile int* abort_flag = &ctrl->abort_flag;

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    // grid = (heads, batch, query tiles): blocks are dispatched x-fastest, so every (head, batch) pair's longest rows
    // (the last query tile: most key tiles under the causal mask) start before anybody's short ones
    const int qt = gridDim.z - 1 - blockIdx.z, h = blockIdx.x, b = blockIdx.y;
    const int kvh = h / (p.n_head / p.n_kv_head);
    const int n_kv = qt + 1;                      // causal: key tiles 0 .. qt

    if (warp == 1) {
        if (lane == 0) {
            mbar_init(smem_u32(&ctrl->q_full), 1);
            for (int i = 0; i < STAGES; ++i) {
                mbar_init(smem_u32(&ctrl->kv_full[i]), 1);
                mbar_init(smem_u32(&ctrl->kv_empty[i]), 1);
            }
            for (int i = 0; i < 2; ++i) {
                mbar_init(smem_u32(&ctrl->s_full[i]), 1);
                mbar_init(smem_u32(&ctrl->s_empty[i]), P_TMEM ? 1 : (4 * NS));   // P_TMEM: freed by the tensor core after P V
                mbar_init(smem_u32(&ctrl->p_full[i]), (4 * NS));
                mbar_init(smem_u32(&ctrl->p_empty[i]), 1);
            }
            mbar_init(smem_u32(&ctrl->pv_done), 1);
            mbar_init(smem_u32(&ctrl->lsum), (4 * NS));
            ctrl->abort_flag = 0;
            fence_mbar_init();
        }
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmO);
    }
    if (warp == 2) {
        tmem_alloc<1>(smem_u32(&ctrl->tmem_base), FA_TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_sync();   // everything above touches no global memory and may overlap the previous kernel's tail
    const uint32_t tmem_base = ctrl->tmem_base;
    const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 256;   // S[b] at +128 b; O of key-column part h at +64 h

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        const bool issuer = elect_one();
        if (issuer) {
            mbar_arrive_expect_tx(smem_u32(&ctrl->q_full), FA_TILE_BYTES);
            tma_load_3d(smem_u32(sQ), &tmQ, smem_u32(&ctrl->q_full), h * FA_HD, qt * FA_BQ, b);
        }
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            const int s = j % STAGES;
            ok = mbar_wait(smem_u32(&ctrl->kv_empty[s]), ((j / STAGES) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (issuer) {
                const uint32_t bar = smem_u32(&ctrl->kv_full[s]);
                const uint32_t dst = smem_u32(sKV + s * 2 * FA_TILE_BYTES);
                mbar_arrive_expect_tx(bar, 2 * FA_TILE_BYTES);
                tma_load_3d(dst, &tmK, bar, kvh * FA_HD, j * FA_BKV, b);
                tma_load_3d(dst + FA_TILE_BYTES, &tmV, bar, kvh * FA_HD, j * FA_BKV, b);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_S = umma_idesc(1, FA_BQ, FA_BKV, 0, 0);   // Q, K: K-major
        constexpr uint32_t idesc_PV = umma_idesc(1, FA_BQ, FA_HD, 0, 1);   // P: K-major, V: MN-major
        const bool issuer = elect_one();
        const uint64_t descQ = umma_smem_desc(smem_u32(sQ), 16, 1024);
        bool ok = mbar_wait(smem_u32(&ctrl->q_full), 0, abort_flag, p.status, DEV_TIMEOUT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        for (int j = 0; j <= n_kv && ok; ++j) {
            if (j < n_kv) {   // S_j = Q K_j^T
                const int s = j & 1, st = j % STAGES;
                ok = mbar_wait(smem_u32(&ctrl->kv_full[st]), (j / STAGES) & 1, abort_flag, p.status, DEV_TIMEOUT_FULL) &&
                     mbar_wait(smem_u32(&ctrl->s_empty[s]), ((j >> 1) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_E);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (issuer) {
                    const uint64_t descK = umma_smem_desc(smem_u32(sKV + st * 2 * FA_TILE_BYTES), 16, 1024);
#pragma unroll
                    for (int k = 0; k < FA_HD / UMMA_K; ++k)
                        umma_f16<1>(tmem_S + s * 128, descQ + ((k * UMMA_K * 2) >> 4), descK + ((k * UMMA_K * 2) >> 4), idesc_S,
                                    k > 0 ? 1u : 0u);
                    umma_commit(smem_u32(&ctrl->s_full[s]));
                }
            }
            if (j >= 1) {     // O_h += P_ih V_ih for the tile before, h = the two 64-column halves of the key tile
                const int i = j - 1, s = i & 1, st = i % STAGES;
                ok = mbar_wait(smem_u32(&ctrl->p_full[s]), (i >> 1) & 1, abort_flag, p.status, DEV_TIMEOUT_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (issuer) {
                    // V tile: 128 contraction rows of 128 bytes, 8-row groups 1024 bytes apart, 16 rows per MMA
                    const uint64_t descV = umma_smem_desc(smem_u32(sKV + st * 2 * FA_TILE_BYTES + FA_TILE_BYTES), 64 * 64 * 2, 1024);
                    const uint32_t pbase = smem_u32(sP + s * 2 * FA_TILE_BYTES);
                    constexpr int KPP = (FA_BKV / UMMA_K) / NS;   // MMAs per part of the key tile
#pragma unroll
                    for (int k = 0; k < FA_BKV / UMMA_K; ++k) {
                        // Part k / KPP of the key columns meets the matching key rows of V and accumulates into its own O:
                        // the parts keep separate maxima.
                        const uint32_t acc = (i > 0 || (k % KPP) > 0) ? 1u : 0u;
                        if constexpr (P_TMEM) {
                            // P of keys 16 k .. 16 k + 15: 8 packed columns in the first half of 32-column group k / 2 of S
                            umma_f16_ts(tmem_O + (k / KPP) * 64, tmem_S + s * 128 + (k >> 1) * 32 + (k & 1) * 8,
                                        descV + ((k * UMMA_K * 128) >> 4), idesc_PV, acc);
                        } else {
                            // P: two 64-column panels of 128-byte rows; 32 bytes per MMA inside a panel
                            const uint64_t descP = umma_smem_desc(pbase + (k >> 2) * FA_TILE_BYTES + (k & 3) * UMMA_K * 2, 16, 1024);
                            umma_f16<1>(tmem_O + (k / KPP) * 64, descP, descV + ((k * UMMA_K * 128) >> 4), idesc_PV, acc);
                        }
                    }
                    if constexpr (P_TMEM) umma_commit(smem_u32(&ctrl->s_empty[s]));   // P lived in this S buffer
                    umma_commit(smem_u32(&ctrl->pv_done));
                    umma_commit(smem_u32(&ctrl->kv_empty[st]));
                    umma_commit(smem_u32(&ctrl->p_empty[s]));
                }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ softmax + epilogue
        const int qrt = warp & 3;                                   // TMEM lane quarter of this warp
        const int part = (warp - 4) >> 2;                           // which 128 / NS key columns of the row
        const int r = qrt * 32 + lane;                              // query row inside the tile
        const int row = qt * FA_BQ + r;                             // query position
        const uint32_t lane_off = static_cast<uint32_t>(qrt * 32) << 16;
        constexpr int HC = FA_BKV / NS;                             // columns of S per thread
        constexpr int OC = FA_HD / NS;                              // output columns per thread in the epilogue
        // Each part of a row is a softmax of its own: reference maximum m (log2 units), row sum l in units of 2^-m, and
        // an accumulator O_part in TMEM that the tensor core adds P_part V_part to.  m follows the true maximum lazily:
        // it moves (and O_part, l are rescaled) only when the maximum has grown by more than FA_RESCALE_STEP, so that
        // P stays below 2^8 and the common tile costs one max, one FMA + exp2 and one add per element and no exchange.
        // The parts are put together once, after the last tile.
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            const int s = j & 1;
            ok = mbar_wait(smem_u32(&ctrl->s_full[s]), (j >> 1) & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_F);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tS = tmem_S + s * 128 + lane_off + part * HC;
            const bool diag = j == qt;                              // the only tile that needs the causal / length mask
            const int col0 = j * FA_BKV + part * HC;
            // this thread's part of the row of S comes into registers with one wait; the S buffer is free for tile j + 2
            float x[HC];
#pragma unroll
            for (int c = 0; c < HC / 32; ++c) tmem_ld_32x32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&x[c * 32]));
            tmem_ld_wait();
            if constexpr (!P_TMEM) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctrl->s_empty[s]));
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (diag) {
#pragma unroll
                for (int e = 0; e < HC; ++e) {
                    const int col = col0 + e;
                    if (col > row || col >= p.T) x[e] = -INFINITY;
                    mx4[e & 3] = fmaxf(mx4[e & 3], x[e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < HC; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], x[e]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2e;   // the scale is positive
            const bool grow = mx > m + FA_RESCALE_STEP;             // also the first finite maximum (m = -inf)
            if (__any_sync(0xffffffffu, grow)) {
                // rare after the first tiles: move this row's reference maximum and bring l and O_part along
                const float m_new = grow ? mx : m;
                const float alpha = (m_new == m) ? 1.0f : fa_exp2(m - m_new);   // 0 when m was -inf
                if (j > 0) {
                    // the products of tile j - 1 must have landed in O; those of tile j wait for this warp's P
                    ok = mbar_wait(smem_u32(&ctrl->pv_done), (j - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_F);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {   // 16 columns at a time: this path is rare and must stay cheap in registers
                        uint32_t acc[16];
                        tmem_ld_32x16(tmem_O + part * FA_HD + lane_off + c * 16, acc);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 16; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
                        tmem_st_32x16(tmem_O + part * FA_HD + lane_off + c * 16, acc);
                    }
                    tmem_st_wait();
                }
                l *= alpha;
                m = m_new;
            }
            if constexpr (!P_TMEM) {
                // the tensor core must have finished reading this P buffer (tile j - 2)
                ok = mbar_wait(smem_u32(&ctrl->p_empty[s]), ((j >> 1) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            // P = exp2(S scale - m) as bf16 into this part's columns of the two 64-column panels, row sum in fp32
            const float neg_m = (m == -INFINITY) ? 0.f : -m;       // a part with nothing visible yet: P = exp2(-inf) = 0
            uint8_t* prow = sP + s * 2 * FA_TILE_BYTES + r * 128;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < HC / 32; ++c) {
                uint32_t packed[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const float p0 = fa_exp2(fmaf(x[c * 32 + e], p.scale_log2e, neg_m));
                    const float p1 = fa_exp2(fmaf(x[c * 32 + e + 1], p.scale_log2e, neg_m));
                    sum4[(e >> 1) & 3] += p0 + p1;
                    packed[e >> 1] = pack_bf16x2(p0, p1);
                }
                const int g32 = part * (HC / 32) + c;   // which 32-column group of the tile: panel g32 >> 1, half-row g32 & 1
                if constexpr (P_TMEM) {
                    // over the first 16 columns of the group's own S columns (already in this thread's registers)
                    tmem_st_32x16(tmem_S + s * 128 + lane_off + g32 * 32, packed);
                } else {
                    uint8_t* panel = prow + (g32 >> 1) * FA_TILE_BYTES;
#pragma unroll
                    for (int qd = 0; qd < 4; ++qd) {   // four 16-byte chunks of the 128-byte panel row, swizzled by the row
                        const int chunk = ((g32 & 1) * 4 + qd) ^ (r & 7);
                        *reinterpret_cast<uint4*>(panel + chunk * 16) =
                            make_uint4(packed[4 * qd], packed[4 * qd + 1], packed[4 * qd + 2], packed[4 * qd + 3]);
                    }
                }
            }
            if constexpr (P_TMEM) tmem_st_wait();
            else fence_proxy_async_smem();
            tc_fence_before();                                         // orders P / a rescale of O before the next product
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->p_full[s]));    // this warp's part of P is ready for the tensor core
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        }
        if (ok) {
            // the parts of a row exchange (m, l); the last products must have retired
            ctrl->mpart[part][r] = m;
            ctrl->lpart[part][r] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->lsum));
            ok = mbar_wait(smem_u32(&ctrl->lsum), 0, abort_flag, p.status, DEV_TIMEOUT_PEER) &&
                 mbar_wait(smem_u32(&ctrl->pv_done), (n_kv - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_F);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after();
            float m_row = -INFINITY;                                    // finite: column `row` itself is always visible
#pragma unroll
            for (int a = 0; a < NS; ++a) m_row = fmaxf(m_row, ctrl->mpart[a][r]);
            float w[NS], l_row = 0.f;
#pragma unroll
            for (int a = 0; a < NS; ++a) {
                const float ma = ctrl->mpart[a][r];
                w[a] = (ma == -INFINITY) ? 0.f : fa_exp2(ma - m_row);
                l_row += ctrl->lpart[a][r] * w[a];
            }
            const float inv = 1.0f / l_row;
            // every tensor-core read of the P buffers has completed (the last commit covers them): stage O in P buffer 0.
            // This thread writes output columns OC part .. OC part + OC - 1 of its row: sum_a w_a O_a over l.
            float y[OC];
#pragma unroll
            for (int e = 0; e < OC; ++e) y[e] = 0.f;
#pragma unroll
            for (int a = 0; a < NS; ++a) {
                const float ca = w[a] * inv;
#pragma unroll
                for (int g = 0; g < OC / 16; ++g) {
                    uint32_t v[16];
                    tmem_ld_32x16(tmem_O + a * FA_HD + lane_off + part * OC + g * 16, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; ++e) y[g * 16 + e] = fmaf(__uint_as_float(v[e]), ca, y[g * 16 + e]);
                }
            }
            uint8_t* orow = sP + r * 128;
#pragma unroll
            for (int qd = 0; qd < OC / 8; ++qd) {
                const int chunk = (part * (OC / 8) + qd) ^ (r & 7);
                *reinterpret_cast<uint4*>(orow + chunk * 16) =
                    make_uint4(pack_bf16x2(y[qd * 8], y[qd * 8 + 1]), pack_bf16x2(y[qd * 8 + 2], y[qd * 8 + 3]),
                               pack_bf16x2(y[qd * 8 + 4], y[qd * 8 + 5]), pack_bf16x2(y[qd * 8 + 6], y[qd * 8 + 7]));
            }
            if (part == 0 && row < p.T)
                p.lse[(static_cast<long long>(b) * p.n_head + h) * p.T + row] = (m_row + log2f(l_row)) * 0.69314718055994531f;
        }
        // All softmax / epilogue warps come here exactly once, whether or not their waits succeeded, so this barrier
        // cannot be left waiting; the tile is stored only if nobody gave up.
        tc_fence_before();
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, %0;" ::"n"(NS * 128) : "memory");
        if (warp == 4 && !*abort_flag) {
            if (elect_one()) {
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                                 reinterpret_cast<uint64_t>(&tmO)),
                             "r"(smem_u32(sP)), "r"(h * FA_HD), "r"(qt * FA_BQ), "r"(b)
                             : "memory");
                tma_store_commit();
                tma_store_wait_read<0>();
            }
        }
    }
    // ------------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, FA_TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------ backward
// With P_ij = exp(s_ij - lse_i) recomputed from the saved row log-sum-exps and delta_i = sum_d dO_id O_id:
//   dP = dO V^T,   dS = P o (dP - delta),   dQ = scale dS K,   dK = scale dS^T Q,   dV = P^T dO
// (the mathematics of cuda/attention.cu:72-231 without its T x T buffers; the contract of
// flash_attention_backward, cuda/kernels.cuh:428-437).  Two kernels, so that every output element is summed inside
// one CTA in a fixed order (no atomics): dQ per 128-row query tile, dK / dV per 128-row key tile.

constexpr int FB_DQ_SMEM_BYTES = 1024 + 2 * FA_TILE_BYTES /*Q, dO*/ + FA_KV_STAGES * 2 * FA_TILE_BYTES /*K, V stages*/ +
                                 2 * 2 * FA_TILE_BYTES /*dS x 2*/ + 1024;

// dS through tensor memory: five K/V stages, one tile of output staging where the dS buffers were
constexpr int FB_DQ_SMEM_BYTES_TS = 1024 + 2 * FA_TILE_BYTES + FA_KV_STAGES_TS * 2 * FA_TILE_BYTES + FA_TILE_BYTES + 1024;

struct FbParams {
    int B, T, n_head, n_kv_head;
    float scale_log2e;     // log2(e) / sqrt(head_dim)
    float scale;           // 1 / sqrt(head_dim)
    const float* lse;      // [B, n_head, T]
    const float* delta;    // [B, n_head, T]
    int* status;
};

struct alignas(8) FbDqCtrl {
    unsigned long long q_full;
    unsigned long long kv_full[FA_KV_STAGES_MAX], kv_empty[FA_KV_STAGES_MAX];
    unsigned long long s_full[2], s_empty[2];      // S double-buffered in TMEM
    unsigned long long dp_full, dp_empty;          // dP single-buffered
    unsigned long long ds_full[2], ds_empty[2];    // dS (bf16) double-buffered in shared memory
    unsigned long long dq_full;                    // all products accumulated
    uint32_t tmem_base;
    int abort_flag;
};

// dQ for one (batch, query head, 128 query rows): per key tile S = Q K^T and dP = dO V^T on the tensor cores, the four
// softmax warps turn them into dS (bf16, K-major in shared memory), and dQ += dS K accumulates in TMEM over all tiles.
// tmQ / tmdO / tmdQ: {n_head*64, T, B}, box {64,128,1};  tmK / tmV: {n_kv_head*64, T, B}, box {64,128,1}.
// NS = softmax threads per query row (2 or 4), as in the forward kernel: 128 / NS key columns each.
// DS_TMEM: dS goes back to tensor memory as bf16 (over the first half of each 32-column group of the S buffer) and is
// the left operand of dS K from there, instead of through shared memory.
template <int NS, bool DS_TMEM>
__global__ void __launch_bounds__(128 + NS * 128, 1)
attn_bwd_dq_sm100(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                  const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                  const __grid_constant__ CUtensorMap tmdQ, const FbParams p) {
    constexpr int STAGES = DS_TMEM ? FA_KV_STAGES_TS : FA_KV_STAGES;
    extern __shared__ uint8_t fa_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    FbDqCtrl* ctrl = reinterpret_cast<FbDqCtrl*>(smem);
    uint8_t* sQ = smem + 1024;
    uint8_t* sdO = sQ + FA_TILE_BYTES;
    uint8_t* sKV = sdO + FA_TILE_BYTES;                       // stage s: [K tile | V tile]
    uint8_t* sdS = sKV + STAGES * 2 * FA_TILE_BYTES;    // buffer b: [key columns 0..63 | 64..127]
    volatile int* abort_flag = &ctrl->abort_flag;

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int qt = gridDim.z - 1 - blockIdx.z, h = blockIdx.x, b = blockIdx.y;   // longest first, as in the forward kernel
    const int kvh = h / (p.n_head / p.n_kv_head);
    const int n_kv = qt + 1;

    if (warp == 1 && lane == 0) {
        mbar_init(smem_u32(&ctrl->q_full), 1);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(smem_u32(&ctrl->kv_full[i]), 1);
            mbar_init(smem_u32(&ctrl->kv_empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&ctrl->s_full[i]), 1);
            mbar_init(smem_u32(&ctrl->s_empty[i]), DS_TMEM ? 1 : (4 * NS));   // DS_TMEM: freed by the tensor core after dS K
            mbar_init(smem_u32(&ctrl->ds_full[i]), (4 * NS));
            mbar_init(smem_u32(&ctrl->ds_empty[i]), 1);
        }
        mbar_init(smem_u32(&ctrl->dp_full), 1);
        mbar_init(smem_u32(&ctrl->dp_empty), (4 * NS));
        mbar_init(smem_u32(&ctrl->dq_full), 1);
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmdO);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmdQ);
    }
    if (warp == 2) {
        tmem_alloc<1>(smem_u32(&ctrl->tmem_base), FA_TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_sync();   // everything above touches no global memory and may overlap the previous kernel's tail
    const uint32_t tmem_base = ctrl->tmem_base;
    const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 256, tmem_dQ = tmem_base + 384;   // S[b] at +128 b

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        const bool issuer = elect_one();
        if (issuer) {
            mbar_arrive_expect_tx(smem_u32(&ctrl->q_full), 2 * FA_TILE_BYTES);
            tma_load_3d(smem_u32(sQ), &tmQ, smem_u32(&ctrl->q_full), h * FA_HD, qt * FA_BQ, b);
            tma_load_3d(smem_u32(sdO), &tmdO, smem_u32(&ctrl->q_full), h * FA_HD, qt * FA_BQ, b);
        }
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            const int s = j % STAGES;
            ok = mbar_wait(smem_u32(&ctrl->kv_empty[s]), ((j / STAGES) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (issuer) {
                const uint32_t bar = smem_u32(&ctrl->kv_full[s]);
                const uint32_t dst = smem_u32(sKV + s * 2 * FA_TILE_BYTES);
                mbar_arrive_expect_tx(bar, 2 * FA_TILE_BYTES);
                tma_load_3d(dst, &tmK, bar, kvh * FA_HD, j * FA_BKV, b);
                tma_load_3d(dst + FA_TILE_BYTES, &tmV, bar, kvh * FA_HD, j * FA_BKV, b);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_S = umma_idesc(1, FA_BQ, FA_BKV, 0, 0);    // Q / dO and K / V: K-major
        constexpr uint32_t idesc_dQ = umma_idesc(1, FA_BQ, FA_HD, 0, 1);    // dS: K-major, K tile: MN-major
        const bool issuer = elect_one();
        const uint64_t descQ = umma_smem_desc(smem_u32(sQ), 16, 1024);
        const uint64_t descdO = umma_smem_desc(smem_u32(sdO), 16, 1024);
        bool ok = mbar_wait(smem_u32(&ctrl->q_full), 0, abort_flag, p.status, DEV_TIMEOUT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        for (int j = 0; j <= n_kv && ok; ++j) {
            if (j < n_kv) {   // S_j = Q K_j^T and dP_j = dO V_j^T
                const int s = j & 1, st = j % STAGES;
                ok = mbar_wait(smem_u32(&ctrl->kv_full[st]), (j / STAGES) & 1, abort_flag, p.status, DEV_TIMEOUT_FULL) &&
                     mbar_wait(smem_u32(&ctrl->s_empty[s]), ((j >> 1) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_E);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t kaddr = smem_u32(sKV + st * 2 * FA_TILE_BYTES);
                if (issuer) {
                    const uint64_t descK = umma_smem_desc(kaddr, 16, 1024);
#pragma unroll
                    for (int k = 0; k < FA_HD / UMMA_K; ++k)
                        umma_f16<1>(tmem_S + s * 128, descQ + ((k * UMMA_K * 2) >> 4), descK + ((k * UMMA_K * 2) >> 4), idesc_S,
                                    k > 0 ? 1u : 0u);
                    umma_commit(smem_u32(&ctrl->s_full[s]));
                }
                ok = mbar_wait(smem_u32(&ctrl->dp_empty), (j & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_E);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (issuer) {
                    const uint64_t descV = umma_smem_desc(kaddr + FA_TILE_BYTES, 16, 1024);
#pragma unroll
                    for (int k = 0; k < FA_HD / UMMA_K; ++k)
                        umma_f16<1>(tmem_dP, descdO + ((k * UMMA_K * 2) >> 4), descV + ((k * UMMA_K * 2) >> 4), idesc_S,
                                    k > 0 ? 1u : 0u);
                    umma_commit(smem_u32(&ctrl->dp_full));
                }
            }
            if (j >= 1) {     // dQ += dS_i K_i for the tile before
                const int i = j - 1, s = i & 1, st = i % STAGES;
                ok = mbar_wait(smem_u32(&ctrl->ds_full[s]), (i >> 1) & 1, abort_flag, p.status, DEV_TIMEOUT_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (issuer) {
                    const uint64_t descKm = umma_smem_desc(smem_u32(sKV + st * 2 * FA_TILE_BYTES), 64 * 64 * 2, 1024);
                    const uint32_t dsbase = smem_u32(sdS + s * 2 * FA_TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < FA_BKV / UMMA_K; ++k) {
                        if constexpr (DS_TMEM) {
                            // dS of keys 16 k .. 16 k + 15: 8 packed columns in the first half of 32-column group k / 2 of S
                            umma_f16_ts(tmem_dQ, tmem_S + s * 128 + (k >> 1) * 32 + (k & 1) * 8, descKm + ((k * UMMA_K * 128) >> 4),
                                        idesc_dQ, (i > 0 || k > 0) ? 1u : 0u);
                        } else {
                            const uint64_t descdS = umma_smem_desc(dsbase + (k >> 2) * FA_TILE_BYTES + (k & 3) * UMMA_K * 2, 16, 1024);
                            umma_f16<1>(tmem_dQ, descdS, descKm + ((k * UMMA_K * 128) >> 4), idesc_dQ, (i > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(smem_u32(&ctrl->kv_empty[st]));
                    if constexpr (DS_TMEM) umma_commit(smem_u32(&ctrl->s_empty[s]));   // dS lived in this S buffer
                    else umma_commit(smem_u32(&ctrl->ds_empty[s]));
                    if (i == n_kv - 1) umma_commit(smem_u32(&ctrl->dq_full));
                }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ dS + epilogue
        const int qrt = warp & 3;
        const int part = (warp - 4) >> 2;   // which 128 / NS key columns (and which 64 / NS columns of dQ) of the row
        constexpr int HC = FA_BKV / NS, OC = FA_HD / NS;
        const int r = qrt * 32 + lane;
        const int row = qt * FA_BQ + r;
        const uint32_t lane_off = static_cast<uint32_t>(qrt * 32) << 16;
        const bool row_ok = row < p.T;
        const long long stat_idx = (static_cast<long long>(b) * p.n_head + h) * p.T + row;
        const float lse2 = row_ok ? p.lse[stat_idx] * 1.4426950408889634f : 0.f;   // in units of log2
        const float delta = row_ok ? p.delta[stat_idx] : 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            const int s = j & 1;
            ok = mbar_wait(smem_u32(&ctrl->s_full[s]), (j >> 1) & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_F) &&
                 mbar_wait(smem_u32(&ctrl->dp_full), j & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_F);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tS = tmem_S + s * 128 + lane_off + part * HC, tP = tmem_dP + lane_off + part * HC;
            // only the diagonal tile and the tiles that reach beyond the sequence need a mask
            const bool masked = j == qt || (j + 1) * FA_BKV > p.T || (qt + 1) * FA_BQ > p.T;
            const int col0 = j * FA_BKV + part * HC;
            uint8_t* dsrow = sdS + s * 2 * FA_TILE_BYTES + r * 128;
            // This thread's columns of dP come into registers at once and the (single) dP accumulator is handed back
            // before any arithmetic: the tensor core forms dP of the next tile while this one is turned into dS.
            uint32_t dv[HC], sv[32];
#pragma unroll
            for (int c = 0; c < HC / 32; ++c) tmem_ld_32x32(tP + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&dv[c * 32]));
            tmem_ld_32x32(tS, sv);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&ctrl->dp_empty));
                if (HC == 32 && !DS_TMEM) mbar_arrive(smem_u32(&ctrl->s_empty[s]));   // its only 32 columns of S are in registers too
            }
            if constexpr (!DS_TMEM) {
                // the tensor core must have finished reading this dS buffer (tile j - 2)
                ok = mbar_wait(smem_u32(&ctrl->ds_empty[s]), ((j >> 1) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
#pragma unroll
            for (int c = 0; c < HC / 32; ++c) {
                if (c == 1) {
                    tmem_ld_32x32(tS + 32, sv);
                    tmem_ld_wait();
                    if constexpr (!DS_TMEM) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&ctrl->s_empty[s]));
                    }
                }
                uint32_t packed[16];
                if (masked) {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const int col = col0 + c * 32 + e;
                        float x0 = fmaf(__uint_as_float(sv[e]), p.scale_log2e, -lse2), x1 = fmaf(__uint_as_float(sv[e + 1]), p.scale_log2e, -lse2);
                        if (col > row || col >= p.T || !row_ok) x0 = -INFINITY;
                        if (col + 1 > row || col + 1 >= p.T || !row_ok) x1 = -INFINITY;
                        packed[e >> 1] = pack_bf16x2(fa_exp2(x0) * (__uint_as_float(dv[c * 32 + e]) - delta),
                                                     fa_exp2(x1) * (__uint_as_float(dv[c * 32 + e + 1]) - delta));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float x0 = fmaf(__uint_as_float(sv[e]), p.scale_log2e, -lse2), x1 = fmaf(__uint_as_float(sv[e + 1]), p.scale_log2e, -lse2);
                        packed[e >> 1] = pack_bf16x2(fa_exp2(x0) * (__uint_as_float(dv[c * 32 + e]) - delta),
                                                     fa_exp2(x1) * (__uint_as_float(dv[c * 32 + e + 1]) - delta));
                    }
                }
                const int g32 = part * (HC / 32) + c;   // 32-column group of the tile: panel g32 >> 1, half-row g32 & 1
                if constexpr (DS_TMEM) {
                    // over the first 16 columns of the group's own S columns (already in this thread's registers)
                    tmem_st_32x16(tmem_S + s * 128 + lane_off + g32 * 32, packed);
                } else {
                    uint8_t* panel = dsrow + (g32 >> 1) * FA_TILE_BYTES;
#pragma unroll
                    for (int qd = 0; qd < 4; ++qd) {
                        const int chunk = ((g32 & 1) * 4 + qd) ^ (r & 7);
                        *reinterpret_cast<uint4*>(panel + chunk * 16) =
                            make_uint4(packed[4 * qd], packed[4 * qd + 1], packed[4 * qd + 2], packed[4 * qd + 3]);
                    }
                }
            }
            if constexpr (DS_TMEM) {
                tmem_st_wait();
                tc_fence_before();
            } else {
                fence_proxy_async_smem();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->ds_full[s]));
        }
        if (ok) {
            ok = mbar_wait(smem_u32(&ctrl->dq_full), 0, abort_flag, p.status, DEV_TIMEOUT_TMEM_F);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after();
            uint8_t* orow = sdS + r * 128;   // every tensor-core read of the dS buffers has completed
#pragma unroll
            for (int g = 0; g < OC / 16; ++g) {
                uint32_t v[16];
                tmem_ld_32x16(tmem_dQ + lane_off + part * OC + g * 16, v);
                tmem_ld_wait();
#pragma unroll
                for (int qd = 0; qd < 2; ++qd) {
                    float x[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[e] = __uint_as_float(v[qd * 8 + e]) * p.scale;
                    const int chunk = (part * (OC / 8) + g * 2 + qd) ^ (r & 7);
                    *reinterpret_cast<uint4*>(orow + chunk * 16) =
                        make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
                }
            }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, %0;" ::"n"(NS * 128) : "memory");   // all softmax warps arrive here exactly once
        if (warp == 4 && !*abort_flag) {
            if (elect_one()) {
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                                 reinterpret_cast<uint64_t>(&tmdQ)),
                             "r"(smem_u32(sdS)), "r"(h * FA_HD), "r"(qt * FA_BQ), "r"(b)
                             : "memory");
                tma_store_commit();
                tma_store_wait_read<0>();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, FA_TMEM_COLS);
    }
}

constexpr int FB_QDO_STAGES = 2;
constexpr int FB_QDO_STAGES_KT = 4;   // transposed form: no P / dS in shared memory, two more Q / dO stages instead
constexpr int FB_QDO_STAGES_MAX = 4;
constexpr int FB_DKV_SMEM_BYTES = 1024 + 2 * FA_TILE_BYTES /*K, V*/ + FB_QDO_STAGES * 2 * FA_TILE_BYTES /*Q, dO stages*/ +
                                  2 * 4 * FA_TILE_BYTES /*(P, dS) x 2, two 64-column panels each*/ + 1024;

// transposed form: four Q / dO stages; where P / dS were: two tiles of output staging and the 3 KB of row statistics
constexpr int FB_DKV_SMEM_BYTES_KT = 1024 + 2 * FA_TILE_BYTES + 4 * 2 * FA_TILE_BYTES + 2 * FA_TILE_BYTES + 4096 + 1024;

struct alignas(8) FbDkvCtrl {
    unsigned long long kv_full;
    unsigned long long qdo_full[FB_QDO_STAGES_MAX], qdo_empty[FB_QDO_STAGES_MAX];
    unsigned long long s_full[2], s_empty[2];
    unsigned long long dp_full, dp_empty;
    unsigned long long pds_full[2], pds_empty[2];   // P and dS (bf16) in shared memory, double-buffered
    unsigned long long dkv_full;
    unsigned long long stat_full[3];                // transposed form: the iteration's lse / delta are in shared memory
    uint32_t tmem_base;
    int abort_flag;
};

// dK, dV for one (batch, KV head, 128 key rows).  Iterations run over the query heads of the group and the query
// tiles at or after the key tile.  Per iteration S = Q K^T and dP = dO V^T (rows = queries, as in the other kernels), the
// softmax warps write P and dS as bf16 [query][key] tiles, and the tensor core reads those tiles as MN-major left
// operands (their rows are the contraction): dV += P^T dO and dK += dS^T Q accumulate in TMEM over all iterations.
// tmQ / tmdO: {n_head*64, T, B};  tmK / tmV / tmdK / tmdV: {n_kv_head*64, T, B};  boxes {64,128,1}.
// KT ("keys on the lanes"): the two score products are formed transposed, S^T = K Q^T and dP^T = V dO^T, so that a
// thread owns a KEY row and P^T, dS^T have the keys along the TMEM lanes: written back as bf16 over the thread's own
// S^T columns (P^T in the first, dS^T in the second 16 columns of each 32-column group) they are the tensor core's
// left operands of dV += P^T dO and dK += dS^T Q straight from tensor memory.  No P / dS in shared memory: the
// kernel's shared-memory traffic per iteration halves.  The per-query statistics (lse, delta) now vary along the
// columns and come through a small double-buffered array in shared memory.
template <int NS, bool KT>   // NS: softmax threads per row of the score tile (2 or 4)
__global__ void __launch_bounds__(128 + NS * 128, 1)
attn_bwd_dkv_sm100(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV, const FbParams p) {
    constexpr int STAGES = KT ? FB_QDO_STAGES_KT : FB_QDO_STAGES;
    extern __shared__ uint8_t fa_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    FbDkvCtrl* ctrl = reinterpret_cast<FbDkvCtrl*>(smem);
    uint8_t* sK = smem + 1024;
    uint8_t* sV = sK + FA_TILE_BYTES;
    uint8_t* sQdO = sV + FA_TILE_BYTES;                        // stage s: [Q tile | dO tile]
    uint8_t* sPdS = sQdO + STAGES * 2 * FA_TILE_BYTES;  // buffer b: [P: 2 panels | dS: 2 panels]
    volatile int* abort_flag = &ctrl->abort_flag;

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int kt = blockIdx.z, kvh = blockIdx.x, b = blockIdx.y;   // key tile 0 meets every query tile: longest first
    const int ratio = p.n_head / p.n_kv_head;
    const int q_tiles = (p.T + FA_BQ - 1) / FA_BQ;
    const int n_q = q_tiles - kt;          // query tiles kt .. q_tiles-1 see this key tile
    const int n_it = ratio * n_q;

    if (warp == 1 && lane == 0) {
        mbar_init(smem_u32(&ctrl->kv_full), 1);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(smem_u32(&ctrl->qdo_full[i]), 1);
            mbar_init(smem_u32(&ctrl->qdo_empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&ctrl->s_full[i]), 1);
            mbar_init(smem_u32(&ctrl->s_empty[i]), KT ? 1 : (4 * NS));   // KT: freed by the tensor core after dV, dK
            mbar_init(smem_u32(&ctrl->pds_full[i]), (4 * NS));
            mbar_init(smem_u32(&ctrl->pds_empty[i]), 1);
        }
        mbar_init(smem_u32(&ctrl->dp_full), 1);
        mbar_init(smem_u32(&ctrl->dp_empty), (4 * NS));
        mbar_init(smem_u32(&ctrl->dkv_full), 1);
        for (int i = 0; i < 3; ++i) mbar_init(smem_u32(&ctrl->stat_full[i]), 4);
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmdO);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmdK);
        tma_prefetch_desc(&tmdV);
    }
    if (warp == 2) {
        tmem_alloc<1>(smem_u32(&ctrl->tmem_base), FA_TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_sync();   // everything above touches no global memory and may overlap the previous kernel's tail
    const uint32_t tmem_base = ctrl->tmem_base;
    const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 256, tmem_dV = tmem_base + 384, tmem_dK = tmem_base + 448;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        const bool issuer = elect_one();
        if (issuer) {
            mbar_arrive_expect_tx(smem_u32(&ctrl->kv_full), 2 * FA_TILE_BYTES);
            tma_load_3d(smem_u32(sK), &tmK, smem_u32(&ctrl->kv_full), kvh * FA_HD, kt * FA_BKV, b);
            tma_load_3d(smem_u32(sV), &tmV, smem_u32(&ctrl->kv_full), kvh * FA_HD, kt * FA_BKV, b);
        }
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            const int s = it % STAGES;
            const int h = kvh * ratio + it / n_q, i = kt + it % n_q;
            ok = mbar_wait(smem_u32(&ctrl->qdo_empty[s]), ((it / STAGES) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (issuer) {
                const uint32_t bar = smem_u32(&ctrl->qdo_full[s]);
                const uint32_t dst = smem_u32(sQdO + s * 2 * FA_TILE_BYTES);
                mbar_arrive_expect_tx(bar, 2 * FA_TILE_BYTES);
                tma_load_3d(dst, &tmQ, bar, h * FA_HD, i * FA_BQ, b);
                tma_load_3d(dst + FA_TILE_BYTES, &tmdO, bar, h * FA_HD, i * FA_BQ, b);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_S = umma_idesc(1, FA_BQ, FA_BKV, 0, 0);     // Q / dO and K / V: K-major
        constexpr uint32_t idesc_T = umma_idesc(1, FA_BKV, FA_HD, 1, 1);     // P / dS and dO / Q: MN-major (contraction = query rows)
        const bool issuer = elect_one();
        const uint64_t descK = umma_smem_desc(smem_u32(sK), 16, 1024);
        const uint64_t descV = umma_smem_desc(smem_u32(sV), 16, 1024);
        bool ok = mbar_wait(smem_u32(&ctrl->kv_full), 0, abort_flag, p.status, DEV_TIMEOUT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        for (int it = 0; it <= n_it && ok; ++it) {
            if (it < n_it) {   // S = Q K^T, dP = dO V^T
                const int s = it & 1, st = it % STAGES;
                ok = mbar_wait(smem_u32(&ctrl->qdo_full[st]), (it / STAGES) & 1, abort_flag, p.status, DEV_TIMEOUT_FULL) &&
                     mbar_wait(smem_u32(&ctrl->s_empty[s]), ((it >> 1) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_E);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t qaddr = smem_u32(sQdO + st * 2 * FA_TILE_BYTES);
                if (issuer) {
                    const uint64_t descQ = umma_smem_desc(qaddr, 16, 1024);
#pragma unroll
                    for (int k = 0; k < FA_HD / UMMA_K; ++k)   // S = Q K^T, or S^T = K Q^T (both operands K-major either way)
                        umma_f16<1>(tmem_S + s * 128, (KT ? descK : descQ) + ((k * UMMA_K * 2) >> 4),
                                    (KT ? descQ : descK) + ((k * UMMA_K * 2) >> 4), idesc_S, k > 0 ? 1u : 0u);
                    umma_commit(smem_u32(&ctrl->s_full[s]));
                }
                ok = mbar_wait(smem_u32(&ctrl->dp_empty), (it & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_E);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (issuer) {
                    const uint64_t descdO = umma_smem_desc(qaddr + FA_TILE_BYTES, 16, 1024);
#pragma unroll
                    for (int k = 0; k < FA_HD / UMMA_K; ++k)   // dP = dO V^T, or dP^T = V dO^T
                        umma_f16<1>(tmem_dP, (KT ? descV : descdO) + ((k * UMMA_K * 2) >> 4),
                                    (KT ? descdO : descV) + ((k * UMMA_K * 2) >> 4), idesc_S, k > 0 ? 1u : 0u);
                    umma_commit(smem_u32(&ctrl->dp_full));
                }
            }
            if (it >= 1) {     // dV += P^T dO, dK += dS^T Q for the iteration before
                const int i = it - 1, s = i & 1, st = i % STAGES;
                ok = mbar_wait(smem_u32(&ctrl->pds_full[s]), (i >> 1) & 1, abort_flag, p.status, DEV_TIMEOUT_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (issuer) {
                    const uint32_t pbase = smem_u32(sPdS + s * 4 * FA_TILE_BYTES);
                    const uint32_t qaddr = smem_u32(sQdO + st * 2 * FA_TILE_BYTES);
                    // left operands: 128 contraction rows (queries) of 128 bytes per 64-key panel, panels 16 KB apart;
                    // right operands: 128 contraction rows of 128 bytes (one 64-wide panel); 16 rows = 2048 bytes per MMA
                    const uint64_t descP = umma_smem_desc(pbase, FA_TILE_BYTES, 1024);
                    const uint64_t descdS = umma_smem_desc(pbase + 2 * FA_TILE_BYTES, FA_TILE_BYTES, 1024);
                    const uint64_t descQm = umma_smem_desc(qaddr, 64 * 64 * 2, 1024);
                    const uint64_t descdOm = umma_smem_desc(qaddr + FA_TILE_BYTES, 64 * 64 * 2, 1024);
                    if constexpr (KT) {
                        constexpr uint32_t idesc_TS = umma_idesc(1, FA_BKV, FA_HD, 0, 1);   // left operand from TMEM, dO / Q MN-major
#pragma unroll
                        for (int k = 0; k < FA_BQ / UMMA_K; ++k)   // queries 16 k .. 16 k + 15: 8 packed columns of group k / 2
                            umma_f16_ts(tmem_dV, tmem_S + s * 128 + (k >> 1) * 32 + (k & 1) * 8, descdOm + ((k * UMMA_K * 128) >> 4),
                                        idesc_TS, (i > 0 || k > 0) ? 1u : 0u);
#pragma unroll
                        for (int k = 0; k < FA_BQ / UMMA_K; ++k)
                            umma_f16_ts(tmem_dK, tmem_S + s * 128 + (k >> 1) * 32 + 16 + (k & 1) * 8, descQm + ((k * UMMA_K * 128) >> 4),
                                        idesc_TS, (i > 0 || k > 0) ? 1u : 0u);
                        umma_commit(smem_u32(&ctrl->qdo_empty[st]));
                        umma_commit(smem_u32(&ctrl->s_empty[s]));   // P^T and dS^T lived in this S buffer
                    } else {
#pragma unroll
                        for (int k = 0; k < FA_BQ / UMMA_K; ++k)
                            umma_f16<1>(tmem_dV, descP + ((k * UMMA_K * 128) >> 4), descdOm + ((k * UMMA_K * 128) >> 4), idesc_T,
                                        (i > 0 || k > 0) ? 1u : 0u);
#pragma unroll
                        for (int k = 0; k < FA_BQ / UMMA_K; ++k)
                            umma_f16<1>(tmem_dK, descdS + ((k * UMMA_K * 128) >> 4), descQm + ((k * UMMA_K * 128) >> 4), idesc_T,
                                        (i > 0 || k > 0) ? 1u : 0u);
                        umma_commit(smem_u32(&ctrl->qdo_empty[st]));
                        umma_commit(smem_u32(&ctrl->pds_empty[s]));
                    }
                    if (i == n_it - 1) umma_commit(smem_u32(&ctrl->dkv_full));
                }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ P, dS + epilogue
        const int qrt = warp & 3;
        const int part = (warp - 4) >> 2;   // which 128 / NS key columns of the row; in the epilogue: a share of dV or of dK
        constexpr int HC = FA_BKV / NS;
        const int r = qrt * 32 + lane;
        const uint32_t lane_off = static_cast<uint32_t>(qrt * 32) << 16;
        bool ok = true;
        // the row statistics of an iteration are fetched one iteration ahead, off the critical path
        auto stats = [&](int it, float& lse2, float& delta) {
            const int h = kvh * ratio + it / n_q, i = kt + it % n_q;
            const int row = i * FA_BQ + r;
            const long long stat_idx = (static_cast<long long>(b) * p.n_head + h) * p.T + row;
            const bool row_ok = row < p.T;
            lse2 = row_ok ? p.lse[stat_idx] * 1.4426950408889634f : 0.f;
            delta = row_ok ? p.delta[stat_idx] : 0.f;
        };
        float lse2_next = 0.f, delta_next = 0.f;
        if (n_it > 0) stats(0, lse2_next, delta_next);
        if constexpr (KT) {
            // keys on the lanes: this thread owns key row `key` of the tile and HC query columns of S^T and dP^T
            // [3 buffers][lse2: 128 | delta: 128].  Three, not two: a thread that starts iteration it has seen S^T of
            // iteration it - 1, which the tensor core forms only after every warp finished iteration it - 3 -- nothing
            // later is guaranteed, so the buffer written at it must not be the one read at it - 2.
            float* stat = reinterpret_cast<float*>(sPdS + 2 * FA_TILE_BYTES);
            const int key = kt * FA_BKV + r;
            for (int it = 0; it < n_it && ok; ++it) {
                const int s = it & 1;
                const int i = kt + it % n_q;
                // the statistics of this iteration's 128 queries: the part-0 thread of a row publishes the pair it
                // fetched one iteration ago (stats() indexes by r = query row here), everybody reads them by column
                const int sb = it % 3;
                if (part == 0) {
                    stat[sb * 256 + r] = lse2_next;
                    stat[sb * 256 + 128 + r] = delta_next;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&ctrl->stat_full[sb]));
                    if (it + 1 < n_it) stats(it + 1, lse2_next, delta_next);
                }
                ok = mbar_wait(smem_u32(&ctrl->s_full[s]), (it >> 1) & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_F) &&
                     mbar_wait(smem_u32(&ctrl->dp_full), it & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_F) &&
                     mbar_wait(smem_u32(&ctrl->stat_full[sb]), (it / 3) & 1, abort_flag, p.status, DEV_TIMEOUT_PEER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tS = tmem_S + s * 128 + lane_off + part * HC, tP = tmem_dP + lane_off + part * HC;
                const bool masked = i == kt || (kt + 1) * FA_BKV > p.T || (i + 1) * FA_BQ > p.T;
                const int q0 = i * FA_BQ + part * HC;            // first query position of this thread's columns
                const float4* lse4 = reinterpret_cast<const float4*>(stat + sb * 256 + part * HC);
                const float4* del4 = reinterpret_cast<const float4*>(stat + sb * 256 + 128 + part * HC);
                uint32_t dv[HC], sv[32];
#pragma unroll
                for (int c = 0; c < HC / 32; ++c) tmem_ld_32x32(tP + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&dv[c * 32]));
                tmem_ld_32x32(tS, sv);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctrl->dp_empty));
#pragma unroll
                for (int c = 0; c < HC / 32; ++c) {
                    if (c == 1) {
                        tmem_ld_32x32(tS + 32, sv);
                        tmem_ld_wait();
                    }
                    uint32_t pp[16], pd[16];
#pragma unroll
                    for (int e4 = 0; e4 < 8; ++e4) {              // four queries at a time: one 16-byte read of each statistic
                        const float4 l4 = lse4[c * 8 + e4], d4 = del4[c * 8 + e4];
                        const float lq[4] = {l4.x, l4.y, l4.z, l4.w}, dq4[4] = {d4.x, d4.y, d4.z, d4.w};
                        float pv[4], dsv[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int e = e4 * 4 + u;
                            float x = fmaf(__uint_as_float(sv[e]), p.scale_log2e, -lq[u]);
                            if (masked) {
                                const int query = q0 + c * 32 + e;
                                if (key > query || key >= p.T || query >= p.T) x = -INFINITY;
                            }
                            pv[u] = fa_exp2(x);
                            dsv[u] = pv[u] * (__uint_as_float(dv[c * 32 + e]) - dq4[u]);
                        }
                        pp[e4 * 2] = pack_bf16x2(pv[0], pv[1]);
                        pp[e4 * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
                        pd[e4 * 2] = pack_bf16x2(dsv[0], dsv[1]);
                        pd[e4 * 2 + 1] = pack_bf16x2(dsv[2], dsv[3]);
                    }
                    // P^T over the first, dS^T over the second 16 columns of this 32-column group of S^T (already in registers)
                    const int g32 = part * (HC / 32) + c;
                    tmem_st_32x16(tmem_S + s * 128 + lane_off + g32 * 32, pp);
                    tmem_st_32x16(tmem_S + s * 128 + lane_off + g32 * 32 + 16, pd);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctrl->pds_full[s]));
            }
        } else {
        for (int it = 0; it < n_it && ok; ++it) {
            const int s = it & 1;
            const int i = kt + it % n_q;
            const int row = i * FA_BQ + r;                      // query position of this thread in this iteration
            const bool row_ok = row < p.T;
            const float lse2 = lse2_next, delta = delta_next;
            if (it + 1 < n_it) stats(it + 1, lse2_next, delta_next);
            ok = mbar_wait(smem_u32(&ctrl->s_full[s]), (it >> 1) & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_F) &&
                 mbar_wait(smem_u32(&ctrl->dp_full), it & 1, abort_flag, p.status, DEV_TIMEOUT_TMEM_F);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tS = tmem_S + s * 128 + lane_off + part * HC, tP = tmem_dP + lane_off + part * HC;
            const bool masked = i == kt || (kt + 1) * FA_BKV > p.T || (i + 1) * FA_BQ > p.T;
            const int col0 = kt * FA_BKV + part * HC;
            uint8_t* prow = sPdS + s * 4 * FA_TILE_BYTES + r * 128;
            uint8_t* dsrow = prow + 2 * FA_TILE_BYTES;
            // as in the dQ kernel: dP into registers at once, its accumulator handed back before the arithmetic
            uint32_t dv[HC], sv[32];
#pragma unroll
            for (int c = 0; c < HC / 32; ++c) tmem_ld_32x32(tP + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&dv[c * 32]));
            tmem_ld_32x32(tS, sv);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&ctrl->dp_empty));
                if (HC == 32) mbar_arrive(smem_u32(&ctrl->s_empty[s]));
            }
            ok = mbar_wait(smem_u32(&ctrl->pds_empty[s]), ((it >> 1) & 1) ^ 1, abort_flag, p.status, DEV_TIMEOUT_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
#pragma unroll
            for (int c = 0; c < HC / 32; ++c) {
                if (c == 1) {
                    tmem_ld_32x32(tS + 32, sv);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&ctrl->s_empty[s]));
                }
                uint32_t pp[16], pd[16];
                if (masked) {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const int col = col0 + c * 32 + e;
                        float x0 = fmaf(__uint_as_float(sv[e]), p.scale_log2e, -lse2), x1 = fmaf(__uint_as_float(sv[e + 1]), p.scale_log2e, -lse2);
                        if (col > row || col >= p.T || !row_ok) x0 = -INFINITY;
                        if (col + 1 > row || col + 1 >= p.T || !row_ok) x1 = -INFINITY;
                        const float p0 = fa_exp2(x0), p1 = fa_exp2(x1);
                        pp[e >> 1] = pack_bf16x2(p0, p1);
                        pd[e >> 1] = pack_bf16x2(p0 * (__uint_as_float(dv[c * 32 + e]) - delta), p1 * (__uint_as_float(dv[c * 32 + e + 1]) - delta));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float p0 = fa_exp2(fmaf(__uint_as_float(sv[e]), p.scale_log2e, -lse2));
                        const float p1 = fa_exp2(fmaf(__uint_as_float(sv[e + 1]), p.scale_log2e, -lse2));
                        pp[e >> 1] = pack_bf16x2(p0, p1);
                        pd[e >> 1] = pack_bf16x2(p0 * (__uint_as_float(dv[c * 32 + e]) - delta), p1 * (__uint_as_float(dv[c * 32 + e + 1]) - delta));
                    }
                }
                const int g32 = part * (HC / 32) + c;   // 32-column group of the tile: panel g32 >> 1, half-row g32 & 1
                const int poff = (g32 >> 1) * FA_TILE_BYTES;
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    const int chunk = ((g32 & 1) * 4 + qd) ^ (r & 7);
                    *reinterpret_cast<uint4*>(prow + poff + chunk * 16) = make_uint4(pp[4 * qd], pp[4 * qd + 1], pp[4 * qd + 2], pp[4 * qd + 3]);
                    *reinterpret_cast<uint4*>(dsrow + poff + chunk * 16) = make_uint4(pd[4 * qd], pd[4 * qd + 1], pd[4 * qd + 2], pd[4 * qd + 3]);
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->pds_full[s]));
        }
        }
        if (ok) {
            ok = mbar_wait(smem_u32(&ctrl->dkv_full), 0, abort_flag, p.status, DEV_TIMEOUT_TMEM_F);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after();
            // the 2 x 64 output columns of key row r (dV, then dK) are shared out to the row's NS threads; staged in the
            // (free) P / dS buffers
            constexpr int OC = 2 * FA_HD / NS;                 // 64 (NS = 2) or 32 (NS = 4) columns per thread
            const int which = (part * OC) / FA_HD;             // 0: dV, 1: dK
            const int c_first = (part * OC) % FA_HD;           // first column inside that matrix
            uint8_t* orow = sPdS + which * FA_TILE_BYTES + r * 128;
            const float mul = which == 0 ? 1.0f : p.scale;
#pragma unroll
            for (int c = 0; c < OC / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32((which == 0 ? tmem_dV : tmem_dK) + lane_off + c_first + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    float x[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[e] = __uint_as_float(v[qd * 8 + e]) * mul;
                    const int chunk = ((c_first + c * 32) / 8 + qd) ^ (r & 7);
                    *reinterpret_cast<uint4*>(orow + chunk * 16) =
                        make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
                }
            }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, %0;" ::"n"(NS * 128) : "memory");   // all softmax warps arrive here exactly once
        if (warp == 4 && !*abort_flag) {
            if (elect_one()) {
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                                 reinterpret_cast<uint64_t>(&tmdV)),
                             "r"(smem_u32(sPdS)), "r"(kvh * FA_HD), "r"(kt * FA_BKV), "r"(b)
                             : "memory");
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                                 reinterpret_cast<uint64_t>(&tmdK)),
                             "r"(smem_u32(sPdS + FA_TILE_BYTES)), "r"(kvh * FA_HD), "r"(kt * FA_BKV), "r"(b)
                             : "memory");
                tma_store_commit();
                tma_store_wait_read<0>();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, FA_TMEM_COLS);
    }
}

}  // namespace b200
