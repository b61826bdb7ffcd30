// Persistent, warp-specialised bf16 GEMM for sm_100a:
//   TMA -> 128B-swizzled shared-memory ring -> tcgen05.mma (fp32 accumulators in
//   TMEM, double-buffered) -> epilogue warps (tcgen05.ld, fused beta=1 add and
//   bf16 down-cast, TMA store).
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
//
// Work schedule ("slot" = a CTA, or a CTA pair): the first `dp_tiles` output tiles are
// computed whole, round-robin over the slots.  The remaining tiles — the ragged last
// wave, or every tile when the output alone cannot fill the GPU — are each cut into
// `sk_splits` ranges of the contraction, one work item each, and summed in a fixed order (member
// order, not arrival order, so results are the same from run to run) in one of three ways:
// peer split (the ranges of a tile all run at once: they exchange fp32 slices through the
// workspace and each reduces and writes its own columns), last arriver (whole partial tiles
// parked in the workspace, the last to arrive adds them up), or cluster split (p.ksplit: the
// ranges are one thread-block cluster and exchange through distributed shared memory).
#pragma once
#include <cstddef>
#include <cuda_bf16.h>
#include "ptx.cuh"

namespace b200 {

constexpr int BM = 128;        // output rows per CTA = TMEM lanes
constexpr int BK = 64;         // contraction elements per stage = one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;     // contraction elements per tcgen05.mma (bf16)
constexpr int GEMM_THREADS = 384;
constexpr int EPI_WARPS = 8;     // warps 4..11
constexpr int SMEM_BUDGET = 227 * 1024;
constexpr int EPI_BUF_BYTES = 32 * 128;  // one staging buffer: 32 rows x 64 bf16, 128-byte swizzled

constexpr int GRP_NONE = 0x7FFFFFFF;

// Tensor maps of products 1 and 2 of a grouped launch (product 0 uses the kernel's first four maps).
struct alignas(64) GemmGroupMaps {
    CUtensorMap p[2], q[2], d[2], d32[2];
};
// What a launch of a single product passes in their place: nothing (a kilobyte less of kernel parameters per launch).
struct GemmNoMaps {};
// EPI (the kernel's last template parameter): 0 = one product, 1 = SwiGLU forward pair, 2 = LM-head forward with
// cross-entropy statistics, 3 = grouped launch.  1 and 3 carry the extra tensor maps.
template <int EPI>
struct GemmExtraMaps {
    using type = GemmNoMaps;
};
template <>
struct GemmExtraMaps<1> {
    using type = GemmGroupMaps;
};
template <>
struct GemmExtraMaps<3> {
    using type = GemmGroupMaps;
};

struct GemmParams {
    int Mo, No, Kc;          // output rows, output cols, contraction length
    int m_tiles, n_tiles;    // ceil(Mo/(BM*CTAS)), ceil(No/BN)
    int kb_total;            // ceil(Kc/BK)
    int m_fastest;           // tile raster: 1 = consecutive tiles walk down the rows
    int group;               // tiles of the fast dimension per group of the tile order (0 = no grouping)
    int dp_tiles;            // tiles [0, dp_tiles) are computed whole
    int sk_splits;           // tiles [dp_tiles, m_tiles*n_tiles) are cut into this many ranges
    int kb_per_sk;           // ceil(kb_total/sk_splits); every range owns >= 1 block
    int sk_items;            // (m_tiles*n_tiles - dp_tiles) * sk_splits
    int sk_peer;             // 1: the ranges of a split tile exchange partial sums among themselves (all resident
                             //    at once); 0: they park whole partial tiles and the last arriver adds them up
    int late_wait;           // 1: independent of the previous kernel in the stream: run beside its tail and
                             //    wait for it only before finishing (completion order stays stream order)
    int ksplit;              // > 1: a cluster of CTAS*ksplit CTAs shares each tile, every member takes one
                             // range of the contraction and the sum is formed through distributed smem
    int p_3d, q_3d;          // MN-major operand described by a 3-D map: one copy per stage
    // Grouped launch (up to three products in one): column tiles [0, grp_n[0]) belong to product 0,
    // [grp_n[0], grp_n[1]) to product 1, the rest to product 2, each with its own Q and D maps and its own column
    // origin ("N-concatenated": Y_i = X * W_i with X shared); contraction blocks are divided the same way by grp_k
    // ("K-concatenated": dX = sum_i dY_i * W_i^T, one accumulator), each range with its own P and Q maps.
    // GRP_NONE in all four for a single product.
    int grp_n[2], grp_k[2];
    void* out;               // bf16 [Mo,No]
    float* ws;               // split partials: sk_items * CTAS blocks of BM x BN fp32
    int* sk_counters;        // one arrival counter per (split tile, CTA of the pair); zero between launches
    int* status;             // device status word (0 = ok)
};

template <int BN, int CTAS>
struct TileCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_ROWS = BN / CTAS;           // rows of Q this CTA loads
    static constexpr int B_BYTES = B_ROWS * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int CTRL_BYTES = 1024;
    // staging buffers per epilogue warp: two, so that one TMA store can still be reading its buffer while the
    // next chunk is converted into the other (one where a second would leave fewer than 4 pipeline stages)
    static constexpr int EPI_BUFS = (BN == 256 && CTAS == 1) ? 1 : 2;
    static constexpr int EPI_BYTES = EPI_WARPS * EPI_BUFS * EPI_BUF_BYTES;
    static constexpr int STAGES_RAW = (SMEM_BUDGET - CTRL_BYTES - EPI_BYTES - 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + CTRL_BYTES + EPI_BYTES + 1024;  // +1024: manual alignment
    static constexpr int ACC_STRIDE = BN <= 64 ? 64 : (BN <= 128 ? 128 : 256);   // TMEM columns per accumulator
    static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
    static constexpr int PARTIAL_FLOATS = BM * BN;     // one CTA's fp32 partial tile
    static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "tile width");
    static_assert(CTAS == 1 || (CTAS == 2 && B_ROWS % 64 == 0), "pair tiles split Q in 64-row panels");
    static_assert(STAGES >= 3, "pipeline too shallow");
};

// One unit of work of a slot.
struct WorkItem {
    int m_blk, n_blk;   // output tile
    int kb0, kb1;       // contraction blocks [kb0, kb1)
    int sk_item;        // -1: whole tile; else index of this partial in the workspace
    int sk_tile;        // index of the split tile (counter index), when sk_item >= 0
    int sk_split;       // which range of that tile
};

// The i-th work item of `slot` (split items first, then whole tiles); false when the slot is done.
__device__ __forceinline__ bool get_work(const GemmParams& p, int slot, int nslots, int i, WorkItem& w) {
    const int my_sk = p.sk_items > slot ? (p.sk_items - slot + nslots - 1) / nslots : 0;
    int tile;
    if (i < my_sk) {
        const int u = slot + i * nslots;
        w.sk_item = u;
        w.sk_tile = u / p.sk_splits;
        const int split = u - w.sk_tile * p.sk_splits;
        w.sk_split = split;
        tile = p.dp_tiles + w.sk_tile;
        w.kb0 = split * p.kb_per_sk;
        w.kb1 = min(w.kb0 + p.kb_per_sk, p.kb_total);
    } else {
        tile = slot + (i - my_sk) * nslots;
        if (tile >= p.dp_tiles) return false;
        w.sk_item = -1;
        w.sk_tile = 0;
        w.sk_split = 0;
        w.kb0 = 0;
        w.kb1 = p.kb_total;
    }
    // Tile order: the fast dimension is walked in groups of p.group tiles (0: the whole dimension), each
    // group across the whole slow dimension before the next, so that the tiles running at one time form a
    // block of the output (about as many distinct row tiles as column tiles) instead of a thin stripe:
    // fewer distinct operand panels per wave, which is what L2 and HBM see.
    const int fast_tiles = p.m_fastest ? p.m_tiles : p.n_tiles;
    const int slow_tiles = p.m_fastest ? p.n_tiles : p.m_tiles;
    int fast, slow;
    if (p.group > 0 && p.group < fast_tiles) {
        const int per_group = p.group * slow_tiles;
        const int g = tile / per_group;
        const int r = tile - g * per_group;
        const int width = min(p.group, fast_tiles - g * p.group);  // the last group may be narrower
        slow = r / width;
        fast = g * p.group + (r - slow * width);
    } else {
        slow = tile / fast_tiles;
        fast = tile - slow * fast_tiles;
    }
    w.m_blk = p.m_fastest ? fast : slow;
    w.n_blk = p.m_fastest ? slow : fast;
    return true;
}

// Which product of a grouped launch a column tile / contraction block belongs to, and where that product starts.
__device__ __forceinline__ int group_of(int bound0, int bound1, int i, int& base) {
    const int g = (i >= bound0) + (i >= bound1);
    base = g == 0 ? 0 : (g == 1 ? bound0 : bound1);   // no indexing by g: kernel parameters are not addressable
    return g;
}

// Cluster split: member `krank` of the cluster keeps only its own range of the contraction.
__device__ __forceinline__ void narrow_to_krank(const GemmParams& p, int krank, WorkItem& w) {
    if (p.ksplit > 1) {
        const int per = (p.kb_total + p.ksplit - 1) / p.ksplit;
        w.kb0 = krank * per;
        w.kb1 = min(w.kb0 + per, p.kb_total);
    }
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
    unsigned long long sk_written;     // the 4 epilogue warps have stored their part of a partial tile
    unsigned long long sk_decided;     // "am I the last arriver" has been published in sk_last
    unsigned long long sk_read;        // peer split: the 8 epilogue warps have read the other members' partials
    unsigned long long old_bar[8];     // beta = 1: epilogue warp w's copy of the old output block has landed
    unsigned long long ml_done;        // cluster split: the other members have finished their main loops
    unsigned long long cs_recv;        // cluster split: the other members' slices of my columns have landed
    uint32_t tmem_base;
    int abort_flag;
    int sk_last;
};

// Float offset of (epilogue warp q, 32-column group c32, float4 index j4, lane) inside one
// CTA's partial tile.  Chosen so that every warp-wide float4 access is one contiguous 512 bytes.
template <int BN>
__device__ __forceinline__ int partial_offset(int q, int c32, int j4, int lane) {
    return (((q * (BN / 32) + c32) * 8 + j4) * 32 + lane) * 4;
}

// Store this warp's share of the accumulator as an fp32 partial tile.  Epilogue warp (q, hsel)
// owns TMEM lanes 32q..32q+31 and every second 32-column group, starting with group hsel.
template <int BN>
__device__ __forceinline__ void epilogue_store_partial(float* block, uint32_t taddr, int q, int hsel, int lane) {
#pragma unroll 1
    for (int c = hsel; c < BN / 32; c += 2) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(block + partial_offset<BN>(q, c, j, lane)) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    }
}

// acc[0..31] += the 32 values of (q, c32, lane) in one partial tile.
template <int BN>
__device__ __forceinline__ void load_partial32(float4 (&v)[8], const float* blk, int q, int c32, int lane) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
        v[j] = __ldcg(reinterpret_cast<const float4*>(blk + partial_offset<BN>(q, c32, j, lane)));
}
__device__ __forceinline__ void add_partial32(uint32_t* acc, const float4 (&v)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        acc[4 * j + 0] = __float_as_uint(__uint_as_float(acc[4 * j + 0]) + v[j].x);
        acc[4 * j + 1] = __float_as_uint(__uint_as_float(acc[4 * j + 1]) + v[j].y);
        acc[4 * j + 2] = __float_as_uint(__uint_as_float(acc[4 * j + 2]) + v[j].z);
        acc[4 * j + 3] = __float_as_uint(__uint_as_float(acc[4 * j + 3]) + v[j].w);
    }
}

// Write this warp's share of the output tile as bf16.  Epilogue warp (q, hsel) owns rows
// row0..row0+31 and every second 64-column chunk, starting with chunk hsel: chunk ->
// (beta=1: add the old values) -> bf16 -> the warp's 128B-swizzled staging buffer -> one TMA
// store of a 32 x 64 box (TMA clips rows/columns beyond the matrix, so tails need no predicates).
// The fp32 values come from TMEM (FROM_WS = false) or from the sum of `nsplits` partial tiles
// in the workspace, added in the order 0..nsplits-1 (FROM_WS = true).
// beta = 1: the old 32 x 64 block is fetched by TMA into the same staging buffer and updated in
// place (each thread reads and rewrites only its own row), so global memory sees whole lines only.
template <int BN, bool BETA1, bool FROM_WS, int NBUF>
__device__ __forceinline__ bool epilogue_store_bf16(const GemmParams& p, const CUtensorMap* tmD, uint8_t* bufs,
                                                    uint32_t taddr, const float* partials, size_t partial_stride,
                                                    int nsplits, int q, int hsel, int row0, int lane, int n0,
                                                    uint32_t old_bar, uint32_t& old_phase, volatile int* abort_flag) {
    // With two buffers the chunks alternate between them and a chunk only waits for the store before the
    // previous one; whatever this warp stored earlier (any path) has finished reading before the first chunk.
    if constexpr (NBUF == 2) {
        if (elect_one()) tma_store_wait_read<0>();
        __syncwarp();
    }
    int sel = 0;
#pragma unroll 1
    for (int c = hsel; c < BN / 64; c += 2) {
        const int col0 = n0 + c * 64;
        if (col0 >= p.No) break;  // whole chunk beyond the matrix (warp-uniform)
        uint8_t* buf = bufs + sel * EPI_BUF_BYTES;
        sel ^= NBUF - 1;
        uint32_t r[64];
        if constexpr (!FROM_WS) {
            tmem_ld_32x32(taddr + c * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
            tmem_ld_32x32(taddr + c * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        }
        if constexpr (BETA1) {
            // the warp's previous store must have finished reading the staging buffer
            if (elect_one()) {
                tma_store_wait_read<NBUF - 1>();
                mbar_arrive_expect_tx(old_bar, EPI_BUF_BYTES);
                tma_load_2d(smem_u32(buf), tmD, old_bar, col0, row0);  // rows/cols beyond the matrix read as 0
            }
        }
        if constexpr (FROM_WS) {
#pragma unroll
            for (int e = 0; e < 64; ++e) r[e] = 0u;  // +0.0f
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int c32 = 2 * c + half;
                int sp = 0;
                for (; sp + 1 < nsplits; sp += 2) {  // two partial tiles in flight, added in order
                    float4 va[8], vb[8];
                    load_partial32<BN>(va, partials + sp * partial_stride, q, c32, lane);
                    load_partial32<BN>(vb, partials + (sp + 1) * partial_stride, q, c32, lane);
                    add_partial32(&r[32 * half], va);
                    add_partial32(&r[32 * half], vb);
                }
                if (sp < nsplits) {
                    float4 va[8];
                    load_partial32<BN>(va, partials + sp * partial_stride, q, c32, lane);
                    add_partial32(&r[32 * half], va);
                }
            }
        } else {
            tmem_ld_wait();
        }
        if constexpr (BETA1) {
            bool ok = mbar_wait(old_bar, old_phase, abort_flag, p.status, DEV_TIMEOUT_DRAIN);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return false;
            old_phase ^= 1;
        } else {
            // the warp's last store from this buffer must have finished reading it
            if (elect_one()) tma_store_wait_read<NBUF - 1>();
            __syncwarp();
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[8 * j + e]);
            // 128-byte swizzle: 16-byte chunk j of row `lane` lives at chunk (j ^ (lane & 7))
            uint4* slot = reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4));
            if constexpr (BETA1) {
                // Same two roundings as the reference's cuBLAS path: bf16_rn(bf16_rn(acc) + old).
                const uint4 o = *slot;
                const uint32_t a0 = pack_bf16x2(v[0], v[1]), a1 = pack_bf16x2(v[2], v[3]);
                const uint32_t a2 = pack_bf16x2(v[4], v[5]), a3 = pack_bf16x2(v[6], v[7]);
                v[0] = bf16_lo(a0) + bf16_lo(o.x); v[1] = bf16_hi(a0) + bf16_hi(o.x);
                v[2] = bf16_lo(a1) + bf16_lo(o.y); v[3] = bf16_hi(a1) + bf16_hi(o.y);
                v[4] = bf16_lo(a2) + bf16_lo(o.z); v[5] = bf16_hi(a2) + bf16_hi(o.z);
                v[6] = bf16_lo(a3) + bf16_lo(o.w); v[7] = bf16_hi(a3) + bf16_hi(o.w);
            }
            *slot =
                make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                           pack_bf16x2(v[6], v[7]));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (row0 < p.Mo && elect_one()) {
            tma_store_2d(tmD, smem_u32(buf), col0, row0);
            tma_store_commit();
        }
    }
    return true;
}

// LM-head forward with the cross-entropy statistics in the epilogue (EPI = 2; 256-wide tiles, whole tiles only): the
// tile is stored as bf16 like any other, and while its rows are in registers each epilogue warp also forms, over the
// columns it owns of the tile (chunks hsel and hsel + 2: 128 of the 256) and from the bf16-rounded values (what a
// separate pass over the stored logits would read), the row maximum m and s = sum exp(l - m).  One (m, s) pair per
// row, tile and hsel goes to stats[row][2 * n_blk + hsel]; a small kernel merges a row's pairs (ce_merge_partials).
// Columns at or beyond p.No count as -inf.
template <int NBUF>
__device__ __forceinline__ void epilogue_store_stats(const GemmParams& p, const CUtensorMap* tmD, uint8_t* bufs, uint32_t taddr,
                                                     int hsel, int row0, int lane, int n0, int n_blk) {
    constexpr float L2E = 1.4426950408889634f;
    if constexpr (NBUF == 2) {
        if (elect_one()) tma_store_wait_read<0>();
        __syncwarp();
    }
    float m = -INFINITY, ssum = 0.f;
    int sel = 0;
#pragma unroll 1
    for (int c = hsel; c < 4; c += 2) {
        const int col0 = n0 + c * 64;
        if (col0 >= p.No) break;  // whole chunk beyond the matrix (warp-uniform)
        uint8_t* buf = bufs + sel * EPI_BUF_BYTES;
        sel ^= NBUF - 1;
        uint32_t r[64];
        tmem_ld_32x32(taddr + c * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld_32x32(taddr + c * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld_wait();
        if (elect_one()) tma_store_wait_read<NBUF - 1>();   // the warp's last store from this buffer has been read out
        __syncwarp();
        uint32_t pk[32];
        float cm = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            pk[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            const float lo = (col0 + 2 * j < p.No) ? bf16_lo(pk[j]) : -INFINITY;
            const float hi = (col0 + 2 * j + 1 < p.No) ? bf16_hi(pk[j]) : -INFINITY;
            cm = fmaxf(cm, fmaxf(lo, hi));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (row0 < p.Mo && elect_one()) {
            tma_store_2d(tmD, smem_u32(buf), col0, row0);
            tma_store_commit();
        }
        const float mn = fmaxf(m, cm);
        if (mn != -INFINITY) {   // a row with nothing finite so far keeps (m, s) = (-inf, 0)
            const float base = mn * L2E;
            float acc4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float lo = (col0 + 2 * j < p.No) ? bf16_lo(pk[j]) : -INFINITY;
                const float hi = (col0 + 2 * j + 1 < p.No) ? bf16_hi(pk[j]) : -INFINITY;
                acc4[j & 3] += exp2f(fmaf(lo, L2E, -base)) + exp2f(fmaf(hi, L2E, -base));
            }
            ssum = ssum * exp2f(fmaf(m, L2E, -base)) + (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);   // m = -inf: ssum * 0
            m = mn;
        }
    }
    const int row = row0 + lane;
    if (row < p.Mo)
        reinterpret_cast<float2*>(p.ws)[static_cast<size_t>(row) * (2 * p.n_tiles) + 2 * n_blk + hsel] = make_float2(m, ssum);
}

// SwiGLU forward in the epilogue (EPI = 1; 256-wide pair tiles): accumulator columns 0..127 are 128 columns of
// gate = X W_gate, columns 128..255 the same 128 columns of up = X W_up.  Epilogue warp (q, hsel) owns rows
// row0..row0+31 and 64-column chunk hsel of both: it rounds gate and up to bf16 (what the reference's two GEMMs
// store), forms hidden = SiLU(gate) * up from the rounded values (cuda/swiglu.cu:132-140) and stores the three
// 32 x 64 blocks through its two staging buffers (gate -> buffer 0, up -> buffer 1, hidden -> buffer 0 again).
__device__ __forceinline__ float epi_sigmoid(float g) { return 1.0f / (1.0f + __expf(-g)); }
__device__ __forceinline__ void epilogue_swiglu(const GemmParams& p, const CUtensorMap* tmGate, const CUtensorMap* tmUp,
                                                const CUtensorMap* tmHidden, uint8_t* bufs, uint32_t taddr, int hsel,
                                                int row0, int lane, int n0) {
    if (elect_one()) tma_store_wait_read<0>();   // whatever this warp stored earlier has been read out of both buffers
    __syncwarp();
    const int col0 = n0 + hsel * 64;
    uint8_t* buf_g = bufs;
    uint8_t* buf_u = bufs + EPI_BUF_BYTES;
    uint32_t hid[32];   // the 64 hidden values of this thread's row, packed
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t g[32], u[32];
        tmem_ld_32x32(taddr + hsel * 64 + half * 32, g);
        tmem_ld_32x32(taddr + 128 + hsel * 64 + half * 32, u);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) {   // 16-byte chunk 4 * half + j of the 128-byte row
            uint32_t pg[4], pu[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                pg[e] = pack_bf16x2(__uint_as_float(g[8 * j + 2 * e]), __uint_as_float(g[8 * j + 2 * e + 1]));
                pu[e] = pack_bf16x2(__uint_as_float(u[8 * j + 2 * e]), __uint_as_float(u[8 * j + 2 * e + 1]));
                const float g0 = bf16_lo(pg[e]), g1 = bf16_hi(pg[e]);
                hid[half * 16 + 4 * j + e] = pack_bf16x2(g0 * epi_sigmoid(g0) * bf16_lo(pu[e]), g1 * epi_sigmoid(g1) * bf16_hi(pu[e]));
            }
            const int off = lane * 128 + (((4 * half + j) ^ (lane & 7)) << 4);   // 128-byte swizzle
            *reinterpret_cast<uint4*>(buf_g + off) = make_uint4(pg[0], pg[1], pg[2], pg[3]);
            *reinterpret_cast<uint4*>(buf_u + off) = make_uint4(pu[0], pu[1], pu[2], pu[3]);
        }
    }
    fence_proxy_async_smem();
    __syncwarp();
    const bool store = row0 < p.Mo;
    if (store && elect_one()) {
        tma_store_2d(tmGate, smem_u32(buf_g), col0, row0);
        tma_store_commit();
        tma_store_2d(tmUp, smem_u32(buf_u), col0, row0);
        tma_store_commit();
        tma_store_wait_read<1>();   // the gate block has left buffer 0
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(buf_g + lane * 128 + ((j ^ (lane & 7)) << 4)) =
            make_uint4(hid[4 * j], hid[4 * j + 1], hid[4 * j + 2], hid[4 * j + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (store && elect_one()) {
        tma_store_2d(tmHidden, smem_u32(buf_g), col0, row0);
        tma_store_commit();
    }
}

// Write one 32 x 32 block (this warp's rows, one 32-column group) of fp32 sums as bf16 through the
// warp's staging buffer (64-byte swizzle) and a TMA store.  beta = 1: `begin` (called before the
// sums are formed) starts a TMA load of the old block into the same buffer, `finish` updates it in place.
template <bool BETA1>
__device__ __forceinline__ void block32_begin(const CUtensorMap* tmD32, uint8_t* buf, uint32_t old_bar, int col0,
                                              int row0, int lane) {
    if (elect_one()) {
        tma_store_wait_read<0>();  // the previous store of this warp has finished reading the buffer
        if constexpr (BETA1) {
            mbar_arrive_expect_tx(old_bar, 32 * 64);
            tma_load_2d(smem_u32(buf), tmD32, old_bar, col0, row0);  // beyond the matrix reads as 0
        }
    }
}
template <bool BETA1>
__device__ __forceinline__ bool block32_finish(const GemmParams& p, const CUtensorMap* tmD32, uint8_t* buf,
                                               const float (&acc)[32], uint32_t old_bar, uint32_t& old_phase,
                                               int col0, int row0, int lane, volatile int* abort_flag) {
    if constexpr (BETA1) {
        bool ok = mbar_wait(old_bar, old_phase, abort_flag, p.status, DEV_TIMEOUT_DRAIN);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return false;
        old_phase ^= 1;
    } else {
        __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = acc[8 * j + e];
        // 64-byte swizzle: 16-byte chunk j of row `lane` lives at chunk (j ^ ((lane >> 1) & 3))
        uint4* slot16 = reinterpret_cast<uint4*>(buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4));
        if constexpr (BETA1) {
            // Same two roundings as the reference's cuBLAS path: bf16_rn(bf16_rn(acc) + old).
            const uint4 o = *slot16;
            const uint32_t a0 = pack_bf16x2(v[0], v[1]), a1 = pack_bf16x2(v[2], v[3]);
            const uint32_t a2 = pack_bf16x2(v[4], v[5]), a3 = pack_bf16x2(v[6], v[7]);
            v[0] = bf16_lo(a0) + bf16_lo(o.x); v[1] = bf16_hi(a0) + bf16_hi(o.x);
            v[2] = bf16_lo(a1) + bf16_lo(o.y); v[3] = bf16_hi(a1) + bf16_hi(o.y);
            v[4] = bf16_lo(a2) + bf16_lo(o.z); v[5] = bf16_hi(a2) + bf16_hi(o.z);
            v[6] = bf16_lo(a3) + bf16_lo(o.w); v[7] = bf16_hi(a3) + bf16_hi(o.w);
        }
        *slot16 = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                             pack_bf16x2(v[6], v[7]));
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (row0 < p.Mo && elect_one()) {
        tma_store_2d(tmD32, smem_u32(buf), col0, row0);
        tma_store_commit();
    }
    return true;
}

// Cluster split: the ksplit members of a cluster hold partial sums of the SAME output tile (one
// range of the contraction each) in their TMEM.  The tile's 32-column groups are dealt out to the
// members; every member sends each other member that member's groups of its own partial sum
// (st.async into the receiver's shared memory, counted on the receiver's barrier), then adds up
// what it received for its own groups -- in member order 0..ksplit-1, whatever the arrival order --
// applies beta and writes those columns.  Nothing goes through global memory.
// The pipeline stages double as receive space: by then this CTA's main loop has finished, and a
// member only starts sending after every member has said so (ml_done).
// Returns false if a bounded wait ran out.
template <int BN, bool BETA1, int CTAS>
__device__ __forceinline__ bool epilogue_cluster_split(const GemmParams& p, GemmCtrl* ctrl, uint8_t* recv,
                                                       const CUtensorMap* tmD32, uint8_t* buf, uint32_t taddr, int q,
                                                       int hsel, int lane, int warp, int row0, int n0, int krank,
                                                       int rank, uint32_t old_bar, uint32_t& old_phase,
                                                       volatile int* abort_flag) {
    constexpr int G = BN / 32;                    // 32-column groups of the tile
    const int S = p.ksplit;
    const int maxg = (G + S - 1) / S;             // groups per member, upper bound
    const int my_g0 = krank * G / S, my_g1 = (krank + 1) * G / S;
    const uint32_t recv_bar = smem_u32(&ctrl->cs_recv);
    const uint32_t recv_base = smem_u32(recv);
    const int trow = q * 32 + lane;               // row of the tile this thread owns

    if (warp == 4 && lane == 0) {
        mbar_arrive_expect_tx(recv_bar, static_cast<uint32_t>((S - 1) * (my_g1 - my_g0)) * 32u * BM * 4u);
        for (int d = 0; d < S; ++d)
            if (d != krank) mbar_arrive_cluster(smem_u32(&ctrl->ml_done), static_cast<uint32_t>(d * CTAS + rank));
    }
    bool ok = mbar_wait<true>(smem_u32(&ctrl->ml_done), 0, abort_flag, p.status, DEV_TIMEOUT_PEER);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return false;

    // send: my partial sums of every other member's column groups
    for (int dd = 1; dd < S; ++dd) {
        const int d = (krank + dd) % S;           // start with the next member: spreads the traffic
        const int slot = krank < d ? krank : krank - 1;
        const uint32_t target = static_cast<uint32_t>(d * CTAS + rank);
        const uint32_t r_base = map_to_cta(recv_base, target);
        const uint32_t r_bar = map_to_cta(recv_bar, target);
        const int g0 = d * G / S, g1 = (d + 1) * G / S;
#pragma unroll 1
        for (int g = g0 + hsel; g < g1; g += 2) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + g * 32, r);
            tmem_ld_wait();
            const uint32_t dst = r_base + static_cast<uint32_t>(((slot * maxg + (g - g0)) * 8) * BM + trow) * 16u;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                st_async_v4(dst + static_cast<uint32_t>(j * BM) * 16u, r[4 * j], r[4 * j + 1], r[4 * j + 2],
                            r[4 * j + 3], r_bar);
        }
    }

    // receive, then sum my own column groups in member order
    ok = mbar_wait<true>(recv_bar, 0, abort_flag, p.status, DEV_TIMEOUT_PEER);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return false;
    // The output goes out in 32 x 32 blocks through the warp's staging buffer (64-byte swizzle) and
    // a TMA store; with beta = 1 the old block comes in by TMA first and is updated in place.
#pragma unroll 1
    for (int g = my_g0 + hsel; g < my_g1; g += 2) {
        const int col0 = n0 + g * 32;
        if (col0 >= p.No) break;  // whole group beyond the matrix (warp-uniform)
        block32_begin<BETA1>(tmD32, buf, old_bar, col0, row0, lane);
        uint32_t own[32];
        tmem_ld_32x32(taddr + g * 32, own);
        tmem_ld_wait();
        float acc[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[e] = 0.f;
        for (int k = 0; k < S; ++k) {
            if (k == krank) {
#pragma unroll
                for (int e = 0; e < 32; ++e) acc[e] += __uint_as_float(own[e]);
            } else {
                const int slot = k < krank ? k : k - 1;
                const uint8_t* src = recv + static_cast<size_t>(((slot * maxg + (g - my_g0)) * 8) * BM + trow) * 16;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 v = *reinterpret_cast<const float4*>(src + static_cast<size_t>(j * BM) * 16);
                    acc[4 * j] += v.x; acc[4 * j + 1] += v.y; acc[4 * j + 2] += v.z; acc[4 * j + 3] += v.w;
                }
            }
        }
        if (!block32_finish<BETA1>(p, tmD32, buf, acc, old_bar, old_phase, col0, row0, lane, abort_flag)) return false;
    }
    return true;
}

// Peer split: the same exchange as the cluster split, for the ranges of a split tile that run on
// CTAs anywhere on the GPU: partial sums travel through the workspace (L2) instead of distributed
// shared memory.  Member `me` of the tile's `S` ranges stores, for every other member, its partial
// sums of that member's column groups; publishes them with one counter increment; waits (bounded)
// until all S members have published; then sums its own groups (own part from TMEM, the others'
// from the workspace, in member order) and writes them.  Each member reads and writes (S-1)/S of a
// tile instead of one member reading S whole tiles.
// Requires all members of a tile to be resident at once: the host only selects this mode when the
// split work items are the first item of distinct CTAs of a grid that fits the GPU.
// `region` = this tile's exchange space for this CTA rank: S * (S-1) * maxg blocks of BM x 32 fp32.
template <int BN, bool BETA1>
__device__ __forceinline__ bool epilogue_peer_split(const GemmParams& p, GemmCtrl* ctrl, float* region, int* counter,
                                                    const CUtensorMap* tmD32, uint8_t* buf, uint32_t taddr, int q,
                                                    int hsel, int lane, int warp, int row0, int n0, int me,
                                                    uint32_t old_bar, uint32_t& old_phase, uint32_t sk_phase,
                                                    volatile int* abort_flag) {
    constexpr int G = BN / 32;
    constexpr int BLOCK_FLOATS = 8 * BM * 4;      // one 32-column group of a tile: 8 float4 x 128 rows
    const int S = p.sk_splits;
    const int maxg = (G + S - 1) / S;
    const int my_g0 = me * G / S, my_g1 = (me + 1) * G / S;
    const int trow = q * 32 + lane;
    auto block_of = [&](int dest, int slot, int gi) {
        return region + static_cast<size_t>((dest * (S - 1) + slot) * maxg + gi) * BLOCK_FLOATS;
    };
    for (int dd = 1; dd < S; ++dd) {
        const int d = (me + dd) % S;
        const int slot = me < d ? me : me - 1;
        const int g0 = d * G / S, g1 = (d + 1) * G / S;
#pragma unroll 1
        for (int g = g0 + hsel; g < g1; g += 2) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + g * 32, r);
            tmem_ld_wait();
            float* dst = block_of(d, slot, g - g0) + trow * 4;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(dst + j * BM * 4) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
    }
    // publish, then wait for the other members
    __threadfence();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctrl->sk_written));
    if (warp == 4 && lane == 0) {
        int seen = 0;
        if (mbar_wait(smem_u32(&ctrl->sk_written), sk_phase, abort_flag, p.status, DEV_TIMEOUT_PEER)) {
            __threadfence();
            atomicAdd(counter, 1);
            const long long t0 = clock64();
            while (true) {
                seen = *reinterpret_cast<volatile int*>(counter);
                if (seen >= S) break;
                if (*abort_flag) break;
                if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                    *abort_flag = 1;
                    atomicCAS(p.status, 0, DEV_TIMEOUT_PEER);
                    break;
                }
            }
            __threadfence();
        }
        ctrl->sk_last = seen >= S;
        mbar_arrive(smem_u32(&ctrl->sk_decided));
    }
    bool ok = mbar_wait(smem_u32(&ctrl->sk_decided), sk_phase, abort_flag, p.status, DEV_TIMEOUT_PEER);
    ok = __all_sync(0xffffffffu, ok) && ctrl->sk_last;
    if (!ok) return false;
    __threadfence();
#pragma unroll 1
    for (int g = my_g0 + hsel; g < my_g1; g += 2) {
        const int col0 = n0 + g * 32;
        if (col0 >= p.No) break;  // whole group beyond the matrix (warp-uniform)
        block32_begin<BETA1>(tmD32, buf, old_bar, col0, row0, lane);
        uint32_t own[32];
        tmem_ld_32x32(taddr + g * 32, own);
        float acc[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[e] = 0.f;
        tmem_ld_wait();
        // members in order; the two next partial blocks are in flight while one is added
        int k = 0;
        while (k < S) {
            if (k == me) {
#pragma unroll
                for (int e = 0; e < 32; ++e) acc[e] += __uint_as_float(own[e]);
                ++k;
                continue;
            }
            const int k2 = (k + 1 == me) ? k + 2 : k + 1;  // the next member that is not me
            const bool two = k2 < S && k + 1 != me;         // k and k+1 are both others: load both
            float4 va[8], vb[8];
            const float* sa = block_of(me, k < me ? k : k - 1, g - my_g0) + trow * 4;
#pragma unroll
            for (int j = 0; j < 8; ++j) va[j] = __ldcg(reinterpret_cast<const float4*>(sa + j * BM * 4));
            if (two) {
                const float* sb = block_of(me, (k + 1) < me ? k + 1 : k, g - my_g0) + trow * 4;
#pragma unroll
                for (int j = 0; j < 8; ++j) vb[j] = __ldcg(reinterpret_cast<const float4*>(sb + j * BM * 4));
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc[4 * j] += va[j].x; acc[4 * j + 1] += va[j].y; acc[4 * j + 2] += va[j].z; acc[4 * j + 3] += va[j].w;
            }
            if (two) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[4 * j] += vb[j].x; acc[4 * j + 1] += vb[j].y; acc[4 * j + 2] += vb[j].z; acc[4 * j + 3] += vb[j].w;
                }
                k += 2;
            } else {
                k += 1;
            }
            (void)k2;
        }
        if (!block32_finish<BETA1>(p, tmD32, buf, acc, old_bar, old_phase, col0, row0, lane, abort_flag)) return false;
    }
    // everybody has read: the member that counts last puts the counter back to zero
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctrl->sk_read));
    if (warp == 4 && lane == 0) {
        if (mbar_wait(smem_u32(&ctrl->sk_read), sk_phase, abort_flag, p.status, DEV_TIMEOUT_PEER)) {
            const int prev = atomicAdd(counter, 1);
            if (prev == 2 * S - 1) atomicExch(counter, 0);
        }
    }
    return true;
}

// Warp roles: 0 = TMA producer for P, 3 = TMA producer for Q, 1 = MMA issuer (even CTA only in a
// pair), 2 = TMEM allocator, 4..11 = epilogue: warp w may touch TMEM lanes 32*(w%4) .. +31 only, so warps w and
// w+4 share a lane quarter and split its columns between them.
// EPI = 1: the SwiGLU forward pair (see epilogue_swiglu): BN = 256, CTAS = 2, forward layout, whole tiles only.  The even
// CTA of a pair feeds W_gate's columns (tmQ), the odd one the same columns of W_up (gx.q[0]); outputs: gate (tmD), up
// (gx.d[0]), hidden (gx.d[1]); a tile index counts 128-column blocks of those three matrices.
// EPI = 2: the LM-head forward that also leaves per-tile cross-entropy statistics in p.ws (see epilogue_store_stats).
template <int BN, bool P_MN, bool Q_MN, bool BETA1, int CTAS, int EPI = 0>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_sm100(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmD32,
                const __grid_constant__ typename GemmExtraMaps<EPI>::type gx, const GemmParams p) {
    using Cfg = TileCfg<BN, CTAS>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr bool PAIR = CTAS == 2;
    static_assert(EPI != 1 || (BN == 256 && CTAS == 2 && !P_MN && Q_MN && !BETA1), "SwiGLU epilogue: 256-wide pair tiles, forward");
    static_assert(EPI != 2 || (BN == 256 && !P_MN && Q_MN && !BETA1), "cross-entropy statistics: 256-wide tiles, forward");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    GemmCtrl* ctrl = reinterpret_cast<GemmCtrl*>(smem);
    uint8_t* tiles = smem + Cfg::CTRL_BYTES;  // stage s: [P tile | Q tile]
    uint8_t* epi_bufs = tiles + STAGES * Cfg::STAGE_BYTES;  // per epilogue warp: 2 staging buffers
    volatile int* abort_flag = &ctrl->abort_flag;

    // read through a shuffle so that the compiler treats the warp index (and everything derived from
    // it: the role, the TMEM lane quarter, the staging buffer) as uniform across the warp
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const uint32_t ctarank = cluster_ctarank();          // 0 when launched without a cluster
    const uint32_t rank = ctarank % CTAS;                // position in the CTA pair
    const uint32_t leader = ctarank - rank;              // cluster rank of the pair's MMA-issuing CTA
    const int krank = static_cast<int>(ctarank / CTAS);  // which range of the contraction (cluster split)
    const int cluster_ctas = CTAS * p.ksplit;
    const int slot = blockIdx.x / cluster_ctas, nslots = gridDim.x / cluster_ctas;
    const bool clustered = PAIR || p.ksplit > 1;

    if (warp == 1) {
        // the barriers are consecutive 8-byte words at the start of the control block: one lane each
        constexpr int N_BARS = 16 + 4 + 3 + EPI_WARPS + 2;
        static_assert(offsetof(GemmCtrl, cs_recv) == (N_BARS - 1) * 8, "barrier list and control block disagree");
        for (int b = lane; b < N_BARS; b += 32) {
            uint32_t count = 1;  // empty[], tmem_full[], sk_decided, old_bar[], cs_recv
            if (b < 8) count = 2;  // full[]: one arrival (+ byte count) per producer warp
            else if (b >= 16 && b < 18) count = 1;
            else if (b >= 18 && b < 20) count = EPI_WARPS * CTAS;         // tmem_empty[]
            else if (b == 20 || b == 22) count = EPI_WARPS;                // sk_written, sk_read
            else if (b == N_BARS - 2) count = p.ksplit > 1 ? p.ksplit - 1 : 1;  // ml_done
            mbar_init(smem_u32(&ctrl->full[0]) + 8u * b, count);
        }
        if (lane == 0) {
            ctrl->abort_flag = 0;
            ctrl->sk_last = 0;
        }
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmP);
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmD);
        if (p.ksplit > 1 || p.sk_peer) tma_prefetch_desc(&tmD32);
    }
    if (warp == 2) {
        tmem_alloc<CTAS>(smem_u32(&ctrl->tmem_base), Cfg::TMEM_COLS);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before();
    // The other CTAs' barriers must exist before anything signals them.  Every thread arrives at the cluster
    // barrier as soon as its own part of the set-up is done (release), so the barrier's latency overlaps the
    // slowest part (the TMEM allocation) instead of following it.
    if (clustered) cluster_arrive_release();
    __syncthreads();
    if (clustered) cluster_wait_acquire();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;
    // grouped launch: the maps of product g (g = 0: the kernel's own)
    constexpr bool HAS_MAPS = EPI == 1 || EPI == 3, GROUPED = EPI == 3;
    auto map_p = [&](int g) -> const CUtensorMap* {
        if constexpr (HAS_MAPS) return g == 0 ? &tmP : (g == 1 ? &gx.p[0] : &gx.p[1]);
        else return &tmP;
    };
    auto map_q = [&](int g) -> const CUtensorMap* {
        if constexpr (HAS_MAPS) return g == 0 ? &tmQ : (g == 1 ? &gx.q[0] : &gx.q[1]);
        else return &tmQ;
    };
    auto map_d = [&](int g) -> const CUtensorMap* {
        if constexpr (HAS_MAPS) return g == 0 ? &tmD : (g == 1 ? &gx.d[0] : &gx.d[1]);
        else return &tmD;
    };
    auto map_d32 = [&](int g) -> const CUtensorMap* {
        if constexpr (HAS_MAPS) return g == 0 ? &tmD32 : (g == 1 ? &gx.d32[0] : &gx.d32[1]);
        else return &tmD32;
    };
    // which product a column tile / contraction block belongs to: 0 and origin 0 unless this is a grouped launch
    auto grp_n = [&](int n_blk, int& base) {
        if constexpr (GROUPED) return group_of(p.grp_n[0], p.grp_n[1], n_blk, base);
        base = 0;
        return 0;
    };
    auto grp_k = [&](int kb, int& base) {
        if constexpr (GROUPED) return group_of(p.grp_k[0], p.grp_k[1], kb, base);
        base = 0;
        return 0;
    };
    // the first work item does not depend on memory: know it before the dependency wait
    WorkItem w_first;
    const bool have_first = get_work(p, slot, nslots, 0, w_first);
    auto next_work = [&](int i, WorkItem& w) {
        if (i == 0) {
            w = w_first;
            return have_first;
        }
        return get_work(p, slot, nslots, i, w);
    };
    // Programmatic dependent launch: everything above overlapped the tail of the previous kernel
    // in the stream; its results (and its reads of our output buffers) are complete only after
    // this wait.  The next kernel may start its own set-up as soon as our CTAs make room.
    // Programmatic dependent launch: everything above overlapped the tail of the previous kernel in the
    // stream; its results (and its reads of our output buffers) are complete only after this wait.
    // The next kernel is released only after the wait: if that kernel is one that runs beside this one
    // (late_wait), it starts reading at once and relies on everything older than this kernel being
    // complete and visible.
    // While the previous kernel in the stream finishes: ask L2 for the first stages of the first work item.
    // L2 is the point of coherence for device memory, so a line fetched early is still current when the
    // copies into shared memory read it after the wait; inside the step the operands come from HBM (the
    // working set is far larger than L2) and this takes their first-touch latency off the critical path.
    if (EPI != 1 && (warp == 0 || warp == 3) && have_first && !p.late_wait) {
        if (elect_one()) {
            WorkItem w = w_first;
            narrow_to_krank(p, krank, w);
            int n_base;
            const int gn = grp_n(w.n_blk, n_base);
            const int m0 = (w.m_blk * CTAS + static_cast<int>(rank)) * BM;
            const int n0 = (w.n_blk - n_base) * BN + static_cast<int>(rank) * Cfg::B_ROWS;
            const int kb_end = min(w.kb1, w.kb0 + STAGES);
            {
                const bool is_q = warp == 3;
                const bool mn = is_q ? Q_MN : P_MN;
                const bool as3d = is_q ? (p.q_3d != 0) : (p.p_3d != 0);
                const int panels = is_q ? Cfg::B_ROWS / 64 : BM / 64;
                const int r0 = is_q ? n0 : m0;
                for (int kb = w.kb0; kb < kb_end; ++kb) {
                    int k_base;
                    const int gk = grp_k(kb, k_base);
                    const CUtensorMap* tm = is_q ? map_q(gn + gk) : map_p(gk);
                    const int c0 = (kb - k_base) * BK;
                    if (!mn) tma_prefetch_l2_2d(tm, c0, r0);
                    else if (as3d) tma_prefetch_l2_3d(tm, 0, c0, r0 >> 6);
                    else
                        for (int j = 0; j < panels; ++j) tma_prefetch_l2_2d(tm, r0 + 64 * j, c0);
                }
            }
        }
        __syncwarp();
    }
    if (!p.late_wait) griddep_wait();
    griddep_launch_dependents();

    // The three issuing roles below run with all 32 lanes of their warp converged: every lane waits on the
    // barriers and does the (warp-uniform) address arithmetic, and one elected lane issues the copies, the
    // MMAs and the commits.  Their operands then sit in uniform registers; the same loops run by a single
    // lane inside a divergent branch cost several hundred cycles per 64-deep block just to issue.
    if (warp == 0 || warp == 3) {
        // ---------------------------------------------- TMA producers: warp 0 feeds P, warp 3 feeds Q
        {
            const bool do_p = warp == 0, do_q = warp == 3;
            uint32_t stage = 0, phase = 0;
            uint32_t issued = 0;  // number of stage fills issued so far
            bool ok = true;
            WorkItem w;
            auto issue = [&](bool is_q, const CUtensorMap* tm, uint32_t dst, uint32_t bar, int r0, int c0) {
                const bool mn = is_q ? Q_MN : P_MN;
                const bool as3d = is_q ? (p.q_3d != 0) : (p.p_3d != 0);
                const int panels = is_q ? Cfg::B_ROWS / 64 : BM / 64;
                if (!mn) {            // global [rows][Kc]: box = BK contraction x rows
                    if constexpr (PAIR) tma_load_2d_pair(dst, tm, bar, c0, r0);
                    else tma_load_2d(dst, tm, bar, c0, r0);
                } else if (as3d) {    // global [Kc][rows]: all 64-wide column panels in one copy
                    if constexpr (PAIR) tma_load_3d_pair(dst, tm, bar, 0, c0, r0 >> 6);
                    else tma_load_3d(dst, tm, bar, 0, c0, r0 >> 6);
                } else {              // one copy per 64-wide column panel
                    for (int j = 0; j < panels; ++j) {
                        if constexpr (PAIR) tma_load_2d_pair(dst + j * (64 * BK * 2), tm, bar, r0 + 64 * j, c0);
                        else tma_load_2d(dst + j * (64 * BK * 2), tm, bar, r0 + 64 * j, c0);
                    }
                }
            };
            // The state of the next stage's barrier is probed one iteration ahead, so that the probe's
            // latency overlaps the issue of the current stage's copies.
            bool ready = mbar_test_wait(smem_u32(&ctrl->empty[0]), 1);
            const bool issuer = elect_one();  // one lane, the same for the whole loop
            for (int i = 0; ok && next_work(i, w); ++i) {
                narrow_to_krank(p, krank, w);
                int n_base;
                const int gn = EPI == 1 ? (n_base = 0, static_cast<int>(rank)) : grp_n(w.n_blk, n_base);
                const int m0 = (w.m_blk * CTAS + static_cast<int>(rank)) * BM;
                const int n0 = EPI == 1 ? w.n_blk * Cfg::B_ROWS : (w.n_blk - n_base) * BN + static_cast<int>(rank) * Cfg::B_ROWS;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    if (!__all_sync(0xffffffffu, ready)) {
                        ok = mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_flag, p.status,
                                       DEV_TIMEOUT_EMPTY);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                    }
                    const uint32_t next_stage = stage + 1 == STAGES ? 0 : stage + 1;
                    const uint32_t next_phase = next_stage == 0 ? phase ^ 1 : phase;
                    ready = mbar_test_wait(smem_u32(&ctrl->empty[next_stage]), next_phase ^ 1);
                    const uint32_t local_bar = smem_u32(&ctrl->full[stage]);
                    const uint32_t bar = PAIR ? map_to_cta(local_bar, leader) : local_bar;
                    const uint32_t sP = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
                    int k_base;
                    const int gk = grp_k(kb, k_base);
                    const int c0 = (kb - k_base) * BK;
                    if (issuer) {
                        if (rank == 0)
                            mbar_arrive_expect_tx(local_bar, CTAS * (do_p ? Cfg::A_BYTES : Cfg::B_BYTES));
                        if (do_p) issue(false, map_p(gk), sP, bar, m0, c0);
                        if (do_q) issue(true, map_q(gn + gk), sP + Cfg::A_BYTES, bar, n0, c0);
                    }
                    ++issued;
                    stage = next_stage;
                    phase = next_phase;
                }
            }
            if (!ok && rank == 0 && do_p && lane == 0) {
                // Abort path: let every copy counted on this CTA's barriers land before exit.
                const uint32_t n_back = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
                uint32_t s2 = stage, ph = phase;
                for (uint32_t i = 0; i < n_back; ++i) {
                    if (s2 == 0) { s2 = STAGES; ph ^= 1; }
                    --s2;
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&ctrl->full[s2]), ph)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES / 8) {
                            atomicCAS(p.status, 0, DEV_TIMEOUT_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer (the even CTA of a pair)
        if (rank == 0) {
            constexpr uint32_t idesc = umma_idesc(1, BM * CTAS, BN, P_MN ? 1 : 0, Q_MN ? 1 : 0);
            // K-major tile: rows of 128 B, 8-row groups 1024 B apart; +32 B per UMMA_K step.
            // MN-major tile: 64-wide column panels of BK rows x 128 B (LBO = panel pitch),
            //                8-row groups 1024 B apart (SBO); +16 rows = 2048 B per UMMA_K step.
            constexpr uint32_t P_LBO = P_MN ? 64 * BK * 2 : 16, P_STEP = P_MN ? UMMA_K * 128 : UMMA_K * 2;
            constexpr uint32_t Q_LBO = Q_MN ? 64 * BK * 2 : 16, Q_STEP = Q_MN ? UMMA_K * 128 : UMMA_K * 2;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            WorkItem w;
            const uint64_t descP0 = umma_smem_desc(smem_u32(tiles), P_LBO, 1024);
            const uint64_t descQ0 = umma_smem_desc(smem_u32(tiles) + Cfg::A_BYTES, Q_LBO, 1024);
            const uint16_t pair_mask = static_cast<uint16_t>(3u << leader);
            (void)pair_mask;
            // as in the producers: the next stage's barrier is probed while this stage's MMAs are issued
            bool ready = mbar_test_wait(smem_u32(&ctrl->full[0]), 0);
            const bool issuer = elect_one();  // one lane, the same for the whole loop (tcgen05.commit tracks the
                                              // MMAs of the thread that executes it)
            for (int i = 0; ok && next_work(i, w); ++i) {
                narrow_to_krank(p, krank, w);
                const uint32_t acc = i & 1, acc_phase = (i >> 1) & 1;
                ok = mbar_wait<PAIR>(smem_u32(&ctrl->tmem_empty[acc]), acc_phase ^ 1, abort_flag, p.status,
                                     DEV_TIMEOUT_TMEM_E);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    if (!__all_sync(0xffffffffu, ready)) {
                        ok = mbar_wait(smem_u32(&ctrl->full[stage]), phase, abort_flag, p.status, DEV_TIMEOUT_FULL);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    const uint32_t next_stage = stage + 1 == STAGES ? 0 : stage + 1;
                    const uint32_t next_phase = next_stage == 0 ? phase ^ 1 : phase;
                    ready = mbar_test_wait(smem_u32(&ctrl->full[next_stage]), next_phase);
                    // only the 14-bit start-address field of a descriptor changes from stage to stage and
                    // from one UMMA_K step to the next: add to the low word
                    const uint32_t st_off = (stage * Cfg::STAGE_BYTES) >> 4;
                    if (issuer) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint64_t dP = descP0 + (st_off + ((k * P_STEP) >> 4));
                            const uint64_t dQ = descQ0 + (st_off + ((k * Q_STEP) >> 4));
                            umma_f16<CTAS>(d_tmem, dP, dQ, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
                        }
                        // frees the stage (in both CTAs of a pair) when the MMAs retire
                        if constexpr (PAIR) umma_commit_2cta(smem_u32(&ctrl->empty[stage]), pair_mask);
                        else umma_commit(smem_u32(&ctrl->empty[stage]));
                        // the accumulator is complete when the last block's MMAs retire
                        if (kb == w.kb1 - 1) {
                            if constexpr (PAIR) umma_commit_2cta(smem_u32(&ctrl->tmem_full[acc]), pair_mask);
                            else umma_commit(smem_u32(&ctrl->tmem_full[acc]));
                        }
                    }
                    stage = next_stage;
                    phase = next_phase;
                }
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------- epilogue
        const int q = warp & 3;            // TMEM lane quarter
        const int hsel = (warp - 4) >> 2;  // which half of the column chunks
        uint32_t sk_phase = 0, old_phase = 0;
        const uint32_t old_bar = smem_u32(&ctrl->old_bar[warp - 4]);
        bool ok = true;
        WorkItem w;
        for (int i = 0; ok && next_work(i, w); ++i) {
            const uint32_t acc = i & 1, acc_phase = (i >> 1) & 1;
            ok = mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, abort_flag, p.status, DEV_TIMEOUT_TMEM_F);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row0 = (w.m_blk * CTAS + static_cast<int>(rank)) * BM + q * 32;
            int n_base;
            const int gn = grp_n(w.n_blk, n_base);
            const int col_tile = (w.n_blk - n_base) * BN;   // first column of the tile inside its own product
            const CUtensorMap* tmDg = map_d(gn);
            const CUtensorMap* tmD32g = map_d32(gn);
            const uint32_t taddr = tmem_base + acc * Cfg::ACC_STRIDE + (static_cast<uint32_t>(q * 32) << 16);
            uint8_t* my_buf = epi_bufs + (warp - 4) * (Cfg::EPI_BUFS * EPI_BUF_BYTES);
            auto release_acc = [&]() {
                tc_fence_before();
                __syncwarp();
                if (elect_one()) {
                    if constexpr (PAIR) mbar_arrive_cluster(smem_u32(&ctrl->tmem_empty[acc]), leader);
                    else mbar_arrive(smem_u32(&ctrl->tmem_empty[acc]));
                }
            };
            if constexpr (EPI == 1) {
                epilogue_swiglu(p, map_d(0), map_d(1), map_d(2), my_buf, taddr, hsel, row0, lane, w.n_blk * 128);
                release_acc();
            } else if constexpr (EPI == 2) {
                epilogue_store_stats<Cfg::EPI_BUFS>(p, &tmD, my_buf, taddr, hsel, row0, lane, w.n_blk * BN, w.n_blk);
                release_acc();
            } else if (p.ksplit > 1) {
                ok = epilogue_cluster_split<BN, BETA1, CTAS>(p, ctrl, tiles, tmD32g, my_buf, taddr, q, hsel, lane, warp,
                                                             row0, col_tile, krank, static_cast<int>(rank), old_bar,
                                                             old_phase, abort_flag);
                release_acc();
                if (!ok) break;
            } else if (w.sk_item < 0) {
                ok = epilogue_store_bf16<BN, BETA1, false, Cfg::EPI_BUFS>(p, tmDg, my_buf, taddr, nullptr, 0, 0, q, hsel, row0, lane,
                                                               col_tile, old_bar, old_phase, abort_flag);
                release_acc();
                if (!ok) break;
            } else if (p.sk_peer) {
                constexpr int G = BN / 32;
                const int maxg = (G + p.sk_splits - 1) / p.sk_splits;
                float* region = p.ws + (static_cast<size_t>(w.sk_tile) * CTAS + rank) * p.sk_splits * (p.sk_splits - 1) *
                                           maxg * (8 * BM * 4);
                ok = epilogue_peer_split<BN, BETA1>(p, ctrl, region, p.sk_counters + w.sk_tile * CTAS + rank, tmD32g,
                                                    my_buf, taddr, q, hsel, lane, warp, row0, col_tile, w.sk_split,
                                                    old_bar, old_phase, sk_phase, abort_flag);
                sk_phase ^= 1;
                release_acc();
                if (!ok) break;
            } else {
                // One range of a split tile: park the partial, count the arrival, and if every
                // other range of this tile has already arrived, reduce them all and write the tile.
                float* block = p.ws + (static_cast<size_t>(w.sk_item) * CTAS + rank) * Cfg::PARTIAL_FLOATS;
                epilogue_store_partial<BN>(block, taddr, q, hsel, lane);
                release_acc();
                __threadfence();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctrl->sk_written));
                if (warp == 4 && lane == 0) {
                    if (mbar_wait(smem_u32(&ctrl->sk_written), sk_phase, abort_flag, p.status, DEV_TIMEOUT_PEER)) {
                        int* counter = p.sk_counters + w.sk_tile * CTAS + rank;
                        __threadfence();  // the four warps' partial stores, ordered before the count
                        const int prev = atomicAdd(counter, 1);
                        const int last = prev == p.sk_splits - 1;
                        if (last) atomicExch(counter, 0);  // leave the counter ready for the next launch
                        ctrl->sk_last = last;
                        __threadfence();
                    }
                    mbar_arrive(smem_u32(&ctrl->sk_decided));
                }
                ok = mbar_wait(smem_u32(&ctrl->sk_decided), sk_phase, abort_flag, p.status, DEV_TIMEOUT_PEER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                sk_phase ^= 1;
                if (ctrl->sk_last) {
                    __threadfence();
                    const float* first = p.ws + (static_cast<size_t>(w.sk_tile) * p.sk_splits * CTAS + rank) *
                                                    Cfg::PARTIAL_FLOATS;
                    ok = epilogue_store_bf16<BN, BETA1, true, Cfg::EPI_BUFS>(p, tmDg, my_buf, 0, first,
                                                              static_cast<size_t>(CTAS) * Cfg::PARTIAL_FLOATS, p.sk_splits,
                                                              q, hsel, row0, lane, col_tile, old_bar, old_phase,
                                                              abort_flag);
                    if (!ok) break;
                }
                // every warp must have read sk_last before the next split item overwrites it
                __syncwarp();
            }
        }
        // every TMA store of this warp must have read its staging buffer before the CTA gives up its shared
        // memory; the writes themselves are complete when the grid is
        if (elect_one()) tma_store_wait_read<0>();
    }

    // ------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (clustered) {  // no CTA may leave while another can still touch its smem/TMEM
        cluster_arrive_release();
        cluster_wait_acquire();
    }
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<CTAS>(tmem_base, Cfg::TMEM_COLS);
    }
    // A kernel that ran beside its predecessor must not finish before it: whoever waits for this
    // kernel next is entitled to see the predecessor's results as well.
    if (p.late_wait && threadIdx.x == 0) griddep_wait();
}

}  // namespace b200
