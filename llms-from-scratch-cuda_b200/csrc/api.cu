// Host side of libb200_linear.so: context, tensor-map cache, plan selection, kernel
// dispatch and the extern "C" entry points declared in include/b200_linear.h.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "../../include/b200_linear.h"
#include "gemm_sm100.cuh"
#include "gemm_simt.cuh"
#include "gemm_tf32x3_sm100.cuh"
#include "ce_shard.cuh"

using namespace b200;

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

struct TmKey {
    const void* ptr;
    uint64_t inner, outer;
    uint32_t box_inner, box_outer;
    uint64_t ld;  // row pitch in elements
    bool operator==(const TmKey& o) const {
        return ptr == o.ptr && inner == o.inner && outer == o.outer && box_inner == o.box_inner &&
               box_outer == o.box_outer && ld == o.ld;
    }
};
struct TmKeyHash {
    size_t operator()(const TmKey& k) const {
        uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
        h ^= (k.inner + 0x7F4A7C15u) * 0xBF58476D1CE4E5B9ull;
        h ^= (k.outer + 0x1CE4E5B9u) * 0x94D049BB133111EBull;
        h ^= (static_cast<uint64_t>(k.box_inner) << 32 | k.box_outer) * 0xD6E8FEB86659FD93ull;
        h ^= (k.ld + 0x6659FD93u) * 0xC2B2AE3D27D4EB4Full;
        return static_cast<size_t>(h ^ (h >> 29));
    }
};

}  // namespace

struct b200_linear_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    float* ws = nullptr;  // split-K workspace
    size_t ws_bytes = 0;
    float* ws2 = nullptr;  // second workspace + counters: for a kernel that overlaps the previous one
    size_t ws2_bytes = 0;
    int* sk_counters2 = nullptr;
    int sk_counters2_len = 0;
    int* status_dev = nullptr;
    int* sk_counters = nullptr;     // arrival counters of split tiles (zero between launches)
    int sk_counters_len = 0;
    long long launches = 0;
    int last_cuda = 0;
    int force_bn = -1, force_pair = 0, force_splits = 0;
    int use_pdl = 1;
    int no_peer_split = 0;
    int overlap_backward = 1;
    int partition_backward = 1;  // 0: dgrad and wgrad both plan for the whole GPU (wgrad still fills dgrad's tail)
    int force_sm_dgrad = 0;      // > 0: dgrad's share of the SMs in matmul_backward, whatever the cost model says
    int tile_group = 0;          // > 0: tiles of the fast dimension per group of the tile order (0 = plain raster)
    int fp32_simt = 0;  // 1: fp32 products on the CUDA cores only (exact fp32 FMA arithmetic)
    EncodeTiledFn encode = nullptr;
    std::unordered_map<TmKey, CUtensorMap, TmKeyHash> tm_cache;
    std::unordered_map<unsigned long long, int> backward_split;  // (M,N,K) -> SM shares of dgrad | wgrad
};

namespace {

int cuda_fail(b200_linear_ctx* ctx, cudaError_t e) {
    if (ctx) ctx->last_cuda = static_cast<int>(e);
    return B200_E_CUDA;
}
#define CU_TRY(ctx, expr)                                    \
    do {                                                     \
        cudaError_t e__ = (expr);                            \
        if (e__ != cudaSuccess) return cuda_fail((ctx), e__); \
    } while (0)

// bf16 2-D tensor map over a row-major [outer][inner] matrix whose rows are `ld` elements apart (0 = dense:
// ld = inner); 128-byte swizzle for 64-element-wide boxes, 64-byte swizzle for 32-element-wide ones.
int get_tensor_map(b200_linear_ctx* ctx, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                   uint32_t box_outer, CUtensorMap* out, uint64_t ld = 0) {
    if (ld == 0) ld = inner;
    TmKey key{ptr, inner, outer, box_inner, box_outer, ld};
    auto it = ctx->tm_cache.find(key);
    if (it != ctx->tm_cache.end()) {
        *out = it->second;
        return B200_OK;
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ctx->encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                             box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             box_inner == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        ctx->last_cuda = 100000 + static_cast<int>(r);
        return B200_E_CUDA;
    }
    if (ctx->tm_cache.size() > 8192) ctx->tm_cache.clear();
    ctx->tm_cache.emplace(key, *out);
    return B200_OK;
}

// fp32 2-D tensor map over a row-major [outer][inner] matrix, box {32 elements = 128 bytes, box_outer}.
int get_tensor_map_f32(b200_linear_ctx* ctx, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_outer,
                       CUtensorMap* out, bool atom32 = false) {
    TmKey key{ptr, inner, outer, (atom32 ? 0x48000u : 0x40000u) + 32u, box_outer, inner};
    auto it = ctx->tm_cache.find(key);
    if (it != ctx->tm_cache.end()) {
        *out = it->second;
        return B200_OK;
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * 4};
    cuuint32_t box[2] = {32, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ctx->encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE,
                             atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        ctx->last_cuda = 100000 + static_cast<int>(r);
        return B200_E_CUDA;
    }
    if (ctx->tm_cache.size() > 8192) ctx->tm_cache.clear();
    ctx->tm_cache.emplace(key, *out);
    return B200_OK;
}
// fp32 MN-major operand [Kc][rows] (rows a multiple of 32) seen as {32 elements, Kc, rows/32 panels}.
int get_panel_map_f32(b200_linear_ctx* ctx, const void* ptr, uint64_t rows, uint64_t kc, uint32_t panels,
                      CUtensorMap* out) {
    TmKey key{ptr, rows, kc, 0x50000u + panels, T32_BK, rows};
    auto it = ctx->tm_cache.find(key);
    if (it != ctx->tm_cache.end()) {
        *out = it->second;
        return B200_OK;
    }
    cuuint64_t dims[3] = {32, kc, rows / 32};
    cuuint64_t strides[2] = {rows * 4, 128};
    cuuint32_t box[3] = {32, T32_BK, panels};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = ctx->encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        ctx->last_cuda = 100000 + static_cast<int>(r);
        return B200_E_CUDA;
    }
    if (ctx->tm_cache.size() > 8192) ctx->tm_cache.clear();
    ctx->tm_cache.emplace(key, *out);
    return B200_OK;
}

int ensure_workspace(b200_linear_ctx* ctx, size_t bytes, int set = 0) {
    float*& ws = set ? ctx->ws2 : ctx->ws;
    size_t& have = set ? ctx->ws2_bytes : ctx->ws_bytes;
    if (bytes <= have) return B200_OK;
    if (ws) CU_TRY(ctx, cudaFree(ws));
    ws = nullptr;
    have = 0;
    size_t want = bytes + (bytes >> 2);
    CU_TRY(ctx, cudaMalloc(&ws, want));
    have = want;
    return B200_OK;
}

inline int ceil_div_i(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

constexpr int kMaxDevices = 64;

// A context belongs to the device that was current when it was created; its kernels, scratch memory and
// tensor maps are that device's.  Calls made with another device current are refused.
bool on_context_device(const b200_linear_ctx* ctx) {
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess && dev == ctx->device;
}

}  // namespace

// ------------------------------------------------------------------- plan
namespace {

struct Decomp {
    int m_tiles, n_tiles, kb_total, tiles;
    int dp_tiles, sk_splits, kb_per_sk, sk_items;
};

// How the output tiles of one product are spread over `slots` CTAs (or CTA pairs).
//   force_splits >= 2: every tile is cut into that many ranges of the contraction;
//   force_splits == 1: no tile is cut;
//   force_splits == 0: the ragged last wave is cut so that it fills the slots, when that saves
//                      enough main-loop time to pay for the fp32 round trip of the partials.
Decomp decompose(int Mo, int No, int Kc, int bn, int ctas, int slots, int force_splits) {
    Decomp d;
    d.m_tiles = ceil_div_i(Mo, BM * ctas);
    d.n_tiles = ceil_div_i(No, bn);
    d.kb_total = ceil_div_i(Kc, BK);
    d.tiles = d.m_tiles * d.n_tiles;
    d.dp_tiles = d.tiles;
    d.sk_splits = 1;
    d.kb_per_sk = d.kb_total;
    d.sk_items = 0;
    int splits = 1, sk_tiles = 0;
    if (force_splits >= 2) {
        splits = force_splits < d.kb_total ? force_splits : d.kb_total;
        sk_tiles = d.tiles;
    } else if (force_splits == 0) {
        const int rem = d.tiles % slots;
        if (rem != 0) {
            splits = slots / rem;
            const int by_work = d.kb_total / 4;  // at least 4 blocks per range
            if (splits > by_work) splits = by_work;
            sk_tiles = rem;
        }
    }
    if (splits >= 2) {
        const int per = ceil_div_i(d.kb_total, splits);
        splits = ceil_div_i(d.kb_total, per);
        // worth it only if the cut saves at least ~10 blocks of main loop (or was asked for)
        if (splits >= 2 && (force_splits >= 2 || d.kb_total - per >= 10)) {
            d.dp_tiles = d.tiles - sk_tiles;
            d.sk_splits = splits;
            d.kb_per_sk = per;
            d.sk_items = sk_tiles * splits;
        }
    }
    return d;
}

// Main-loop cost of one BK = 64 block of one work item, in nanoseconds, measured on a B200 (graph replay,
// SM clock ~1.85 GHz), the same for the three operand layouts.  `lo`: a few CTAs alone on the GPU -- the
// issue loop's floor of ~480 cycles per block, or the tensor pipe for the 256-wide pair tile.  `hi`: all
// 148 SMs busy, where the shared L2 -> SM feed adds to it.  In between, by the busy fraction of the SMs.
double per_block_ns(int bn, int ctas, double busy) {
    double lo, hi;
    if (ctas == 2) {
        lo = bn == 256 ? 275.0 : 256.0;
        hi = bn == 256 ? 386.0 : 256.0;
    } else {
        lo = bn == 256 ? 275.0 : 256.0;
        hi = bn == 256 ? 480.0 : bn == 192 ? 430.0 : bn == 128 ? 320.0 : 260.0;  // slowest GPUs seen, not the average
    }
    if (busy > 1.0) busy = 1.0;
    return lo + (hi - lo) * busy;
}

// Cost outside the main loops: launch gap, set-up, first copies' latency, tear-down (a CTA pair also
// waits for its cluster to be scheduled, the longer the fuller the GPU, and synchronises it twice), and
// the last, exposed epilogue.
double fixed_ns(int bn, int ctas, double busy) {
    if (busy > 1.0) busy = 1.0;
    return 2560.0 + (ctas == 2 ? 1840.0 * busy : 0.0) + 600.0 + 4.0 * bn;
}

// Estimated duration in nanoseconds of the persistent schedule described by `d`.
double plan_cost_ns(const Decomp& d, int bn, int ctas, int slots) {
    const long long items = static_cast<long long>(d.dp_tiles) + d.sk_items;
    const double busy = static_cast<double>(items < slots ? items : slots) / slots;
    const double per_kb = per_block_ns(bn, ctas, busy);
    const int dp_rounds = (d.dp_tiles + slots - 1) / slots;
    const int sk_rounds = (d.sk_items + slots - 1) / slots;
    // an item cannot go faster than its epilogue (short contractions): ~0.5 us + 8 ns per output column
    const double epi = 500.0 + 8.0 * bn;
    const double dp_item = d.kb_total * per_kb + 300.0;  // + pipeline refill at the item boundary
    const double sk_item = d.kb_per_sk * per_kb + 300.0;
    double t = dp_rounds * (dp_item > epi ? dp_item : epi) + sk_rounds * (sk_item > epi ? sk_item : epi);
    t += fixed_ns(bn, ctas, busy);
    if (d.sk_items > 0) {
        // partial sums through L2: peers exchanging slices (all resident) or a last arriver adding whole tiles
        const bool peer = d.sk_items <= slots && d.sk_splits <= bn / 32;
        t += peer ? 5000.0 + 750.0 * d.sk_splits : 6000.0 + 1500.0 * d.sk_splits;
    }
    return t;
}

// Same for a cluster split: every tile shared by `ks` CTAs (or pairs) that add up through distributed
// shared memory; the exchange costs about a microsecond per member.
double cluster_split_cost_ns(int tiles, int kb_total, int ks, int bn, int ctas, int sm_count) {
    const int per = ceil_div_i(kb_total, ks);
    const double busy = static_cast<double>(tiles) * ks * ctas / sm_count;
    return per * per_block_ns(bn, ctas, busy) + 300.0 + fixed_ns(bn, ctas, busy) + 1500.0 + 1000.0 * ks;
}

// Clusters of `size` CTAs (one CTA per SM) that can be resident at once, measured on a 148-SM B200
// with cudaOccupancyMaxActiveClusters and scaled to the SM count at hand.
int max_resident_clusters(int size, int sm_count) {
    static const int per148[9] = {0, 148, 74, 45, 33, 26, 22, 15, 15};
    if (size < 1 || size > 8) return 0;
    return per148[size] * sm_count / 148;
}

}  // namespace

namespace {
// The plan for an output of Mo x No with a contraction of Kc.  n_align > 0: only tile widths that divide it (a
// grouped launch, where a tile must not straddle two products).
void plan_dims(int Mo, int No, int Kc, int sm_count, int n_align, b200_linear_plan_t* plan);
}  // namespace

extern "C" int b200_linear_plan_bf16(int which, int beta1, int M, int N, int K, int sm_count,
                                     b200_linear_plan_t* plan) {
    (void)beta1;
    if (!plan || M <= 0 || N <= 0 || K <= 0 || sm_count <= 0 || which < 0 || which > 2) return B200_E_BADARG;
    int Mo, No, Kc;
    if (which == B200_GEMM_FWD_NN) { Mo = M; No = N; Kc = K; }
    else if (which == B200_GEMM_DGRAD_NT) { Mo = M; No = K; Kc = N; }
    else { Mo = K; No = N; Kc = M; }
    memset(plan, 0, sizeof(*plan));
    if ((N % 8) != 0 || (K % 8) != 0) {  // a row pitch that TMA cannot describe
        plan->bn = 0;
        plan->splits = 1;
        plan->tiles = ceil_div_i(Mo, ST_BM) * ceil_div_i(No, ST_BN);
        plan->dp_tiles = plan->tiles;
        return B200_OK;
    }
    plan_dims(Mo, No, Kc, sm_count, 0, plan);
    return B200_OK;
}

namespace {
void plan_dims(int Mo, int No, int Kc, int sm_count, int n_align, b200_linear_plan_t* plan) {
    static const int cand[6][2] = {{256, 2}, {128, 2}, {256, 1}, {192, 1}, {128, 1}, {64, 1}};
    double best = -1.0;
    for (int ci = 0; ci < 6; ++ci) {
        const int bn = cand[ci][0], ctas = cand[ci][1];
        if (n_align > 0 && (n_align % bn) != 0) continue;
        if (bn > 64 && bn - No >= 64) continue;  // tile much wider than the output
        if (ctas == 2 && sm_count < 2) continue;
        const int slots = sm_count / ctas;
        const Decomp d = decompose(Mo, No, Kc, bn, ctas, slots, 0);
        const double c = plan_cost_ns(d, bn, ctas, slots);
        if (best < 0 || c < best) {
            best = c;
            plan->bn = bn;
            plan->cta_pair = ctas == 2;
            plan->splits = d.sk_splits;
            plan->tiles = d.tiles;
            plan->dp_tiles = d.dp_tiles;
            plan->sk_items = d.sk_items;
            plan->cluster_split = 0;
            plan->est_ns = static_cast<int>(c);
            plan->waves_x100 = static_cast<int>(100LL * (d.dp_tiles + d.sk_items) / slots);
        }
        // Small outputs: every tile shared by a cluster whose members split the contraction and add
        // up through distributed shared memory -- only if all clusters are resident in one wave.
        const int kb_total = ceil_div_i(Kc, BK);
        for (int ks = 8 / ctas; ks >= 2; --ks) {
            if (ks > bn / 32 || kb_total / ks < 4) continue;
            if (d.tiles > max_resident_clusters(ks * ctas, sm_count)) continue;
            const int per = ceil_div_i(kb_total, ks);
            if (ceil_div_i(kb_total, per) != ks) continue;
            const double cc = cluster_split_cost_ns(d.tiles, kb_total, ks, bn, ctas, sm_count);
            if (cc < best) {
                best = cc;
                plan->bn = bn;
                plan->cta_pair = ctas == 2;
                plan->splits = 1;
                plan->tiles = d.tiles;
                plan->dp_tiles = d.tiles;
                plan->sk_items = 0;
                plan->cluster_split = ks;
                plan->est_ns = static_cast<int>(cc);
                plan->waves_x100 = static_cast<int>(100LL * d.tiles * ks / slots);
            }
        }
    }
    plan->m_fastest = Mo <= No ? 1 : 0;
}
}  // namespace

// ---------------------------------------------------------------- launch
namespace {

// MN-major operand [Kc][rows] (rows a multiple of 64) seen as {64 elements, Kc, rows/64 panels}
// so that one copy brings every 64-wide panel of a stage into its own 128B-swizzled block.
int get_panel_map(b200_linear_ctx* ctx, const void* ptr, uint64_t rows, uint64_t kc, uint32_t panels,
                  CUtensorMap* out, uint64_t ld = 0) {
    if (ld == 0) ld = rows;
    TmKey key{ptr, rows, kc, 0x30000u + panels, BK, ld};
    auto it = ctx->tm_cache.find(key);
    if (it != ctx->tm_cache.end()) {
        *out = it->second;
        return B200_OK;
    }
    cuuint64_t dims[3] = {64, kc, rows / 64};
    cuuint64_t strides[2] = {ld * 2, 128};
    cuuint32_t box[3] = {64, BK, panels};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = ctx->encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box,
                             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        ctx->last_cuda = 100000 + static_cast<int>(r);
        return B200_E_CUDA;
    }
    if (ctx->tm_cache.size() > 8192) ctx->tm_cache.clear();
    ctx->tm_cache.emplace(key, *out);
    return B200_OK;
}

int ensure_counters(b200_linear_ctx* ctx, int n, int set = 0) {
    int*& counters = set ? ctx->sk_counters2 : ctx->sk_counters;
    int& have = set ? ctx->sk_counters2_len : ctx->sk_counters_len;
    if (n <= have) return B200_OK;
    if (counters) CU_TRY(ctx, cudaFree(counters));
    counters = nullptr;
    have = 0;
    const int want = n + 1024;
    CU_TRY(ctx, cudaMalloc(&counters, want * sizeof(int)));
    CU_TRY(ctx, cudaMemset(counters, 0, want * sizeof(int)));
    have = want;
    return B200_OK;
}

// EPI = 0: one product (gx is GemmNoMaps); EPI = 3: grouped launch (gx carries the other products' maps)
template <int BN, bool P_MN, bool Q_MN, bool BETA1, int CTAS, int EPI>
int launch_one(b200_linear_ctx* ctx, const typename GemmExtraMaps<EPI>::type& gx, const CUtensorMap& tmP, const CUtensorMap& tmQ, const CUtensorMap& tmD,
               const CUtensorMap& tmD32, const GemmParams& gp, int grid) {
    using Cfg = TileCfg<BN, CTAS>;
    if (gp.ksplit > 1) {  // the receive space of the cluster exchange must fit the pipeline stages
        const int maxg = (BN / 32 + gp.ksplit - 1) / gp.ksplit;
        if ((gp.ksplit - 1) * maxg * 8 * BM * 16 > Cfg::STAGES * Cfg::STAGE_BYTES || gp.ksplit > BN / 32 ||
            CTAS * gp.ksplit > 8)
            return B200_E_BADARG;
    }
    // the opt-in to more than 48 KB of dynamic shared memory is a per-device property of the function
    static bool configured[kMaxDevices] = {};
    auto kern = gemm_bf16_sm100<BN, P_MN, Q_MN, BETA1, CTAS, EPI>;
    if (!configured[ctx->device]) {
        CU_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        configured[ctx->device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS * gp.ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // The kernel's set-up may overlap the tail of the previous kernel in the stream; it waits
    // (griddepcontrol.wait) before it touches global memory.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = ctx->use_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    CU_TRY(ctx, cudaLaunchKernelEx(&cfg, kern, tmP, tmQ, tmD, tmD32, gx, gp));
    ctx->launches++;
    return B200_OK;
}

template <bool P_MN, bool Q_MN, bool BETA1, int EPI>
int launch_bn(b200_linear_ctx* ctx, const typename GemmExtraMaps<EPI>::type& gx, int bn, int ctas, const CUtensorMap& tmP, const CUtensorMap& tmQ,
              const CUtensorMap& tmD, const CUtensorMap& tmD32, const GemmParams& gp, int grid) {
    if (ctas == 2) {
        switch (bn) {
            case 256: return launch_one<256, P_MN, Q_MN, BETA1, 2, EPI>(ctx, gx, tmP, tmQ, tmD, tmD32, gp, grid);
            case 128: return launch_one<128, P_MN, Q_MN, BETA1, 2, EPI>(ctx, gx, tmP, tmQ, tmD, tmD32, gp, grid);
            default: return B200_E_BADARG;
        }
    }
    switch (bn) {
        case 256: return launch_one<256, P_MN, Q_MN, BETA1, 1, EPI>(ctx, gx, tmP, tmQ, tmD, tmD32, gp, grid);
        case 192: return launch_one<192, P_MN, Q_MN, BETA1, 1, EPI>(ctx, gx, tmP, tmQ, tmD, tmD32, gp, grid);
        case 128: return launch_one<128, P_MN, Q_MN, BETA1, 1, EPI>(ctx, gx, tmP, tmQ, tmD, tmD32, gp, grid);
        case 64: return launch_one<64, P_MN, Q_MN, BETA1, 1, EPI>(ctx, gx, tmP, tmQ, tmD, tmD32, gp, grid);
        default: return B200_E_BADARG;
    }
}

template <bool P_MN, bool Q_MN, int EPI>
int launch_beta(b200_linear_ctx* ctx, const typename GemmExtraMaps<EPI>::type& gx, int bn, int ctas, int beta1, const CUtensorMap& tmP,
                const CUtensorMap& tmQ, const CUtensorMap& tmD, const CUtensorMap& tmD32, const GemmParams& gp, int grid) {
    return beta1 ? launch_bn<P_MN, Q_MN, true, EPI>(ctx, gx, bn, ctas, tmP, tmQ, tmD, tmD32, gp, grid)
                 : launch_bn<P_MN, Q_MN, false, EPI>(ctx, gx, bn, ctas, tmP, tmQ, tmD, tmD32, gp, grid);
}
// what a single product passes where a grouped launch has its other products' maps
const GemmNoMaps g_no_group = {};

template <typename T>
int launch_simt(b200_linear_ctx* ctx, int which, int beta1, T* out, const T* x, const T* y, int M, int N,
                int K);

// SM shares for the two independent kernels of one matmul_backward (0, 0 = one after the other on all SMs).
void split_sms_for_backward(b200_linear_ctx* ctx, int M, int N, int K, int* sm_dgrad, int* sm_wgrad) {
    *sm_dgrad = 0;
    *sm_wgrad = 0;
    if ((N % 8) != 0 || (K % 8) != 0) return;
    const unsigned long long key = (static_cast<unsigned long long>(M) << 42) ^ (static_cast<unsigned long long>(N) << 21) ^
                                   static_cast<unsigned long long>(K);
    if (ctx->force_sm_dgrad > 0 && ctx->force_sm_dgrad < ctx->sm_count - 1) {
        *sm_dgrad = ctx->force_sm_dgrad;
        *sm_wgrad = (ctx->sm_count - ctx->force_sm_dgrad) & ~1;
        return;
    }
    auto it = ctx->backward_split.find(key);
    if (it != ctx->backward_split.end()) {
        *sm_dgrad = it->second >> 16;
        *sm_wgrad = it->second & 0xFFFF;
        return;
    }
    b200_linear_plan_t pd, pw;
    b200_linear_plan_bf16(B200_GEMM_DGRAD_NT, 0, M, N, K, ctx->sm_count, &pd);
    b200_linear_plan_bf16(B200_GEMM_WGRAD_TN, 1, M, N, K, ctx->sm_count, &pw);
    // one after the other: two set-ups and two tails are exposed (the estimates contain one each)
    double best = static_cast<double>(pd.est_ns) + pw.est_ns + 2500.0;
    int best_d = 0, best_w = 0;
    for (int sd = 8; sd <= ctx->sm_count - 8; sd += 4) {
        const int sw = (ctx->sm_count - sd) & ~1;
        b200_linear_plan_bf16(B200_GEMM_DGRAD_NT, 0, M, N, K, sd, &pd);
        b200_linear_plan_bf16(B200_GEMM_WGRAD_TN, 1, M, N, K, sw, &pw);
        // both feed from the same L2; among equal maxima (a weight gradient shared out to clusters needs a
        // fixed number of SMs, whatever it is offered) the split that also shortens the other kernel wins
        const double hi = pd.est_ns > pw.est_ns ? pd.est_ns : pw.est_ns, lo = pd.est_ns + pw.est_ns - hi;
        const double t = hi * 1.05 + 0.1 * lo;
        if (t < best) {
            best = t;
            best_d = sd;
            best_w = sw;
        }
    }
    if (ctx->backward_split.size() > 4096) ctx->backward_split.clear();
    ctx->backward_split.emplace(key, (best_d << 16) | best_w);
    *sm_dgrad = best_d;
    *sm_wgrad = best_w;
}

// From a plan to the kernel's work schedule: tile shape, splits, grid, split-K scratch.  `honour_force`: take the
// context's forced tile shape (a test / tuning knob) instead of the plan's.
int schedule_launch(b200_linear_ctx* ctx, const b200_linear_plan_t& plan, int Mo, int No, int Kc, int sm_count, int overlap_prev,
                    bool honour_force, GemmParams& gp, int& bn_out, int& ctas_out, int& grid_out) {
    int rc;
    int bn = plan.bn, ctas = plan.cta_pair ? 2 : 1, force_splits = 0, ksplit = plan.cluster_split > 1 ? plan.cluster_split : 1;
    if (honour_force && ctx->force_bn > 0) {
        bn = ctx->force_bn;
        ctas = ctx->force_pair ? 2 : 1;
        force_splits = ctx->force_splits;
        ksplit = 1;
        if (force_splits < 0) {  // cluster split: |splits| members per tile
            ksplit = -force_splits;
            force_splits = 1;
            const int kb = ceil_div_i(Kc, BK);
            if (ksplit > kb) ksplit = kb;
            if (ksplit < 1) ksplit = 1;
            const int per = ceil_div_i(kb, ksplit);
            ksplit = ceil_div_i(kb, per);  // every member owns at least one block
        }
    }
    if (ksplit > 1) force_splits = 1;
    if (sm_count < ctas) return B200_E_NODEVICE;
    const int max_slots = ksplit > 1 ? 0x7FFFFFFF : sm_count / ctas;  // CTAs (or pairs) resident at once
    const Decomp d = decompose(Mo, No, Kc, bn, ctas, ksplit > 1 ? 1 : max_slots, force_splits);
    const long long items = static_cast<long long>(d.dp_tiles) + d.sk_items;
    if (items * ksplit * ctas > 0x7FFFFFFFLL || static_cast<long long>(d.tiles) * (d.sk_splits > 1 ? d.sk_splits : 1) > 0x7FFFFFFFLL)
        return B200_E_TOOBIG;
    // cluster split: one cluster per tile; otherwise a persistent grid of at most one CTA (pair) per SM
    const int slots = items < max_slots ? static_cast<int>(items) : max_slots;

    gp.Mo = Mo; gp.No = No; gp.Kc = Kc;
    gp.m_tiles = d.m_tiles; gp.n_tiles = d.n_tiles; gp.kb_total = d.kb_total;
    gp.m_fastest = plan.m_fastest;
    // Grouped tile order (B200_LINEAR_TILE_GROUP=n): measured no gain over the plain raster on any shape,
    // up to 8192 x 32000 x 32000, with the runs interleaved; off unless asked for.
    gp.group = ctx->tile_group > 0 ? ctx->tile_group : 0;
    gp.dp_tiles = d.dp_tiles; gp.sk_splits = d.sk_splits; gp.kb_per_sk = d.kb_per_sk; gp.sk_items = d.sk_items;
    gp.ksplit = ksplit;
    gp.late_wait = (overlap_prev && ctx->use_pdl && ctx->overlap_backward) ? 1 : 0;
    gp.out = nullptr;
    gp.status = ctx->status_dev;
    gp.ws = nullptr;
    gp.sk_counters = nullptr;
    gp.sk_peer = 0;
    if (d.sk_items > 0) {
        // The ranges of a split tile can exchange partial sums among themselves only if they are all
        // running at once: each must be the first work item of its own CTA (pair) of a grid that fits.
        const int groups = bn / 32;
        gp.sk_peer = (d.sk_items <= max_slots && d.sk_splits <= groups && !ctx->no_peer_split) ? 1 : 0;
        size_t ws_bytes = static_cast<size_t>(d.sk_items) * ctas * BM * bn * sizeof(float);
        if (gp.sk_peer) {
            const int maxg = (groups + d.sk_splits - 1) / d.sk_splits;
            ws_bytes = static_cast<size_t>(d.tiles - d.dp_tiles) * ctas * d.sk_splits * (d.sk_splits - 1) * maxg *
                       (8 * BM * 4) * sizeof(float);
        }
        const int set = overlap_prev ? 1 : 0;  // never share scratch with a kernel that may still be running
        rc = ensure_workspace(ctx, ws_bytes, set);
        if (rc) return rc;
        rc = ensure_counters(ctx, (d.tiles - d.dp_tiles) * ctas, set);
        if (rc) return rc;
        gp.ws = set ? ctx->ws2 : ctx->ws;
        gp.sk_counters = set ? ctx->sk_counters2 : ctx->sk_counters;
    }

    gp.grp_n[0] = gp.grp_n[1] = gp.grp_k[0] = gp.grp_k[1] = GRP_NONE;
    bn_out = bn;
    ctas_out = ctas;
    grid_out = slots * ctas * ksplit;
    return B200_OK;
}

// One bf16 product on the tensor cores (or the CUDA-core kernel for TMA-unfriendly pitches).
// overlap_prev = 1: the caller vouches that this product neither reads what the kernel launched just
// before it on the stream writes, nor writes what that kernel touches (the weight gradient after the
// input gradient of the same matmul_backward).  The kernel then starts on whatever SMs that kernel
// has already left and only waits for it before it finishes itself, so that completion order, and with it
// every later kernel's view of memory, stays what the stream promises.
// ld_out / ld_x / ld_y: row pitch in elements of the output and of the two inputs (0 = dense, the inner
// extent), for operands that are column ranges of a wider matrix (a vocabulary shard of the LM head).
int gemm_bf16(b200_linear_ctx* ctx, int which, int beta1, void* out, const void* x, const void* y, int M,
              int N, int K, int overlap_prev = 0, int sm_limit = 0, long long ld_out = 0, long long ld_x = 0,
              long long ld_y = 0) {
    if (!ctx || !out || !x || !y || M <= 0 || N <= 0 || K <= 0 || which < 0 || which > 2)
        return B200_E_BADARG;
    if (!on_context_device(ctx)) return B200_E_BADARG;
    {   // inner extents of out, x, y for this product
        const long long in_out = which == B200_GEMM_DGRAD_NT ? K : N;
        const long long in_x = which == B200_GEMM_DGRAD_NT ? N : K;
        const long long in_y = N;
        if ((ld_out && ld_out < in_out) || (ld_x && ld_x < in_x) || (ld_y && ld_y < in_y)) return B200_E_BADARG;
        if (ld_out == in_out) ld_out = 0;
        if (ld_x == in_x) ld_x = 0;
        if (ld_y == in_y) ld_y = 0;
    }
    const bool pitched = ld_out || ld_x || ld_y;
    if (pitched && ((ld_out | ld_x | ld_y) % 8) != 0) return B200_E_BADARG;  // TMA needs 16-byte row pitches
    // sm_limit > 0: plan for, and occupy, only that many SMs (a concurrent kernel has the others)
    const int sm_count = (sm_limit > 0 && sm_limit < ctx->sm_count) ? sm_limit : ctx->sm_count;
    b200_linear_plan_t plan;
    int rc = b200_linear_plan_bf16(which, beta1, M, N, K, sm_count, &plan);
    if (rc) return rc;
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x) |
                             reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    if ((plan.bn == 0 || !aligned16) && pitched) return B200_E_BADARG;  // the CUDA-core kernel takes dense operands only
    if (plan.bn == 0 || !aligned16)
        return launch_simt<__nv_bfloat16>(ctx, which, beta1, static_cast<__nv_bfloat16*>(out),
                                          static_cast<const __nv_bfloat16*>(x),
                                          static_cast<const __nv_bfloat16*>(y), M, N, K);
    int Mo, No, Kc;
    bool p_mn, q_mn;
    if (which == B200_GEMM_FWD_NN) { Mo = M; No = N; Kc = K; p_mn = false; q_mn = true; }
    else if (which == B200_GEMM_DGRAD_NT) { Mo = M; No = K; Kc = N; p_mn = false; q_mn = false; }
    else { Mo = K; No = N; Kc = M; p_mn = true; q_mn = true; }

    GemmParams gp;
    int bn, ctas, grid;
    rc = schedule_launch(ctx, plan, Mo, No, Kc, sm_count, overlap_prev, true, gp, bn, ctas, grid);
    if (rc) return rc;
    gp.out = out;
    const int ksplit = gp.ksplit;

    // Operand P has Mo rows, operand Q has No rows; x,y map onto them per product.
    // K-major: [rows][Kc], box {BK, rows-per-CTA}.  MN-major: [Kc][rows], one 3-D copy of all the
    // CTA's 64-wide panels when rows % 64 == 0, else one 2-D copy {64, BK} per panel.
    const void* P = x;
    const void* Q = y;
    CUtensorMap tmP, tmQ, tmD;
    gp.p_3d = p_mn && (Mo % 64) == 0;
    gp.q_3d = q_mn && (No % 64) == 0;
    if (gp.p_3d) rc = get_panel_map(ctx, P, Mo, Kc, BM / 64, &tmP, ld_x);
    else if (p_mn) rc = get_tensor_map(ctx, P, Mo, Kc, 64, BK, &tmP, ld_x);
    else rc = get_tensor_map(ctx, P, Kc, Mo, BK, BM, &tmP, ld_x);
    if (rc) return rc;
    if (gp.q_3d) rc = get_panel_map(ctx, Q, No, Kc, bn / ctas / 64, &tmQ, ld_y);
    else if (q_mn) rc = get_tensor_map(ctx, Q, No, Kc, 64, BK, &tmQ, ld_y);
    else rc = get_tensor_map(ctx, Q, Kc, No, BK, bn / ctas, &tmQ, ld_y);
    if (rc) return rc;
    // Output map for the epilogue's TMA stores: [Mo][No] bf16, box = 64 columns x 32 rows.
    rc = get_tensor_map(ctx, out, No, Mo, 64, 32, &tmD, ld_out);
    if (rc) return rc;
    CUtensorMap tmD32 = tmD;  // 32-column blocks: the cluster-split and peer-split epilogues use it
    if (ksplit > 1 || gp.sk_peer) {
        rc = get_tensor_map(ctx, out, No, Mo, 32, 32, &tmD32, ld_out);
        if (rc) return rc;
    }

    if (p_mn) return launch_beta<true, true, 0>(ctx, g_no_group, bn, ctas, beta1, tmP, tmQ, tmD, tmD32, gp, grid);
    if (q_mn) return launch_beta<false, true, 0>(ctx, g_no_group, bn, ctas, beta1, tmP, tmQ, tmD, tmD32, gp, grid);
    return launch_beta<false, false, 0>(ctx, g_no_group, bn, ctas, beta1, tmP, tmQ, tmD, tmD32, gp, grid);
}

// Up to three products in one launch (dense operands).
//   FWD_NN   outs[i][M, Ns[i]]  = xs[0][M, K] * ys[i][K, Ns[i]]              (one input, several weights)
//   WGRAD_TN outs[i][K, Ns[i]] (+)= xs[0][M, K]^T * ys[i][M, Ns[i]]          (one input, several output gradients)
//   DGRAD_NT outs[0][M, K]     (+)= sum_i xs[i][M, Ns[i]] * ys[i][K, Ns[i]]^T (one accumulator over all of them:
//                                   the sum is formed in fp32 and rounded once)
// The first two concatenate the products along the output columns (each column tile belongs to one product), the
// third along the contraction.  Shapes or pointers that the tensor-core kernel cannot take this way run as `count`
// single products instead (the input gradient then accumulates through beta = 1, one rounding per product).
int gemm_bf16_grouped(b200_linear_ctx* ctx, int which, int beta1, int count, void* const* outs, const void* const* xs,
                      const void* const* ys, int M, const int* Ns, int K, int overlap_prev = 0, int sm_limit = 0) {
    if (!ctx || !outs || !xs || !ys || !Ns || count < 1 || count > 3 || M <= 0 || K <= 0 || which < 0 || which > 2)
        return B200_E_BADARG;
    if (!on_context_device(ctx)) return B200_E_BADARG;
    const bool k_concat = which == B200_GEMM_DGRAD_NT;
    long long n_total = 0;
    int n_align = 0;
    bool fast = count > 1 && (K % 8) == 0 && (which != B200_GEMM_WGRAD_TN || (K % 64) == 0);
    uintptr_t bits = 0;
    for (int i = 0; i < count; ++i) {
        if (Ns[i] <= 0 || !ys[i] || !(k_concat ? xs[i] : xs[0]) || !(k_concat ? outs[0] : outs[i])) return B200_E_BADARG;
        n_total += Ns[i];
        if ((Ns[i] % 64) != 0) fast = false;
        int a = n_align, b = Ns[i];
        while (b) { const int t = a % b; a = b; b = t; }
        n_align = a;   // gcd
        bits |= reinterpret_cast<uintptr_t>(ys[i]) | reinterpret_cast<uintptr_t>(k_concat ? xs[i] : xs[0]) |
                reinterpret_cast<uintptr_t>(k_concat ? outs[0] : outs[i]);
    }
    if ((bits & 15) != 0 || n_total > 0x7FFFFFFF) fast = false;
    if (!fast) {
        for (int i = 0; i < count; ++i) {
            const int rc = k_concat ? gemm_bf16(ctx, which, (beta1 || i > 0) ? 1 : 0, outs[0], xs[i], ys[i], M, Ns[i], K, 0, sm_limit)
                                    : gemm_bf16(ctx, which, beta1, outs[i], xs[0], ys[i], M, Ns[i], K, (overlap_prev && i == 0) ? 1 : 0,
                                                sm_limit);
            if (rc) return rc;
        }
        return B200_OK;
    }
    int Mo, No, Kc;
    bool p_mn, q_mn;
    const int Nt = static_cast<int>(n_total);
    if (which == B200_GEMM_FWD_NN) { Mo = M; No = Nt; Kc = K; p_mn = false; q_mn = true; }
    else if (which == B200_GEMM_DGRAD_NT) { Mo = M; No = K; Kc = Nt; p_mn = false; q_mn = false; }
    else { Mo = K; No = Nt; Kc = M; p_mn = true; q_mn = true; }
    const int sm_count = (sm_limit > 0 && sm_limit < ctx->sm_count) ? sm_limit : ctx->sm_count;
    b200_linear_plan_t plan;
    memset(&plan, 0, sizeof(plan));
    plan_dims(Mo, No, Kc, sm_count, k_concat ? 0 : n_align, &plan);
    if (plan.bn == 0) return B200_E_BADARG;
    GemmParams gp;
    int bn, ctas, grid;
    // a forced tile shape (tests, tuning) is taken when no tile of that width would straddle two products
    const bool honour_force = ctx->force_bn > 0 && (k_concat || (n_align % ctx->force_bn) == 0);
    int rc = schedule_launch(ctx, plan, Mo, No, Kc, sm_count, overlap_prev, honour_force, gp, bn, ctas, grid);
    if (rc) return rc;
    gp.out = outs[0];
    gp.p_3d = p_mn ? 1 : 0;   // Mo % 64 == 0 and every Ns[i] % 64 == 0 were checked above
    gp.q_3d = q_mn ? 1 : 0;
    int acc = 0;
    for (int i = 0; i + 1 < count; ++i) {
        acc += Ns[i];
        if (k_concat) gp.grp_k[i] = acc / BK;
        else gp.grp_n[i] = acc / bn;
    }
    const bool need32 = gp.ksplit > 1 || gp.sk_peer;
    CUtensorMap tmP[3], tmQ[3], tmD[3], tmD32[3];
    for (int i = 0; i < count; ++i) {
        const int Ni = Ns[i];
        // P: shared by the column-concatenated products (only product 0's map is read), one per range of the contraction
        if (k_concat || i == 0) {
            const void* P = k_concat ? xs[i] : xs[0];
            if (p_mn) rc = get_panel_map(ctx, P, Mo, Kc, BM / 64, &tmP[i]);
            else rc = get_tensor_map(ctx, P, k_concat ? Ni : Kc, Mo, BK, BM, &tmP[i]);
            if (rc) return rc;
        } else {
            tmP[i] = tmP[0];
        }
        if (q_mn) rc = get_panel_map(ctx, ys[i], Ni, Kc, bn / ctas / 64, &tmQ[i]);
        else rc = get_tensor_map(ctx, ys[i], Ni, No, BK, bn / ctas, &tmQ[i]);   // K-concatenated: [K][Ni], contraction contiguous
        if (rc) return rc;
        if (!k_concat || i == 0) {
            void* D = k_concat ? outs[0] : outs[i];
            const int cols = k_concat ? No : Ni;
            rc = get_tensor_map(ctx, D, cols, Mo, 64, 32, &tmD[i]);
            if (rc) return rc;
            tmD32[i] = tmD[i];
            if (need32) {
                rc = get_tensor_map(ctx, D, cols, Mo, 32, 32, &tmD32[i]);
                if (rc) return rc;
            }
        } else {
            tmD[i] = tmD[0];
            tmD32[i] = tmD32[0];
        }
    }
    GemmGroupMaps gx = {};
    for (int i = 1; i < count; ++i) {
        gx.p[i - 1] = tmP[i];
        gx.q[i - 1] = tmQ[i];
        gx.d[i - 1] = tmD[i];
        gx.d32[i - 1] = tmD32[i];
    }
    if (p_mn) return launch_beta<true, true, 3>(ctx, gx, bn, ctas, beta1, tmP[0], tmQ[0], tmD[0], tmD32[0], gp, grid);
    if (q_mn) return launch_beta<false, true, 3>(ctx, gx, bn, ctas, beta1, tmP[0], tmQ[0], tmD[0], tmD32[0], gp, grid);
    return launch_beta<false, false, 3>(ctx, gx, bn, ctas, beta1, tmP[0], tmQ[0], tmD[0], tmD32[0], gp, grid);
}

// gate = X W_gate, up = X W_up and hidden = SiLU(gate) * up in one launch: 256-wide pair tiles whose left half is 128
// columns of gate and whose right half is the same 128 columns of up, hidden formed in the epilogue from the rounded
// values.  B200_E_BADARG for shapes this kernel does not take (ff % 128, K % 8, alignment, fewer than two SMs): the
// caller then issues the products and the element-wise kernel separately.
int gemm_swiglu_fwd(b200_linear_ctx* ctx, void* gate, void* up, void* hidden, const void* x, const void* w_gate,
                    const void* w_up, int M, int ff, int K) {
    if (!ctx || !gate || !up || !hidden || !x || !w_gate || !w_up || M <= 0 || ff <= 0 || K <= 0) return B200_E_BADARG;
    if (!on_context_device(ctx)) return B200_E_BADARG;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(hidden) |
                           reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_gate) | reinterpret_cast<uintptr_t>(w_up);
    if ((bits & 15) != 0 || (ff % 128) != 0 || (K % 8) != 0 || ctx->sm_count < 2 || ff > 0x3FFFFFFF) return B200_E_BADARG;
    constexpr int bn = 256, ctas = 2;
    // the schedule of an M x 2 ff product in whole 256 x 256 pair tiles, round-robin over the CTA pairs
    const int max_slots = ctx->sm_count / ctas;
    const Decomp d = decompose(M, 2 * ff, K, bn, ctas, max_slots, 1);
    const int slots = d.dp_tiles < max_slots ? d.dp_tiles : max_slots;
    GemmParams gp;
    gp.Mo = M; gp.No = 2 * ff; gp.Kc = K;
    gp.m_tiles = d.m_tiles; gp.n_tiles = d.n_tiles; gp.kb_total = d.kb_total;
    gp.m_fastest = M <= 2 * ff ? 1 : 0;
    gp.group = 0;
    gp.dp_tiles = d.dp_tiles; gp.sk_splits = 1; gp.kb_per_sk = d.kb_total; gp.sk_items = 0;
    gp.sk_peer = 0; gp.late_wait = 0; gp.ksplit = 1;
    gp.p_3d = 0; gp.q_3d = 1;
    gp.grp_n[0] = gp.grp_n[1] = gp.grp_k[0] = gp.grp_k[1] = GRP_NONE;
    gp.out = gate; gp.ws = nullptr; gp.sk_counters = nullptr; gp.status = ctx->status_dev;
    const int grid = slots * ctas;
    int rc;
    CUtensorMap tmP, tmQg, tmQu, tmG, tmU, tmH;
    rc = get_tensor_map(ctx, x, K, M, BK, BM, &tmP);
    if (rc) return rc;
    rc = get_panel_map(ctx, w_gate, ff, K, bn / ctas / 64, &tmQg);
    if (rc) return rc;
    rc = get_panel_map(ctx, w_up, ff, K, bn / ctas / 64, &tmQu);
    if (rc) return rc;
    rc = get_tensor_map(ctx, gate, ff, M, 64, 32, &tmG);
    if (rc) return rc;
    rc = get_tensor_map(ctx, up, ff, M, 64, 32, &tmU);
    if (rc) return rc;
    rc = get_tensor_map(ctx, hidden, ff, M, 64, 32, &tmH);
    if (rc) return rc;
    GemmGroupMaps gx = {};
    gx.q[0] = tmQu;
    gx.d[0] = tmU;
    gx.d[1] = tmH;
    using Cfg = TileCfg<bn, ctas>;
    static bool configured[kMaxDevices] = {};
    auto kern = gemm_bf16_sm100<bn, false, true, false, ctas, 1>;
    if (!configured[ctx->device]) {
        CU_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        configured[ctx->device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = ctx->use_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    CU_TRY(ctx, cudaLaunchKernelEx(&cfg, kern, tmP, tmQg, tmG, tmG, gx, gp));
    ctx->launches++;
    return B200_OK;
}

// The LM-head forward of a (vocabulary shard of a) model together with the cross-entropy statistics of its rows:
// logits[M, N] = x[M, K] w[K, N] stored as bf16, and per row the maximum, sum exp(l - max) and the target's logit of
// those N columns (global columns col0 .. col0 + N) -- what b200_ce_shard_stats_bf16 computes in a pass of its own over
// the stored logits.  The GEMM's epilogue forms (max, sum) per row and tile from the rounded values while they are in
// registers (gemm_sm100.cuh, EPI = 2); ce_merge_partials merges a row's pairs.  Operands may be pitched.
int forward_ce_stats(b200_linear_ctx* ctx, void* logits, long long ld_out, const void* x, long long ld_x, const void* w,
                     long long ld_w, int M, int N, int K, const int* targets, int col0, float* row_max, float* row_sum,
                     float* row_target) {
    if (!ctx || !logits || !x || !w || !targets || !row_max || !row_sum || !row_target || M <= 0 || N <= 0 || K <= 0 || col0 < 0)
        return B200_E_BADARG;
    if (!on_context_device(ctx)) return B200_E_BADARG;
    if (ld_out == 0) ld_out = N;
    if (ld_x == 0) ld_x = K;
    if (ld_w == 0) ld_w = N;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w);
    if ((bits & 15) != 0 || (N % 8) != 0 || (K % 8) != 0 || ((ld_out | ld_x | ld_w) % 8) != 0 || ld_out < N || ld_x < K || ld_w < N ||
        ctx->sm_count < 2)
        return B200_E_BADARG;
    constexpr int bn = 256, ctas = 2;
    const int max_slots = ctx->sm_count / ctas;
    const Decomp d = decompose(M, N, K, bn, ctas, max_slots, 1);
    const int slots = d.dp_tiles < max_slots ? d.dp_tiles : max_slots;
    const int np = 2 * d.n_tiles;
    int rc = ensure_workspace(ctx, static_cast<size_t>(M) * np * sizeof(float2), 0);
    if (rc) return rc;
    GemmParams gp;
    gp.Mo = M; gp.No = N; gp.Kc = K;
    gp.m_tiles = d.m_tiles; gp.n_tiles = d.n_tiles; gp.kb_total = d.kb_total;
    gp.m_fastest = M <= N ? 1 : 0;
    gp.group = 0;
    gp.dp_tiles = d.dp_tiles; gp.sk_splits = 1; gp.kb_per_sk = d.kb_total; gp.sk_items = 0;
    gp.sk_peer = 0; gp.late_wait = 0; gp.ksplit = 1;
    gp.p_3d = 0; gp.q_3d = (N % 64) == 0 ? 1 : 0;
    gp.grp_n[0] = gp.grp_n[1] = gp.grp_k[0] = gp.grp_k[1] = GRP_NONE;
    gp.out = logits; gp.ws = ctx->ws; gp.sk_counters = nullptr; gp.status = ctx->status_dev;
    CUtensorMap tmP, tmQ, tmD;
    rc = get_tensor_map(ctx, x, K, M, BK, BM, &tmP, ld_x == K ? 0 : ld_x);
    if (rc) return rc;
    if (gp.q_3d) rc = get_panel_map(ctx, w, N, K, bn / ctas / 64, &tmQ, ld_w == N ? 0 : ld_w);
    else rc = get_tensor_map(ctx, w, N, K, 64, BK, &tmQ, ld_w == N ? 0 : ld_w);
    if (rc) return rc;
    rc = get_tensor_map(ctx, logits, N, M, 64, 32, &tmD, ld_out == N ? 0 : ld_out);
    if (rc) return rc;
    using Cfg = TileCfg<bn, ctas>;
    static bool configured[kMaxDevices] = {};
    auto kern = gemm_bf16_sm100<bn, false, true, false, ctas, 2>;
    if (!configured[ctx->device]) {
        CU_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        configured[ctx->device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(slots * ctas, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = ctx->use_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    CU_TRY(ctx, cudaLaunchKernelEx(&cfg, kern, tmP, tmQ, tmD, tmD, g_no_group, gp));
    ctx->launches++;
    const int rows_per_cta = b200::CE_THREADS / 32;
    const int want = (M + rows_per_cta - 1) / rows_per_cta;
    const int grid = want < ctx->sm_count * 8 ? want : ctx->sm_count * 8;
    b200::ce_merge_partials<<<grid, b200::CE_THREADS, 0, ctx->stream>>>(reinterpret_cast<const float2*>(ctx->ws), np,
                                                                      static_cast<const __nv_bfloat16*>(logits), M, N, ld_out, targets,
                                                                      col0, row_max, row_sum, row_target);
    CU_TRY(ctx, cudaGetLastError());
    ctx->launches++;
    return B200_OK;
}

template <typename T, bool P_MN, bool Q_MN>
int launch_simt_layout(b200_linear_ctx* ctx, const SimtParams& sp, bool vec) {
    dim3 grid(ceil_div_i(sp.No, ST_BN), ceil_div_i(sp.Mo, ST_BM), sp.splits);
    if (grid.y > 65535u) return B200_E_TOOBIG;
    if constexpr (sizeof(T) == 4) {
        if (vec) gemm_simt<T, P_MN, Q_MN, true><<<grid, ST_THREADS, 0, ctx->stream>>>(sp);
        else     gemm_simt<T, P_MN, Q_MN, false><<<grid, ST_THREADS, 0, ctx->stream>>>(sp);
    } else {
        gemm_simt<T, P_MN, Q_MN, false><<<grid, ST_THREADS, 0, ctx->stream>>>(sp);
    }
    CU_TRY(ctx, cudaGetLastError());
    ctx->launches++;
    return B200_OK;
}

template <typename T>
int launch_simt(b200_linear_ctx* ctx, int which, int beta1, T* out, const T* x, const T* y, int M, int N,
                int K) {
    if (!ctx || !out || !x || !y || M <= 0 || N <= 0 || K <= 0 || which < 0 || which > 2)
        return B200_E_BADARG;
    SimtParams sp;
    if (which == B200_GEMM_FWD_NN) { sp.Mo = M; sp.No = N; sp.Kc = K; }
    else if (which == B200_GEMM_DGRAD_NT) { sp.Mo = M; sp.No = K; sp.Kc = N; }
    else { sp.Mo = K; sp.No = N; sp.Kc = M; }
    sp.P = x; sp.Q = y;
    // Split the contraction when the output alone cannot fill the GPU.
    const long long tiles = 1LL * ceil_div_i(sp.Mo, ST_BM) * ceil_div_i(sp.No, ST_BN);
    int splits = 1;
    if (tiles < ctx->sm_count) {
        splits = static_cast<int>((2LL * ctx->sm_count + tiles - 1) / tiles);
        const int max_splits = sp.Kc / 256 > 0 ? sp.Kc / 256 : 1;
        if (splits > max_splits) splits = max_splits;
        if (splits > 64) splits = 64;
    }
    int per = ceil_div_i(ceil_div_i(sp.Kc, splits), ST_BK) * ST_BK;
    splits = ceil_div_i(sp.Kc, per);
    sp.splits = splits;
    sp.kc_per_split = per;
    sp.beta1 = beta1;
    if (splits > 1) {
        int rc = ensure_workspace(ctx, static_cast<size_t>(splits) * sp.Mo * sp.No * sizeof(float));
        if (rc) return rc;
        sp.out = ctx->ws;
    } else {
        sp.out = out;
    }
    const bool vec = sizeof(T) == 4 && (N % 4) == 0 && (K % 4) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    int rc;
    if (which == B200_GEMM_FWD_NN) rc = launch_simt_layout<T, false, true>(ctx, sp, vec);
    else if (which == B200_GEMM_DGRAD_NT) rc = launch_simt_layout<T, false, false>(ctx, sp, vec);
    else rc = launch_simt_layout<T, true, true>(ctx, sp, vec);
    if (rc) return rc;
    if (splits > 1) {
        const long long n = 1LL * sp.Mo * sp.No;
        long long blocks = (n + 255) / 256;
        if (blocks > 8LL * ctx->sm_count) blocks = 8LL * ctx->sm_count;
        splitk_reduce_generic<T><<<static_cast<int>(blocks), 256, 0, ctx->stream>>>(out, ctx->ws, n, splits, beta1);
        CU_TRY(ctx, cudaGetLastError());
        ctx->launches++;
    }
    return B200_OK;
}

}  // namespace

namespace {

template <int BN, bool P_MN, bool Q_MN, bool BETA1>
int launch_tf32x3(b200_linear_ctx* ctx, const CUtensorMap& tmP, const CUtensorMap& tmQ, const CUtensorMap& tmD,
                  const GemmParams& gp, int grid) {
    using Cfg = T32Cfg<BN>;
    static bool configured[kMaxDevices] = {};
    auto kern = gemm_tf32x3_sm100<BN, P_MN, Q_MN, BETA1>;
    if (!configured[ctx->device]) {
        CU_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        configured[ctx->device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(T32_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->use_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CU_TRY(ctx, cudaLaunchKernelEx(&cfg, kern, tmP, tmQ, tmD, gp));
    ctx->launches++;
    return B200_OK;
}

template <bool P_MN, bool Q_MN>
int launch_tf32x3_variants(b200_linear_ctx* ctx, int bn, int beta1, const CUtensorMap& tmP, const CUtensorMap& tmQ,
                           const CUtensorMap& tmD, const GemmParams& gp, int grid) {
    if (bn == 128)
        return beta1 ? launch_tf32x3<128, P_MN, Q_MN, true>(ctx, tmP, tmQ, tmD, gp, grid)
                     : launch_tf32x3<128, P_MN, Q_MN, false>(ctx, tmP, tmQ, tmD, gp, grid);
    return beta1 ? launch_tf32x3<64, P_MN, Q_MN, true>(ctx, tmP, tmQ, tmD, gp, grid)
                 : launch_tf32x3<64, P_MN, Q_MN, false>(ctx, tmP, tmQ, tmD, gp, grid);
}

// One fp32 product: on the tensor cores (3xTF32, fp32-grade accuracy) when TMA can describe the
// operands, else on the CUDA cores.
int gemm_f32(b200_linear_ctx* ctx, int which, int beta1, float* out, const float* x, const float* y, int M, int N,
             int K) {
    if (!ctx || !out || !x || !y || M <= 0 || N <= 0 || K <= 0 || which < 0 || which > 2) return B200_E_BADARG;
    if (!on_context_device(ctx)) return B200_E_BADARG;
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x) |
                             reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    if (ctx->fp32_simt || !aligned16 || (N % 4) != 0 || (K % 4) != 0)
        return launch_simt<float>(ctx, which, beta1, out, x, y, M, N, K);
    int Mo, No, Kc;
    bool p_mn, q_mn;
    if (which == B200_GEMM_FWD_NN) { Mo = M; No = N; Kc = K; p_mn = false; q_mn = true; }
    else if (which == B200_GEMM_DGRAD_NT) { Mo = M; No = K; Kc = N; p_mn = false; q_mn = false; }
    else { Mo = K; No = N; Kc = M; p_mn = true; q_mn = true; }
    // 128-wide tiles unless they would leave more than half of the SMs without a tile (this kernel does not split
    // the contraction): 64-wide tiles then put twice as many SMs to work.
    const long long tiles128 = 1LL * ceil_div_i(Mo, BM) * ceil_div_i(No, 128);
    const int bn = (No > 64 && tiles128 * 2 > ctx->sm_count) ? 128 : 64;
    GemmParams gp = {};
    gp.Mo = Mo; gp.No = No; gp.Kc = Kc;
    gp.m_tiles = ceil_div_i(Mo, BM);
    gp.n_tiles = ceil_div_i(No, bn);
    gp.kb_total = ceil_div_i(Kc, T32_BK);
    gp.m_fastest = Mo <= No ? 1 : 0;
    gp.group = 0;
    const long long tiles = 1LL * gp.m_tiles * gp.n_tiles;
    if (tiles > 0x7FFFFFFFLL) return B200_E_TOOBIG;
    gp.dp_tiles = static_cast<int>(tiles);
    gp.sk_splits = 1; gp.kb_per_sk = gp.kb_total; gp.sk_items = 0; gp.sk_peer = 0; gp.ksplit = 1; gp.late_wait = 0;
    gp.out = out;
    gp.status = ctx->status_dev;
    gp.p_3d = p_mn && (Mo % 32) == 0;
    gp.q_3d = q_mn && (No % 32) == 0;
    CUtensorMap tmP, tmQ, tmD;
    int rc;
    if (gp.p_3d) rc = get_panel_map_f32(ctx, x, Mo, Kc, BM / 32, &tmP);
    else if (p_mn) rc = get_tensor_map_f32(ctx, x, Mo, Kc, T32_BK, &tmP, true);
    else rc = get_tensor_map_f32(ctx, x, Kc, Mo, BM, &tmP);
    if (rc) return rc;
    if (gp.q_3d) rc = get_panel_map_f32(ctx, y, No, Kc, bn / 32, &tmQ);
    else if (q_mn) rc = get_tensor_map_f32(ctx, y, No, Kc, T32_BK, &tmQ, true);
    else rc = get_tensor_map_f32(ctx, y, Kc, No, bn, &tmQ);
    if (rc) return rc;
    rc = get_tensor_map_f32(ctx, out, No, Mo, 32, &tmD);
    if (rc) return rc;
    const int grid = tiles < ctx->sm_count ? static_cast<int>(tiles) : ctx->sm_count;
    if (p_mn) return launch_tf32x3_variants<true, true>(ctx, bn, beta1, tmP, tmQ, tmD, gp, grid);
    if (q_mn) return launch_tf32x3_variants<false, true>(ctx, bn, beta1, tmP, tmQ, tmD, gp, grid);
    return launch_tf32x3_variants<false, false>(ctx, bn, beta1, tmP, tmQ, tmD, gp, grid);
}

}  // namespace

// ------------------------------------------------------------ C entry points
extern "C" int b200_linear_create(b200_linear_ctx** out) {
    if (!out) return B200_E_BADARG;
    *out = nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_E_NODEVICE;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return B200_E_NODEVICE;
    if (prop.major != 10) return B200_E_NODEVICE;  // tcgen05 / TMEM exist on sm_100 only
    b200_linear_ctx* ctx = new b200_linear_ctx();
    ctx->device = dev;
    ctx->sm_count = prop.multiProcessorCount;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
        delete ctx;
        return B200_E_CUDA;
    }
    ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
    if (const char* e = getenv("B200_LINEAR_PDL")) ctx->use_pdl = atoi(e) != 0;
    if (const char* e = getenv("B200_LINEAR_PEER_SPLIT")) ctx->no_peer_split = atoi(e) == 0;
    if (const char* e = getenv("B200_LINEAR_OVERLAP_BACKWARD")) ctx->overlap_backward = atoi(e) != 0;
    if (const char* e = getenv("B200_LINEAR_PARTITION_BACKWARD")) ctx->partition_backward = atoi(e) != 0;
    if (const char* e = getenv("B200_LINEAR_TILE_GROUP")) ctx->tile_group = atoi(e);
    if (const char* e = getenv("B200_LINEAR_FP32_SIMT")) ctx->fp32_simt = atoi(e) != 0;
    if (cudaMalloc(&ctx->status_dev, sizeof(int)) != cudaSuccess ||
        cudaMemset(ctx->status_dev, 0, sizeof(int)) != cudaSuccess) {
        delete ctx;
        return B200_E_CUDA;
    }
    ctx->ws_bytes = 64ull << 20;
    if (cudaMalloc(&ctx->ws, ctx->ws_bytes) != cudaSuccess) {
        cudaFree(ctx->status_dev);
        delete ctx;
        return B200_E_CUDA;
    }
    *out = ctx;
    return B200_OK;
}

extern "C" int b200_linear_destroy(b200_linear_ctx* ctx) {
    if (!ctx) return B200_E_BADARG;
    cudaStreamSynchronize(ctx->stream);
    cudaFree(ctx->ws);
    cudaFree(ctx->status_dev);
    if (ctx->sk_counters) cudaFree(ctx->sk_counters);
    if (ctx->ws2) cudaFree(ctx->ws2);
    if (ctx->sk_counters2) cudaFree(ctx->sk_counters2);
    delete ctx;
    return B200_OK;
}

extern "C" int b200_linear_set_stream(b200_linear_ctx* ctx, void* cuda_stream) {
    if (!ctx) return B200_E_BADARG;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    return B200_OK;
}

extern "C" int b200_linear_sync(b200_linear_ctx* ctx, int* device_code) {
    if (!ctx) return B200_E_BADARG;
    CU_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    int code = 0;
    CU_TRY(ctx, cudaMemcpy(&code, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
    if (device_code) *device_code = code;
    if (code != 0) {
        CU_TRY(ctx, cudaMemset(ctx->status_dev, 0, sizeof(int)));
        if (ctx->sk_counters) CU_TRY(ctx, cudaMemset(ctx->sk_counters, 0, ctx->sk_counters_len * sizeof(int)));
        if (ctx->sk_counters2) CU_TRY(ctx, cudaMemset(ctx->sk_counters2, 0, ctx->sk_counters2_len * sizeof(int)));
        return B200_E_DEVICE_WAIT;
    }
    return B200_OK;
}

namespace b200 {
// One warp waits on a barrier phase that nothing will ever complete, with a short limit: the wait gives
// up, records `code` in the status word and the kernel returns.  This is the whole life of a bounded wait
// that runs out, made to happen on purpose so that the host side of it (status read-back, clean-up, the
// next launches on the same context) can be tested without any kernel misbehaving.
__global__ void wait_timeout_probe(int* status, long long limit_cycles, int code) {
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    mbar_wait(smem_u32(&bar), 0, &abort_flag, status, code, limit_cycles);
}
}  // namespace b200

extern "C" int b200_linear_selftest_wait_timeout(b200_linear_ctx* ctx, long long limit_cycles) {
    if (!ctx || limit_cycles <= 0 || limit_cycles > WAIT_LIMIT_CYCLES) return B200_E_BADARG;
    if (!on_context_device(ctx)) return B200_E_BADARG;
    wait_timeout_probe<<<1, 32, 0, ctx->stream>>>(ctx->status_dev, limit_cycles, DEV_TIMEOUT_FULL);
    CU_TRY(ctx, cudaGetLastError());
    ctx->launches++;
    return B200_OK;
}

extern "C" int* b200_linear_status_word(b200_linear_ctx* ctx) { return ctx ? ctx->status_dev : nullptr; }

extern "C" long long b200_linear_launch_count(const b200_linear_ctx* ctx) { return ctx ? ctx->launches : -1; }
extern "C" int b200_linear_last_cuda_error(const b200_linear_ctx* ctx) { return ctx ? ctx->last_cuda : -1; }

extern "C" const char* b200_linear_strerror(int code) {
    switch (code) {
        case B200_OK: return "ok";
        case B200_E_BADARG: return "bad argument";
        case B200_E_CUDA: return "CUDA call failed";
        case B200_E_NODEVICE: return "no sm_100 device current";
        case B200_E_DEVICE_WAIT: return "a kernel gave up on a bounded wait";
        case B200_E_TOOBIG: return "size beyond limit";
        default: return "unknown error";
    }
}

extern "C" int b200_linear_force_backward_split(b200_linear_ctx* ctx, int sm_dgrad) {
    if (!ctx || sm_dgrad < 0 || sm_dgrad >= ctx->sm_count) return B200_E_BADARG;
    ctx->force_sm_dgrad = sm_dgrad;
    return B200_OK;
}

extern "C" int b200_linear_force_plan(b200_linear_ctx* ctx, int bn, int cta_pair, int splits) {
    if (!ctx) return B200_E_BADARG;
    if (bn > 0 && bn != 64 && bn != 128 && bn != 192 && bn != 256) return B200_E_BADARG;
    if (bn > 0 && cta_pair && bn != 128 && bn != 256) return B200_E_BADARG;
    if (bn > 0 && splits < 0 && (-splits * (cta_pair ? 2 : 1) > 8 || -splits > bn / 32)) return B200_E_BADARG;
    ctx->force_bn = bn;
    ctx->force_pair = cta_pair;
    ctx->force_splits = splits;
    return B200_OK;
}

extern "C" int b200_linear_gemm_bf16(b200_linear_ctx* ctx, int which, int beta1, void* out, const void* x,
                                     const void* y, int M, int N, int K) {
    return gemm_bf16(ctx, which, beta1 ? 1 : 0, out, x, y, M, N, K);
}
extern "C" int b200_linear_gemm_bf16_ld(b200_linear_ctx* ctx, int which, int beta1, void* out, long long ld_out,
                                        const void* x, long long ld_x, const void* y, long long ld_y, int M, int N,
                                        int K) {
    if (ld_out < 0 || ld_x < 0 || ld_y < 0) return B200_E_BADARG;
    return gemm_bf16(ctx, which, beta1 ? 1 : 0, out, x, y, M, N, K, 0, 0, ld_out, ld_x, ld_y);
}
// The plan of a grouped launch (pure host arithmetic, like b200_linear_plan_bf16): plan->bn == 0 when the shapes do
// not suit the one-launch path and the products would run one by one.
extern "C" int b200_linear_plan_grouped_bf16(int which, int count, int M, const int* Ns, int K, int sm_count,
                                             b200_linear_plan_t* plan) {
    if (!plan || !Ns || count < 1 || count > 3 || M <= 0 || K <= 0 || sm_count <= 0 || which < 0 || which > 2) return B200_E_BADARG;
    memset(plan, 0, sizeof(*plan));
    long long n_total = 0;
    int n_align = 0;
    bool fast = count > 1 && (K % 8) == 0 && (which != B200_GEMM_WGRAD_TN || (K % 64) == 0);
    for (int i = 0; i < count; ++i) {
        if (Ns[i] <= 0) return B200_E_BADARG;
        n_total += Ns[i];
        if ((Ns[i] % 64) != 0) fast = false;
        int a = n_align, b = Ns[i];
        while (b) { const int t = a % b; a = b; b = t; }
        n_align = a;
    }
    if (n_total > 0x7FFFFFFF) return B200_E_BADARG;
    if (!fast) return B200_OK;   // bn = 0: single products
    const int Nt = static_cast<int>(n_total);
    if (which == B200_GEMM_FWD_NN) plan_dims(M, Nt, K, sm_count, n_align, plan);
    else if (which == B200_GEMM_DGRAD_NT) plan_dims(M, K, Nt, sm_count, 0, plan);
    else plan_dims(K, Nt, M, sm_count, n_align, plan);
    return B200_OK;
}
extern "C" int b200_linear_gemm_bf16_grouped(b200_linear_ctx* ctx, int which, int beta1, int count, void* const* outs,
                                             const void* const* xs, const void* const* ys, int M, const int* Ns, int K) {
    return gemm_bf16_grouped(ctx, which, beta1, count, outs, xs, ys, M, Ns, K);
}
extern "C" int b200_linear_forward_ce_stats_bf16(b200_linear_ctx* ctx, void* logits, long long ld_out, const void* x,
                                                 long long ld_x, const void* w, long long ld_w, int M, int N, int K,
                                                 const int* targets, int col0, float* row_max, float* row_sum,
                                                 float* row_target) {
    return forward_ce_stats(ctx, logits, ld_out, x, ld_x, w, ld_w, M, N, K, targets, col0, row_max, row_sum, row_target);
}
extern "C" int b200_linear_swiglu_forward_bf16(b200_linear_ctx* ctx, void* gate, void* up, void* hidden, const void* x,
                                               const void* w_gate, const void* w_up, int M, int ff, int K) {
    return gemm_swiglu_fwd(ctx, gate, up, hidden, x, w_gate, w_up, M, ff, K);
}
extern "C" int b200_linear_backward_bf16_grouped(b200_linear_ctx* ctx, int count, void* dA, int beta1_dA, void* const* dBs,
                                                 const void* const* dCs, const void* A, const void* const* Bs, int M,
                                                 const int* Ns, int K) {
    if (!ctx || (!dA && !dBs) || !dCs || !Ns || count < 1 || count > 3 || M <= 0 || K <= 0) return B200_E_BADARG;
    long long n_total = 0;
    for (int i = 0; i < count; ++i) n_total += Ns[i] > 0 ? Ns[i] : 0;
    if (n_total <= 0 || n_total > 0x7FFFFFFF) return B200_E_BADARG;
    // as in b200_linear_backward_bf16: the two launches side by side on complementary shares of the SMs
    int sm_dgrad = 0, sm_wgrad = 0;
    if (dA && dBs && ctx->use_pdl && ctx->overlap_backward && ctx->partition_backward && ctx->force_bn <= 0 && ctx->sm_count >= 16)
        split_sms_for_backward(ctx, M, static_cast<int>(n_total), K, &sm_dgrad, &sm_wgrad);
    if (dA) {
        if (!Bs) return B200_E_BADARG;
        void* const outs[3] = {dA, dA, dA};
        const int rc = gemm_bf16_grouped(ctx, B200_GEMM_DGRAD_NT, beta1_dA, count, outs, dCs, Bs, M, Ns, K, 0, sm_dgrad);
        if (rc) return rc;
    }
    if (dBs) {
        if (!A) return B200_E_BADARG;
        const void* const xs[3] = {A, A, A};
        return gemm_bf16_grouped(ctx, B200_GEMM_WGRAD_TN, 1, count, dBs, xs, dCs, M, Ns, K, dA ? 1 : 0, sm_wgrad);
    }
    return B200_OK;
}
extern "C" int b200_linear_gemm_f32(b200_linear_ctx* ctx, int which, int beta1, float* out, const float* x,
                                    const float* y, int M, int N, int K) {
    return gemm_f32(ctx, which, beta1 ? 1 : 0, out, x, y, M, N, K);
}

extern "C" int b200_linear_forward_bf16(b200_linear_ctx* ctx, void* C, const void* A, const void* B, int M,
                                        int N, int K) {
    return gemm_bf16(ctx, B200_GEMM_FWD_NN, 0, C, A, B, M, N, K);
}
extern "C" int b200_linear_backward_bf16(b200_linear_ctx* ctx, void* dA, void* dB, const void* dC,
                                         const void* A, const void* B, int M, int N, int K) {
    if (!ctx || (!dA && !dB)) return B200_E_BADARG;
    // dB does not depend on dA.  The two kernels therefore run side by side, each planned for its own
    // share of the SMs (the split that the cost model says finishes soonest), unless running them one
    // after the other on the whole GPU is estimated to be faster.  The second kernel starts as soon as
    // the first one's CTAs are all resident and waits for the first only before it exits.
    int sm_dgrad = 0, sm_wgrad = 0;
    if (dA && dB && M > 0 && N > 0 && K > 0 && ctx->use_pdl && ctx->overlap_backward && ctx->partition_backward && ctx->force_bn <= 0 &&
        ctx->sm_count >= 16)
        split_sms_for_backward(ctx, M, N, K, &sm_dgrad, &sm_wgrad);
    if (dA) {
        int rc = gemm_bf16(ctx, B200_GEMM_DGRAD_NT, 0, dA, dC, B, M, N, K, 0, sm_dgrad);
        if (rc) return rc;
    }
    if (dB) return gemm_bf16(ctx, B200_GEMM_WGRAD_TN, 1, dB, A, dC, M, N, K, dA ? 1 : 0, sm_wgrad);
    return B200_OK;
}
extern "C" int b200_linear_forward_f32(b200_linear_ctx* ctx, float* C, const float* A, const float* B, int M,
                                       int N, int K) {
    return gemm_f32(ctx, B200_GEMM_FWD_NN, 0, C, A, B, M, N, K);
}
extern "C" int b200_linear_backward_f32(b200_linear_ctx* ctx, float* dA, float* dB, const float* dC,
                                        const float* A, const float* B, int M, int N, int K) {
    if (!dA && !dB) return B200_E_BADARG;
    if (dA) {
        int rc = gemm_f32(ctx, B200_GEMM_DGRAD_NT, 0, dA, dC, B, M, N, K);
        if (rc) return rc;
    }
    if (dB) return gemm_f32(ctx, B200_GEMM_WGRAD_TN, 1, dB, A, dC, M, N, K);
    return B200_OK;
}

// ------------------------------------------------- weight gradient without any allocation
// For hosts that must not see this library allocate device memory: a trainer that has handed
// the whole GPU to an arena of its own at start-up (a later cudaMalloc simply fails there), or a
// step loop that cannot afford the device-wide synchronisation that cudaMalloc / cudaFree imply
// when the context's workspace has to grow for a shape it has not seen yet.  The split-K
// scratch (fp32 partial tiles, arrival counters, status word) lives in the fixed array below,
// which every GPU that loads this library carries until the process exits.
namespace {

constexpr int NA_BN = 128;                 // tile width used by this entry point (single-CTA tiles)
constexpr int NA_MAX_ITEMS = 128;          // partial tiles that fit the array
constexpr int NA_COUNTERS = 256;
struct NoAllocScratch {
    float partials[static_cast<size_t>(NA_MAX_ITEMS) * BM * NA_BN];  // 8 MiB
    int counters[NA_COUNTERS];
    int status;  // sticky: only b200_linear_noalloc_status clears it
};

struct NoAllocDevice {
    bool ready = false;
    NoAllocScratch* scratch = nullptr;  // device address of g_noalloc_scratch on that device
    int sm_count = 0;
    EncodeTiledFn encode = nullptr;
};
NoAllocDevice g_noalloc_dev[kMaxDevices];
std::mutex g_noalloc_mutex;  // guards the once-per-device set-up below

}  // namespace

// In host code this name is only a handle for cudaGetSymbolAddress; kernels get the address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

// dB[K,N] = bf16_rn(bf16_rn(A[M,K]^T * dC[M,N]) + dB)   -- the beta = 1 product of matmul_backward.
extern "C" int b200_linear_wgrad_bf16_noalloc(void* dB, const void* A, const void* dC, int M, int N, int K,
                                              void* cuda_stream) {
    if (!dB || !A || !dC || M <= 0 || N <= 0 || K <= 0) return B200_E_BADARG;
    if ((N % 8) != 0 || (K % 8) != 0 ||
        ((reinterpret_cast<uintptr_t>(dB) | reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(dC)) & 15) != 0)
        return B200_E_BADARG;  // no CUDA-core fallback here: TMA needs 16-byte pitches and pointers
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_E_NODEVICE;
    NoAllocDevice& nd = g_noalloc_dev[dev];
    using Cfg = TileCfg<NA_BN, 1>;
    auto kern = gemm_bf16_sm100<NA_BN, true, true, true, 1>;
    std::unique_lock<std::mutex> setup_lock(g_noalloc_mutex);
    if (!nd.ready) {  // once per device, with that device current
        int major = 0, sms = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
            return B200_E_NODEVICE;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            return B200_E_CUDA;
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || !fn)
            return B200_E_CUDA;
        void* base = nullptr;
        if (cudaGetSymbolAddress(&base, g_noalloc_scratch) != cudaSuccess || !base) return B200_E_CUDA;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
            return B200_E_CUDA;
        nd.scratch = static_cast<NoAllocScratch*>(base);
        nd.sm_count = sms;
        nd.encode = reinterpret_cast<EncodeTiledFn>(fn);
        nd.ready = true;
    }
    setup_lock.unlock();
    const int Mo = K, No = N, Kc = M;  // output rows/cols, contraction over the tokens
    const int tiles = ceil_div_i(Mo, BM) * ceil_div_i(No, NA_BN);
    if (tiles > NA_MAX_ITEMS || tiles > NA_COUNTERS) return B200_E_TOOBIG;
    int splits = NA_MAX_ITEMS / tiles;
    if (splits > nd.sm_count / tiles) splits = nd.sm_count / tiles;
    const int kb_total = ceil_div_i(Kc, BK);
    if (splits > kb_total / 4) splits = kb_total / 4;
    if (splits < 1) splits = 1;
    const Decomp d = decompose(Mo, No, Kc, NA_BN, 1, nd.sm_count, splits);
    if (d.sk_items > NA_MAX_ITEMS) return B200_E_TOOBIG;
    const int items = d.dp_tiles + d.sk_items;
    const int grid = items < nd.sm_count ? items : nd.sm_count;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    GemmParams gp;
    gp.Mo = Mo; gp.No = No; gp.Kc = Kc;
    gp.m_tiles = d.m_tiles; gp.n_tiles = d.n_tiles; gp.kb_total = d.kb_total;
    gp.m_fastest = Mo <= No ? 1 : 0;
    gp.group = 0;
    gp.dp_tiles = d.dp_tiles; gp.sk_splits = d.sk_splits; gp.kb_per_sk = d.kb_per_sk; gp.sk_items = d.sk_items;
    gp.ksplit = 1;
    gp.late_wait = 0;
    gp.sk_peer = 0;
    gp.p_3d = (Mo % 64) == 0;
    gp.q_3d = (No % 64) == 0;
    gp.out = dB;
    gp.ws = nd.scratch->partials;
    gp.sk_counters = nd.scratch->counters;
    gp.grp_n[0] = gp.grp_n[1] = gp.grp_k[0] = gp.grp_k[1] = GRP_NONE;
    gp.status = &nd.scratch->status;

    auto encode = [&](CUtensorMap* tm, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                      const cuuint32_t* box) {
        const cuuint32_t estr[3] = {1, 1, 1};
        return nd.encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    auto mn_major_map = [&](CUtensorMap* tm, const void* ptr, int rows, bool as3d, int panels) {
        if (as3d) {
            const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(Kc), static_cast<cuuint64_t>(rows / 64)};
            const cuuint64_t strides[2] = {static_cast<cuuint64_t>(rows) * 2, 128};
            const cuuint32_t box[3] = {64, BK, static_cast<cuuint32_t>(panels)};
            return encode(tm, ptr, 3, dims, strides, box);
        }
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(Kc)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(rows) * 2};
        const cuuint32_t box[2] = {64, BK};
        return encode(tm, ptr, 2, dims, strides, box);
    };
    CUtensorMap tmP, tmQ, tmD;
    if (!mn_major_map(&tmP, A, Mo, gp.p_3d != 0, BM / 64)) return B200_E_CUDA;
    if (!mn_major_map(&tmQ, dC, No, gp.q_3d != 0, NA_BN / 64)) return B200_E_CUDA;
    {
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(No), static_cast<cuuint64_t>(Mo)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(No) * 2};
        const cuuint32_t box[2] = {64, 32};
        if (!encode(&tmD, dB, 2, dims, strides, box)) return B200_E_CUDA;
    }
    // The array keeps whatever the previous call left: the arrival counters must start at zero.  The status
    // word is left alone, so that a wait that ran out in an earlier call stays visible until it is read.
    if (cudaMemsetAsync(nd.scratch->counters, 0, sizeof(int) * NA_COUNTERS, stream) != cudaSuccess)
        return B200_E_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, tmP, tmQ, tmD, tmD, g_no_group, gp) != cudaSuccess) return B200_E_CUDA;
    return B200_OK;
}

// Waits for `cuda_stream`, then reads (and clears) the status word that the kernels of
// b200_linear_wgrad_bf16_noalloc write when one of their bounded waits runs out.  Allocates nothing: the
// word lives in the fixed scratch array and is copied straight into *device_code.
extern "C" int b200_linear_noalloc_status(int* device_code, void* cuda_stream) {
    if (device_code) *device_code = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_E_NODEVICE;
    NoAllocScratch* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (g_noalloc_dev[dev].ready) scratch = g_noalloc_dev[dev].scratch;
    }
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(cuda_stream)) != cudaSuccess) return B200_E_CUDA;
    if (!scratch) return B200_OK;  // the entry point has not run on this device yet: nothing to report
    int code = 0;
    if (cudaMemcpy(&code, &scratch->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return B200_E_CUDA;
    if (device_code) *device_code = code;
    if (code == 0) return B200_OK;
    if (cudaMemset(&scratch->status, 0, sizeof(int)) != cudaSuccess) return B200_E_CUDA;
    return B200_E_DEVICE_WAIT;
}

// ---------------------------------------------------------------- vocabulary-sharded cross-entropy
namespace {
int ce_launch_status() { return cudaGetLastError() == cudaSuccess ? B200_OK : B200_E_CUDA; }
int ce_sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}
}  // namespace

extern "C" int b200_ce_shard_stats_bf16(const void* logits, int rows, int cols, long long ld, const int* targets,
                                        int col0, float* row_max, float* row_sum, float* row_target,
                                        void* cuda_stream) {
    if (!targets || !row_max || !row_sum || !row_target || rows <= 0 || cols < 0 || ld < cols || col0 < 0 ||
        (cols > 0 && !logits))
        return B200_E_BADARG;
    const int sms = ce_sm_count();
    if (sms <= 0) return B200_E_NODEVICE;
    const int ctas = (rows + b200::CE_THREADS / 32 - 1) / (b200::CE_THREADS / 32);  // one warp per row
    const int grid = ctas < sms * 8 ? ctas : sms * 8;  // 8 CTAs of 256 threads fill an SM
    b200::ce_shard_stats_bf16<<<grid, b200::CE_THREADS, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), rows, cols, ld, targets, col0, row_max, row_sum, row_target);
    return ce_launch_status();
}

extern "C" int b200_ce_shard_rescale(const float* local_max, const float* global_max, float* row_sum, int rows,
                                     void* cuda_stream) {
    if (!local_max || !global_max || !row_sum || rows <= 0) return B200_E_BADARG;
    b200::ce_shard_rescale<<<(rows + 255) / 256, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        local_max, global_max, row_sum, rows);
    return ce_launch_status();
}

extern "C" int b200_ce_shard_loss(float* loss, const float* global_max, const float* global_sum,
                                  const float* target_logit, int rows, void* cuda_stream) {
    if (!loss || !global_max || !global_sum || !target_logit || rows <= 0) return B200_E_BADARG;
    b200::ce_shard_loss<<<(rows + 255) / 256, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        loss, global_max, global_sum, target_logit, rows);
    return ce_launch_status();
}

extern "C" int b200_ce_shard_backward_bf16(void* dlogits, const void* logits, int rows, int cols, long long ld,
                                           const int* targets, int col0, const float* global_max,
                                           const float* global_sum, float scale, void* cuda_stream) {
    if (!targets || !global_max || !global_sum || rows <= 0 || cols < 0 || ld < cols || col0 < 0 ||
        (cols > 0 && (!logits || !dlogits)))
        return B200_E_BADARG;
    if (cols == 0) return B200_OK;
    const int per_cta = 8 * b200::CE_THREADS;
    dim3 grid((cols + per_cta - 1) / per_cta, rows < 4096 ? rows : 4096, 1);
    b200::ce_shard_backward_bf16<<<grid, b200::CE_THREADS, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<__nv_bfloat16*>(dlogits), static_cast<const __nv_bfloat16*>(logits), rows, cols, ld, targets, col0,
        global_max, global_sum, scale);
    return ce_launch_status();
}
