// Multi-GPU training driver around the reference's own training objects (one process per GPU, NCCL).
//
// The reference trains on one GPU (llama2-mistral/src/main.cpp:140-210): per optimizer step it runs
// `accum` micro-batches through ModelBF16::forward / backward (whose linear layers are this library's
// GEMMs once the binary is linked against libb200_linear.so), then takes the gradient norm, clips and
// updates.  This driver shards that work along the two seams the linear-layer path offers:
//
//  * by tokens (always): every per-layer GEMM is independent along the token dimension, so micro-batch g
//    of a step goes to rank g % R.  What has to be exchanged is the gradient sum, once per step:
//    grads.storage past the embedding rows (bf16) and dwte_fp32 (fp32), all-reduce SUM -- a sum, not a
//    mean: the reference never divides by the number of micro-batches (cuda/crossentropy.cu:155 scales by
//    1/BT only).  Every rank then runs the identical norm / clip / AdamW update on identical gradients.
//
//  * by vocabulary (--vocab-parallel): the LM head w_out[C, V] is split by columns in whole 256-column
//    tiles; rank r owns columns [col0_r, col0_r + V_r) and multiplies by them where they lie (row pitch V,
//    b200_linear_gemm_bf16_ld).  The R micro-batches that run at the same time form a round: the ranks
//    gather their final hidden states [R*BT, C], every rank computes the logits of all R*BT tokens for its
//    columns (b200_linear_forward_ce_stats_bf16: the rows' maximum and sum of exponentials come out of that GEMM's
//    epilogue), these are combined with two small all-reduces (b200_ce_shard_* kernels), dlogits is formed in place, the weight gradient lands in the
//    rank's own columns of dw_out, and the input gradient [R*BT, C] is reduce-scattered back so that every
//    rank continues the backward pass of its own micro-batch.  No rank ever holds a whole row of logits.
//    This replaces llama2-mistral/src/model.cpp:612-614 (LM-head GEMM, crossentropy_forward) and :634-635
//    (crossentropy_softmax_backward, LM-head matmul_backward); the model code on either side of those lines
//    (model.cpp:591-611 and :636-680) is called exactly as ModelBF16::forward / backward call it.
//
// Compiled together with the reference's unmodified model.cpp, dataloader.cpp and kernel sources, taken
// from the reference checkout at build time (oracle/build.py); it includes the reference's headers and
// copies nothing from them.  The step logic follows main.cpp:149-196 call for call, the checkpoint file is
// the reference's (main.cpp:212-254 writes it, :93-112 and model.cpp:564-580 read it).
//
// Usage: train_dp <tokens.bin> --ranks R [--steps S] [--batch B] [--seq T] [--accum A] [--warmup W] [--lr LR]
//                 [--vocab-parallel] [--save-every N] [--checkpoint path] [--start-step N] [--timers]
//   A = micro-batches per optimizer step over all ranks (a multiple of R).  The processes are forked before
//   any CUDA call; the NCCL id travels from rank 0 over pipes.  Before every group of collectives the ranks
//   meet on the host (rank_rendezvous.h): a rank that failed stops the others there, between steps, instead
//   of leaving them inside a collective.
#include <nccl.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "../../include/b200_linear.h"
#include "dataloader.h"
#include "kernels.cuh"
#include "model.h"
#include "rank_rendezvous.h"

namespace {

// llama2-mistral/src/main.cpp:9-21: linear warm-up, then cosine decay to min_lr.
float lr_at(int step, float peak_lr, float min_lr, int warmup_steps, int max_steps) {
    if (step < warmup_steps) return peak_lr * (static_cast<float>(step) / static_cast<float>(warmup_steps));
    float progress = static_cast<float>(step - warmup_steps) / static_cast<float>(max_steps - warmup_steps);
    if (progress > 1.0f) progress = 1.0f;
    return min_lr + (peak_lr - min_lr) * 0.5f * (1.0f + cosf(3.14159265f * progress));
}

struct Options {
    const char* data = nullptr;
    const char* checkpoint = nullptr;
    int ranks = 1, steps = 3, batch = 16, seq = 0, accum = 16, warmup = 2000, save_every = 0, start_step = 0;
    float lr = 3e-4f;
    bool vocab_parallel = false, timers = false;
    double rendezvous_timeout_s = 600.0;
};

b200::RendezvousPage* g_page = nullptr;
int g_rank = 0;

// Any error ends this rank; the stop flag tells the others before they start another collective.
[[noreturn]] void die(const char* what, const char* detail, const char* file, int line) {
    fprintf(stderr, "rank %d: %s error %s:%d: %s\n", g_rank, what, file, line, detail);
    if (g_page) b200::rendezvous_fail(g_page, g_rank);
    _exit(EXIT_FAILURE);
}
#define NCCL_TRY(call)                                                              \
    do {                                                                            \
        ncclResult_t r_ = (call);                                                   \
        if (r_ != ncclSuccess) die("NCCL", ncclGetErrorString(r_), __FILE__, __LINE__); \
    } while (0)
#define CUDA_TRY(call)                                                              \
    do {                                                                            \
        cudaError_t e_ = (call);                                                    \
        if (e_ != cudaSuccess) die("CUDA", cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)
#define B200_TRY(call)                                                              \
    do {                                                                            \
        int rc_ = (call);                                                           \
        if (rc_ != B200_OK) die("b200_linear", b200_linear_strerror(rc_), __FILE__, __LINE__); \
    } while (0)

// Meet the other ranks on the host before enqueueing collectives.  False: somebody failed, leave.
bool meet(const Options& opt) {
    if (opt.ranks == 1) return true;
    const b200::RendezvousResult r = b200::rendezvous_arrive(g_page, g_rank, opt.rendezvous_timeout_s);
    if (r == b200::RV_OK) return true;
    fprintf(stderr, "rank %d: leaving before the next collective (%s, rank %d)\n", g_rank,
            r == b200::RV_TIMEOUT ? "a rank did not arrive in time" : "a rank failed", g_page->failed_rank.load());
    return false;
}

struct PhaseTimers {
    bool on = false;
    double t_last = 0, zero = 0, loader = 0, micro = 0, lm_head = 0, exchange = 0, norm = 0, update = 0;
    void start() { if (on) { cudaDeviceSynchronize(); t_last = b200::rendezvous_now(); } }
    void lap(double& acc) {
        if (!on) return;
        cudaDeviceSynchronize();
        const double t = b200::rendezvous_now();
        acc += t - t_last;
        t_last = t;
    }
};

// Vocabulary shard of rank r: whole 256-column tiles, as even as the tile count allows.
void vocab_shard(int V, int ranks, int r, int* col0, int* cols) {
    const int tile = 256, tiles = (V + tile - 1) / tile;
    const int base = tiles / ranks, extra = tiles % ranks;
    const int t0 = r * base + (r < extra ? r : extra), n = base + (r < extra ? 1 : 0);
    *col0 = t0 * tile < V ? t0 * tile : V;
    const int end = (t0 + n) * tile < V ? (t0 + n) * tile : V;
    *cols = end - *col0;
}

// ModelBF16::forward up to the final RMSNorm (llama2-mistral/src/model.cpp:591-611), on the model's own
// buffers, with the same calls in the same order.
void forward_trunk(ModelBF16& m, const int* input_ids, int B, int T) {
    const ModelConfig& c = m.config;
    const int C = c.n_embd, BT = B * T;
    embedding_forward(m.x, m.wte, input_ids, B, T, C);
    for (int l = 0; l < c.n_layer; ++l) {
        CUDA_TRY(cudaMemcpy(m.x_ckpt + static_cast<size_t>(l) * BT * C, m.x, static_cast<size_t>(BT) * C * sizeof(__nv_bfloat16),
                            cudaMemcpyDeviceToDevice));
        rmsnorm_forward(m.ln1_out, m.rrms1, m.x, m.rms1_w[l], c.norm_eps, BT, C);
        attention_forward(m.attn_out, m.q, m.k, m.v, m.att, m.ln1_out, m.wq[l], m.wk[l], m.wv[l], m.wo[l], B, T, C,
                          c.n_head, c.n_kv_head, c.rope_theta, m.cublas_handle);
        residual_forward(m.x, m.x, m.attn_out, BT * C);
        rmsnorm_forward(m.ln2_out, m.rrms2, m.x, m.rms2_w[l], c.norm_eps, BT, C);
        swiglu_forward(m.mlp_out, m.gate_buf, m.up_buf, m.hidden_buf, m.ln2_out, m.w_gate[l], m.w_up[l], m.w_down[l],
                       BT, C, c.ffn_hidden, m.cublas_handle);
        residual_forward(m.x, m.x, m.mlp_out, BT * C);
    }
    rmsnorm_forward(m.ln_final, m.rrms_final, m.x, m.rmsf_w, c.norm_eps, BT, C);
}

// ModelBF16::backward from the final RMSNorm down (llama2-mistral/src/model.cpp:636-680); m.dln_final holds
// the gradient of the final hidden state.
void backward_trunk(ModelBF16& m, int B, int T) {
    const ModelConfig& c = m.config;
    const int C = c.n_embd, BT = B * T, ff = c.ffn_hidden;
    const size_t act_bytes = static_cast<size_t>(BT) * C * sizeof(__nv_bfloat16);
    rmsnorm_backward(m.dx, m.drmsf_w, m.dln_final, m.x, m.rmsf_w, m.rrms_final, BT, C);
    for (int l = c.n_layer - 1; l >= 0; --l) {
        __nv_bfloat16* x_in = m.x_ckpt + static_cast<size_t>(l) * BT * C;
        rmsnorm_forward(m.ln1_out, m.rrms1, x_in, m.rms1_w[l], c.norm_eps, BT, C);
        attention_forward(m.attn_out, m.q, m.k, m.v, m.att, m.ln1_out, m.wq[l], m.wk[l], m.wv[l], m.wo[l], B, T, C,
                          c.n_head, c.n_kv_head, c.rope_theta, m.cublas_handle);
        residual_forward(m.x_mid, x_in, m.attn_out, BT * C);
        rmsnorm_forward(m.ln2_out, m.rrms2, m.x_mid, m.rms2_w[l], c.norm_eps, BT, C);
        swiglu_forward(m.mlp_out, m.gate_buf, m.up_buf, m.hidden_buf, m.ln2_out, m.w_gate[l], m.w_up[l], m.w_down[l],
                       BT, C, ff, m.cublas_handle);
        CUDA_TRY(cudaMemcpy(m.dx_tmp, m.dx, act_bytes, cudaMemcpyDeviceToDevice));
        CUDA_TRY(cudaMemset(m.dmlp_out, 0, act_bytes));
        residual_backward(m.dx, m.dmlp_out, m.dx_tmp, BT * C);
        swiglu_backward(m.dln2_out, m.dw_gate[l], m.dw_up[l], m.dw_down[l], m.dmlp_out, m.ln2_out, m.gate_buf, m.up_buf,
                        m.w_gate[l], m.w_up[l], m.w_down[l], BT, C, ff, m.cublas_handle);
        rmsnorm_backward(m.dx_tmp, m.drms2_w[l], m.dln2_out, m.x_mid, m.rms2_w[l], m.rrms2, BT, C);
        residual_forward(m.dx, m.dx, m.dx_tmp, BT * C);
        CUDA_TRY(cudaMemcpy(m.dx_tmp, m.dx, act_bytes, cudaMemcpyDeviceToDevice));
        CUDA_TRY(cudaMemset(m.dattn_out, 0, act_bytes));
        residual_backward(m.dx, m.dattn_out, m.dx_tmp, BT * C);
        attention_backward(m.dln1_out, m.dwq[l], m.dwk[l], m.dwv[l], m.dwo[l], m.dattn_out, m.ln1_out, m.q, m.k, m.v, m.att,
                           m.wq[l], m.wk[l], m.wv[l], m.wo[l], B, T, C, c.n_head, c.n_kv_head, c.rope_theta,
                           m.cublas_handle);
        rmsnorm_backward(m.dx_tmp, m.drms1_w[l], m.dln1_out, x_in, m.rms1_w[l], m.rrms1, BT, C);
        residual_forward(m.dx, m.dx, m.dx_tmp, BT * C);
    }
}

// Scratch of the vocabulary-parallel LM head: the gathered hidden states and targets of one round, the
// per-row statistics and the un-scattered input gradient.  The logits live in the model's own logits /
// probs buffers (contiguous, 2 * BT * V elements: room for [R*BT, V_r] whatever the tile rounding).
struct VocabParallel {
    int col0 = 0, cols = 0, rows = 0;
    b200_linear_ctx* ctx = nullptr;
    __nv_bfloat16* x_all = nullptr;     // [R*BT, C]
    __nv_bfloat16* dx_all = nullptr;    // [R*BT, C]
    int* targets_all = nullptr;         // [R*BT]
    float* stats = nullptr;             // local max | global max | sum | target logit | loss: 5 x [R*BT]
    float* loss_host = nullptr;
};

void vp_setup(VocabParallel& vp, ModelBF16& m, const Options& opt, int BT) {
    vocab_shard(m.config.vocab_size, opt.ranks, g_rank, &vp.col0, &vp.cols);
    vp.rows = opt.ranks * BT;
    if (static_cast<long long>(vp.rows) * vp.cols > 2LL * BT * m.config.vocab_size)
        die("driver", "logits of one round do not fit the model's logits + probs buffers", __FILE__, __LINE__);
    const int C = m.config.n_embd;
    B200_TRY(b200_linear_create(&vp.ctx));
    CUDA_TRY(cudaMalloc(&vp.x_all, static_cast<size_t>(vp.rows) * C * sizeof(__nv_bfloat16)));
    CUDA_TRY(cudaMalloc(&vp.dx_all, static_cast<size_t>(vp.rows) * C * sizeof(__nv_bfloat16)));
    CUDA_TRY(cudaMalloc(&vp.targets_all, static_cast<size_t>(vp.rows) * sizeof(int)));
    CUDA_TRY(cudaMalloc(&vp.stats, 5 * static_cast<size_t>(vp.rows) * sizeof(float)));
    vp.loss_host = static_cast<float*>(malloc(static_cast<size_t>(vp.rows) * sizeof(float)));
}

// One round of the sharded LM head + cross-entropy, forward and backward.  On return m.dln_final holds the
// gradient of this rank's own final hidden state and *round_loss the mean loss over the round's R micro-batches.
bool vp_lm_head_round(VocabParallel& vp, ModelBF16& m, const int* targets, const Options& opt, ncclComm_t comm, int B,
                      int T, float* round_loss) {
    const int C = m.config.n_embd, V = m.config.vocab_size, BT = B * T, R = opt.ranks, rows = vp.rows;
    float *lmax = vp.stats, *gmax = vp.stats + rows, *sum = vp.stats + 2 * rows, *tgt = vp.stats + 3 * rows,
          *loss = vp.stats + 4 * rows;
    __nv_bfloat16* logits = m.logits;  // [rows, cols], dense
    if (!meet(opt)) return false;
    if (R > 1) {
        NCCL_TRY(ncclGroupStart());
        NCCL_TRY(ncclAllGather(m.ln_final, vp.x_all, static_cast<size_t>(BT) * C, ncclBfloat16, comm, 0));
        NCCL_TRY(ncclAllGather(targets, vp.targets_all, static_cast<size_t>(BT), ncclInt32, comm, 0));
        NCCL_TRY(ncclGroupEnd());
    } else {
        CUDA_TRY(cudaMemcpy(vp.x_all, m.ln_final, static_cast<size_t>(BT) * C * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice));
        CUDA_TRY(cudaMemcpy(vp.targets_all, targets, static_cast<size_t>(BT) * sizeof(int), cudaMemcpyDeviceToDevice));
    }
    // logits_r = x_all * w_out[:, col0 : col0 + cols]
    // with the rows' maxima, sums of exponentials and target logits formed in the GEMM's epilogue; where the operands
    // do not suit that kernel: the plain product, then a pass over the stored logits
    const int fused_rc = b200_linear_forward_ce_stats_bf16(vp.ctx, logits, vp.cols, vp.x_all, C, m.w_out + vp.col0, V, rows, vp.cols,
                                                           C, vp.targets_all, vp.col0, lmax, sum, tgt);
    if (fused_rc == B200_E_BADARG) {
        B200_TRY(b200_linear_gemm_bf16_ld(vp.ctx, B200_GEMM_FWD_NN, 0, logits, vp.cols, vp.x_all, C, m.w_out + vp.col0, V, rows,
                                          vp.cols, C));
        B200_TRY(b200_ce_shard_stats_bf16(logits, rows, vp.cols, vp.cols, vp.targets_all, vp.col0, lmax, sum, tgt, nullptr));
    } else {
        B200_TRY(fused_rc);
    }
    CUDA_TRY(cudaMemcpyAsync(gmax, lmax, static_cast<size_t>(rows) * sizeof(float), cudaMemcpyDeviceToDevice, 0));
    if (R > 1) NCCL_TRY(ncclAllReduce(gmax, gmax, static_cast<size_t>(rows), ncclFloat, ncclMax, comm, 0));
    B200_TRY(b200_ce_shard_rescale(lmax, gmax, sum, rows, nullptr));
    if (R > 1) NCCL_TRY(ncclAllReduce(sum, sum, 2 * static_cast<size_t>(rows), ncclFloat, ncclSum, comm, 0));  // sum | target logit
    B200_TRY(b200_ce_shard_loss(loss, gmax, sum, tgt, rows, nullptr));
    // dlogits in place; the reference scales by loss_scale / BT of one micro-batch (cuda/crossentropy.cu:155)
    B200_TRY(b200_ce_shard_backward_bf16(logits, logits, rows, vp.cols, vp.cols, vp.targets_all, vp.col0, gmax, sum,
                                         m.loss_scale / static_cast<float>(BT), nullptr));
    // dx_all (partial) = dlogits_r * w_r^T ;  dw_out[:, shard] += x_all^T * dlogits_r
    B200_TRY(b200_linear_gemm_bf16_ld(vp.ctx, B200_GEMM_DGRAD_NT, 0, vp.dx_all, C, logits, vp.cols, m.w_out + vp.col0, V,
                                      rows, vp.cols, C));
    B200_TRY(b200_linear_gemm_bf16_ld(vp.ctx, B200_GEMM_WGRAD_TN, 1, m.dw_out + vp.col0, V, vp.x_all, C, logits, vp.cols,
                                      rows, vp.cols, C));
    if (R > 1) {
        NCCL_TRY(ncclReduceScatter(vp.dx_all, m.dln_final, static_cast<size_t>(BT) * C, ncclBfloat16, ncclSum, comm, 0));
    } else {
        CUDA_TRY(cudaMemcpyAsync(m.dln_final, vp.dx_all, static_cast<size_t>(BT) * C * sizeof(__nv_bfloat16),
                                 cudaMemcpyDeviceToDevice, 0));
    }
    CUDA_TRY(cudaMemcpy(vp.loss_host, loss, static_cast<size_t>(rows) * sizeof(float), cudaMemcpyDeviceToHost));
    int code = 0;
    if (b200_linear_sync(vp.ctx, &code) != B200_OK) die("b200_linear", "a kernel gave up on a bounded wait", __FILE__, __LINE__);
    // per micro-batch mean first (fp32, row order), as ModelBF16::forward does (model.cpp:618-621), then over the round
    float total = 0.0f;
    for (int r = 0; r < R; ++r) {
        float s = 0.0f;
        for (int i = 0; i < BT; ++i) s += vp.loss_host[static_cast<size_t>(r) * BT + i];
        total += s / static_cast<float>(BT);
    }
    *round_loss = total / static_cast<float>(R);
    return true;
}

// The reference's checkpoint file (llama2-mistral/src/main.cpp:212-254): n fp32 master weights, the magic
// 0x4F50544D, the step, n fp32 first moments, n fp32 second moments.
void save_checkpoint(ModelBF16& m, int global_step) {
    mkdir("checkpoints", 0777);
    char path[256];
    snprintf(path, sizeof(path), "checkpoints/step_%d.bin", global_step);
    const size_t n = m.master_params.numel;
    std::vector<float> host(n);
    FILE* f = fopen(path, "wb");
    if (!f) {
        printf("Warning: could not write checkpoint %s\n", path);
        return;
    }
    CUDA_TRY(cudaMemcpy(host.data(), m.master_params.data, n * sizeof(float), cudaMemcpyDeviceToHost));
    fwrite(host.data(), sizeof(float), n, f);
    const int magic = 0x4F50544D;
    fwrite(&magic, sizeof(int), 1, f);
    fwrite(&global_step, sizeof(int), 1, f);
    CUDA_TRY(cudaMemcpy(host.data(), m.adam_m.data, n * sizeof(float), cudaMemcpyDeviceToHost));
    fwrite(host.data(), sizeof(float), n, f);
    CUDA_TRY(cudaMemcpy(host.data(), m.adam_v.data, n * sizeof(float), cudaMemcpyDeviceToHost));
    fwrite(host.data(), sizeof(float), n, f);
    fclose(f);
    printf("Saved checkpoint: %s\n", path);
}

// Weights through the reference's own ModelBF16::load; optimizer state as main.cpp:93-112 restores it.
// Returns the step stored in the file (0 for a weights-only file).
int load_checkpoint(ModelBF16& m, const char* path) {
    m.load(path);
    const size_t n = m.master_params.numel;
    FILE* f = fopen(path, "rb");
    if (!f) return 0;
    int saved_step = 0, magic = 0;
    fseek(f, static_cast<long>(n * sizeof(float)), SEEK_SET);
    if (fread(&magic, sizeof(int), 1, f) == 1 && magic == 0x4F50544D && fread(&saved_step, sizeof(int), 1, f) == 1) {
        std::vector<float> host(n);
        if (fread(host.data(), sizeof(float), n, f) == n)
            CUDA_TRY(cudaMemcpy(m.adam_m.data, host.data(), n * sizeof(float), cudaMemcpyHostToDevice));
        if (fread(host.data(), sizeof(float), n, f) == n)
            CUDA_TRY(cudaMemcpy(m.adam_v.data, host.data(), n * sizeof(float), cudaMemcpyHostToDevice));
    } else {
        saved_step = 0;
    }
    fclose(f);
    return saved_step;
}

int run_rank(int rank, const Options& opt, int id_read_fd, const std::vector<int>& id_write_fds) {
    g_rank = rank;
    CUDA_TRY(cudaSetDevice(rank));
    ncclComm_t comm = nullptr;
    if (opt.ranks > 1) {
        ncclUniqueId id;
        if (rank == 0) {
            NCCL_TRY(ncclGetUniqueId(&id));
            for (int fd : id_write_fds)
                if (write(fd, &id, sizeof(id)) != static_cast<ssize_t>(sizeof(id))) die("driver", "pipe write", __FILE__, __LINE__);
        } else if (read(id_read_fd, &id, sizeof(id)) != static_cast<ssize_t>(sizeof(id))) {
            die("driver", "pipe read", __FILE__, __LINE__);
        }
        NCCL_TRY(ncclCommInitRank(&comm, opt.ranks, id, rank));
    }

    ModelConfig model_cfg;
    TrainConfig train_cfg;
    train_cfg.learning_rate = opt.lr;
    train_cfg.max_steps = opt.steps;
    train_cfg.warmup_steps = opt.warmup;
    const int B = opt.batch, T = opt.seq > 0 ? opt.seq : train_cfg.seq_len, accum = opt.accum, BT = B * T;
    ModelBF16 model;  // every rank builds the same weights: the reference seeds its own generator
    model.build(model_cfg, B, T);
    int start_step = opt.start_step;
    if (opt.checkpoint) {
        const int saved = load_checkpoint(model, opt.checkpoint);
        if (start_step == 0) start_step = saved;
        if (rank == 0 && saved > 0) printf("Restored optimizer state from step %d\n", saved);
    }
    DataLoader loader;
    loader.open(opt.data, B, T);
    float* loss_dev = nullptr;
    CUDA_TRY(cudaMalloc(&loss_dev, sizeof(float)));
    VocabParallel vp;
    if (opt.vocab_parallel) vp_setup(vp, model, opt, BT);

    const int N = static_cast<int>(model.params.storage.numel);
    const int emb_N = model.config.vocab_size * model.config.n_embd;
    const long long tokens_per_step = 1LL * BT * accum;
    if (rank == 0) {
        printf("%d GPU(s): %d micro-batches of %d x %d tokens per step (%lld tokens), %d per rank, by tokens%s\n", opt.ranks,
               accum, B, T, tokens_per_step, accum / opt.ranks,
               opt.vocab_parallel ? "; LM head + cross-entropy sharded by vocabulary" : "");
        if (opt.vocab_parallel) printf("rank 0 owns LM-head columns [%d, %d) of %d\n", vp.col0, vp.col0 + vp.cols, model.config.vocab_size);
    }

    PhaseTimers tm;
    tm.on = opt.timers;
    auto t_start = std::chrono::steady_clock::now();
    for (int step = 1; step <= opt.steps; ++step) {
        const int global_step = step + start_step;
        if (step == 2) {  // the first step carries set-up costs (allocations, NCCL connections): time from the second
            CUDA_TRY(cudaDeviceSynchronize());
            t_start = std::chrono::steady_clock::now();
            tm = PhaseTimers();
            tm.on = opt.timers;
        }
        const float lr = lr_at(global_step, train_cfg.learning_rate, train_cfg.min_lr, train_cfg.warmup_steps,
                               train_cfg.max_steps + start_step);
        tm.start();
        model.zero_grad();
        tm.lap(tm.zero);
        float local_loss = 0.0f;
        for (int micro = 0; micro < accum; ++micro) {
            if (micro % opt.ranks != rank) {
                // another rank's micro-batch: only the stream position moves (dataloader.cpp:33-50 without the copies)
                if (loader.pos + static_cast<size_t>(BT) + 1 > loader.n_tokens) loader.reset();
                loader.pos += BT;
                continue;
            }
            if (!loader.next_batch()) {
                loader.reset();
                loader.next_batch();
            }
            tm.lap(tm.loader);
            if (!opt.vocab_parallel) {
                model.forward(loader.input_ids_gpu, loader.targets_gpu, B, T);
                model.backward(B, T);
                local_loss += model.loss;
                tm.lap(tm.micro);
            } else {
                forward_trunk(model, loader.input_ids_gpu, B, T);
                tm.lap(tm.micro);
                float round_loss = 0.0f;
                if (!vp_lm_head_round(vp, model, loader.targets_gpu, opt, comm, B, T, &round_loss)) return 3;
                local_loss += round_loss;  // every rank holds the same value: the mean over the round
                tm.lap(tm.lm_head);
                backward_trunk(model, B, T);
            }
            embedding_backward(model.dwte_fp32, model.dx, loader.input_ids_gpu, B, T, model.config.n_embd);
            tm.lap(tm.micro);
        }
        // one exchange per optimizer step, on the stream the reference's kernels use (the legacy default stream)
        if (opt.ranks > 1) {
            if (!meet(opt)) return 3;
            NCCL_TRY(ncclGroupStart());
            NCCL_TRY(ncclAllReduce(model.grads.storage.data + emb_N, model.grads.storage.data + emb_N,
                                   static_cast<size_t>(N - emb_N), ncclBfloat16, ncclSum, comm, 0));
            NCCL_TRY(ncclAllReduce(model.dwte_fp32, model.dwte_fp32, static_cast<size_t>(emb_N), ncclFloat, ncclSum, comm, 0));
            NCCL_TRY(ncclGroupEnd());
            if (!opt.vocab_parallel) {  // sum of the ranks' loss sums; in the sharded mode every rank already has the mean per round
                CUDA_TRY(cudaMemcpy(loss_dev, &local_loss, sizeof(float), cudaMemcpyHostToDevice));
                NCCL_TRY(ncclAllReduce(loss_dev, loss_dev, 1, ncclFloat, ncclSum, comm, 0));
                CUDA_TRY(cudaMemcpy(&local_loss, loss_dev, sizeof(float), cudaMemcpyDeviceToHost));
            }
        }
        tm.lap(tm.exchange);
        const float loss = opt.vocab_parallel ? local_loss / (accum / opt.ranks) : local_loss / accum;
        const float global_norm = compute_grad_norm_bf16(model.dwte_fp32, emb_N, model.grads.storage.data + emb_N,
                                                         N - emb_N, model.loss_scale);
        tm.lap(tm.norm);
        const float clip_scale = global_norm > train_cfg.grad_clip ? train_cfg.grad_clip / global_norm : 1.0f;
        model.update(lr, train_cfg, global_step, clip_scale);
        CUDA_TRY(cudaDeviceSynchronize());
        tm.lap(tm.update);
        if (rank == 0) {
            const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count();
            if (step >= 2)
                printf("step %5d | loss %.8f | lr %.2e | norm %.4f | %.0f tok/s (wall clock, steps 2..%d)\n", global_step, loss,
                       lr, global_norm, (step - 1) * tokens_per_step / secs, step);
            else
                printf("step %5d | loss %.8f | lr %.2e | norm %.4f\n", global_step, loss, lr, global_norm);
            fflush(stdout);
            if (opt.save_every > 0 && step % opt.save_every == 0) save_checkpoint(model, global_step);
        }
    }
    if (rank == 0 && opt.timers && opt.steps >= 2) {
        const double n = opt.steps - 1;
        printf("phases, seconds per step over steps 2..%d (rank 0, device synchronised after each): zero_grad %.4f | loader %.4f | "
               "micro-batches %.4f | sharded LM head %.4f | gradient exchange %.4f | gradient norm %.4f | update %.4f\n",
               opt.steps, tm.zero / n, tm.loader / n, tm.micro / n, tm.lm_head / n, tm.exchange / n, tm.norm / n, tm.update / n);
        fflush(stdout);
    }
    CUDA_TRY(cudaFree(loss_dev));
    if (comm) {
        if (!meet(opt)) return 3;
        NCCL_TRY(ncclCommDestroy(comm));
    }
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    Options opt;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--ranks") && i + 1 < argc) opt.ranks = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--steps") && i + 1 < argc) opt.steps = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--batch") && i + 1 < argc) opt.batch = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--seq") && i + 1 < argc) opt.seq = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--accum") && i + 1 < argc) opt.accum = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) opt.warmup = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--lr") && i + 1 < argc) opt.lr = static_cast<float>(atof(argv[++i]));
        else if (!strcmp(argv[i], "--save-every") && i + 1 < argc) opt.save_every = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--checkpoint") && i + 1 < argc) opt.checkpoint = argv[++i];
        else if (!strcmp(argv[i], "--start-step") && i + 1 < argc) opt.start_step = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--vocab-parallel")) opt.vocab_parallel = true;
        else if (!strcmp(argv[i], "--timers")) opt.timers = true;
        else if (argv[i][0] != '-') opt.data = argv[i];
    }
    if (!opt.data || opt.ranks < 1 || opt.ranks > 8 || opt.accum < 1 || opt.accum % opt.ranks != 0 || opt.steps < 1) {
        fprintf(stderr,
                "usage: %s <tokens.bin> --ranks R [--steps S] [--batch B] [--seq T] [--accum A (multiple of R)] [--warmup W] "
                "[--lr LR] [--vocab-parallel] [--save-every N] [--checkpoint path] [--start-step N] [--timers]\n",
                argv[0]);
        return 2;
    }
    // A rank that dies with its memory bound to an NVLink multicast object can disturb the other GPUs of the
    // box; the collectives here are small next to a step, so they run without in-switch reduction.
    setenv("NCCL_NVLS_ENABLE", "0", 0);
    g_page = b200::rendezvous_create(opt.ranks);
    if (!g_page) return 2;
    // fork before any CUDA call: every child creates its own context on its own GPU
    std::vector<int> write_fds;
    std::vector<int> read_fds(opt.ranks, -1);
    for (int r = 1; r < opt.ranks; ++r) {
        int fds[2];
        if (pipe(fds) != 0) return 2;
        read_fds[r] = fds[0];
        write_fds.push_back(fds[1]);
    }
    std::vector<pid_t> children;
    for (int r = 0; r < opt.ranks; ++r) {
        const pid_t pid = fork();
        if (pid < 0) return 2;
        if (pid == 0) _exit(run_rank(r, opt, read_fds[r], r == 0 ? write_fds : std::vector<int>()));
        children.push_back(pid);
    }
    // A rank that fails raises the stop flag itself where it can; the parent raises it for a rank that died
    // without a word.  The survivors see it at their next host rendezvous and leave on their own, between
    // steps, with no collective in flight: nobody is signalled.
    int rc = 0;
    for (size_t done = 0; done < children.size(); ++done) {
        int status = 0;
        const pid_t pid = wait(&status);
        const bool ok = pid > 0 && WIFEXITED(status) && WEXITSTATUS(status) == 0;
        if (!ok) {
            int which = -1;
            for (size_t r = 0; r < children.size(); ++r)
                if (children[r] == pid) which = static_cast<int>(r);
            if (rc == 0) rc = 1;
            b200::rendezvous_fail(g_page, which);
        }
    }
    b200::rendezvous_destroy(g_page);
    return rc;
}
