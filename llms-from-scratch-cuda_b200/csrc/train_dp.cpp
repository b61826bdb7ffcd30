// Data-parallel driver around the reference's own training objects (one process per GPU, NCCL).
//
// The reference trains on one GPU (llama2-mistral/src/main.cpp:140-210): per optimizer step it runs
// `accum` micro-batches through ModelBF16::forward / backward (whose linear layers are this library's
// GEMMs once the binary is linked against libb200_linear.so), then takes the gradient norm, clips and
// updates.  Every per-layer GEMM is independent along the token dimension, so the micro-batches of a step
// can be dealt out to R ranks; what has to be exchanged is the gradient sum, once per step:
//   * grads.storage past the embedding rows (bf16)  and  dwte_fp32 (fp32)  -> all-reduce SUM
//     (a sum, not a mean: the reference never divides by the number of micro-batches,
//      cuda/crossentropy.cu:155 scales by 1/BT only)
//   * then every rank runs the identical norm / clip / AdamW update on identical gradients.
// This file is compiled together with the reference's unmodified model.cpp, dataloader.cpp and kernel
// sources, taken from the reference checkout at build time (oracle/build.py); it includes the reference's
// headers and copies nothing from them.  The step logic below follows main.cpp:149-196 call for call.
//
// Usage: train_dp <tokens.bin> --ranks R [--steps S] [--batch B] [--accum A] [--warmup W] [--lr LR]
//   A = micro-batches per optimizer step over all ranks (a multiple of R); micro-batch g of a step goes to
//   rank g % R, so R ranks together consume exactly the token stream the single-GPU program consumes.
//   The processes are forked before any CUDA call; the NCCL id travels from rank 0 over pipes.
#include <nccl.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <csignal>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "dataloader.h"
#include "kernels.cuh"
#include "model.h"

namespace {

// llama2-mistral/src/main.cpp:9-21: linear warm-up, then cosine decay to min_lr.
float lr_at(int step, float peak_lr, float min_lr, int warmup_steps, int max_steps) {
    if (step < warmup_steps) return peak_lr * (static_cast<float>(step) / static_cast<float>(warmup_steps));
    float progress = static_cast<float>(step - warmup_steps) / static_cast<float>(max_steps - warmup_steps);
    if (progress > 1.0f) progress = 1.0f;
    return min_lr + (peak_lr - min_lr) * 0.5f * (1.0f + cosf(3.14159265f * progress));
}

#define NCCL_TRY(call)                                                                      \
    do {                                                                                    \
        ncclResult_t r_ = (call);                                                           \
        if (r_ != ncclSuccess) {                                                            \
            fprintf(stderr, "NCCL error %s:%d: %s\n", __FILE__, __LINE__, ncclGetErrorString(r_)); \
            exit(EXIT_FAILURE);                                                             \
        }                                                                                   \
    } while (0)

struct Options {
    const char* data = nullptr;
    int ranks = 1, steps = 3, batch = 16, accum = 16, warmup = 2000;
    float lr = 3e-4f;
};

int run_rank(int rank, const Options& opt, int id_read_fd, const std::vector<int>& id_write_fds) {
    CUDA_CHECK(cudaSetDevice(rank));
    ncclUniqueId id;
    if (rank == 0) {
        NCCL_TRY(ncclGetUniqueId(&id));
        for (int fd : id_write_fds)
            if (write(fd, &id, sizeof(id)) != static_cast<ssize_t>(sizeof(id))) return 2;
    } else if (read(id_read_fd, &id, sizeof(id)) != static_cast<ssize_t>(sizeof(id))) {
        return 2;
    }
    ncclComm_t comm;
    NCCL_TRY(ncclCommInitRank(&comm, opt.ranks, id, rank));

    ModelConfig model_cfg;
    TrainConfig train_cfg;
    train_cfg.learning_rate = opt.lr;
    train_cfg.max_steps = opt.steps;
    train_cfg.warmup_steps = opt.warmup;
    const int B = opt.batch, T = train_cfg.seq_len, accum = opt.accum;
    ModelBF16 model;  // every rank builds the same weights: the reference seeds its own generator
    model.build(model_cfg, B, T);
    DataLoader loader;
    loader.open(opt.data, B, T);
    float* loss_dev = nullptr;
    CUDA_CHECK(cudaMalloc(&loss_dev, sizeof(float)));

    const int N = static_cast<int>(model.params.storage.numel);
    const int emb_N = model.config.vocab_size * model.config.n_embd;
    const long long tokens_per_step = 1LL * B * T * accum;
    if (rank == 0)
        printf("data parallel over %d GPUs: %d micro-batches of %d x %d tokens per step (%lld tokens), %d per rank\n",
               opt.ranks, accum, B, T, tokens_per_step, accum / opt.ranks);

    auto t_start = std::chrono::steady_clock::now();
    for (int step = 1; step <= opt.steps; ++step) {
        if (step == 2) {  // the first step carries set-up costs (allocations, NCCL connections): time from the second
            CUDA_CHECK(cudaDeviceSynchronize());
            t_start = std::chrono::steady_clock::now();
        }
        const float lr = lr_at(step, train_cfg.learning_rate, train_cfg.min_lr, train_cfg.warmup_steps, train_cfg.max_steps);
        model.zero_grad();
        float local_loss = 0.0f;
        for (int micro = 0; micro < accum; ++micro) {
            if (!loader.next_batch()) {
                loader.reset();
                loader.next_batch();
            }
            if (micro % opt.ranks != rank) continue;  // another rank's micro-batch: only the stream position moves
            model.forward(loader.input_ids_gpu, loader.targets_gpu, B, T);
            model.backward(B, T);
            embedding_backward(model.dwte_fp32, model.dx, loader.input_ids_gpu, B, T, model.config.n_embd);
            local_loss += model.loss;
        }
        // one exchange per optimizer step, on the stream the reference's kernels use (the legacy default stream)
        if (opt.ranks > 1) {
            NCCL_TRY(ncclGroupStart());
            NCCL_TRY(ncclAllReduce(model.grads.storage.data + emb_N, model.grads.storage.data + emb_N,
                                   static_cast<size_t>(N - emb_N), ncclBfloat16, ncclSum, comm, 0));
            NCCL_TRY(ncclAllReduce(model.dwte_fp32, model.dwte_fp32, static_cast<size_t>(emb_N), ncclFloat, ncclSum, comm, 0));
            NCCL_TRY(ncclGroupEnd());
            CUDA_CHECK(cudaMemcpy(loss_dev, &local_loss, sizeof(float), cudaMemcpyHostToDevice));
            NCCL_TRY(ncclAllReduce(loss_dev, loss_dev, 1, ncclFloat, ncclSum, comm, 0));
            CUDA_CHECK(cudaMemcpy(&local_loss, loss_dev, sizeof(float), cudaMemcpyDeviceToHost));
        }
        const float loss = local_loss / accum;
        const float global_norm = compute_grad_norm_bf16(model.dwte_fp32, emb_N, model.grads.storage.data + emb_N,
                                                         N - emb_N, model.loss_scale);
        const float clip_scale = global_norm > train_cfg.grad_clip ? train_cfg.grad_clip / global_norm : 1.0f;
        model.update(lr, train_cfg, step, clip_scale);
        CUDA_CHECK(cudaDeviceSynchronize());
        if (rank == 0) {
            const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count();
            if (step >= 2)
                printf("step %5d | loss %.4f | lr %.2e | norm %.4f | %.0f tok/s (wall clock, steps 2..%d)\n", step, loss,
                       lr, global_norm, (step - 1) * tokens_per_step / secs, step);
            else
                printf("step %5d | loss %.4f | lr %.2e | norm %.4f\n", step, loss, lr, global_norm);
            fflush(stdout);
        }
    }
    CUDA_CHECK(cudaFree(loss_dev));
    NCCL_TRY(ncclCommDestroy(comm));
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    Options opt;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--ranks") && i + 1 < argc) opt.ranks = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--steps") && i + 1 < argc) opt.steps = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--batch") && i + 1 < argc) opt.batch = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--accum") && i + 1 < argc) opt.accum = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) opt.warmup = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--lr") && i + 1 < argc) opt.lr = static_cast<float>(atof(argv[++i]));
        else if (argv[i][0] != '-') opt.data = argv[i];
    }
    if (!opt.data || opt.ranks < 1 || opt.ranks > 8 || opt.accum < 1 || opt.accum % opt.ranks != 0 || opt.steps < 1) {
        fprintf(stderr, "usage: %s <tokens.bin> --ranks R [--steps S] [--batch B] [--accum A (multiple of R)] [--warmup W] [--lr LR]\n",
                argv[0]);
        return 2;
    }
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
    int rc = 0;
    for (size_t done = 0; done < children.size(); ++done) {
        int status = 0;
        const pid_t pid = wait(&status);
        const bool ok = pid > 0 && WIFEXITED(status) && WEXITSTATUS(status) == 0;
        if (!ok && rc == 0) {
            rc = 1;  // one rank failed: the others would wait for it in the next collective
            for (pid_t c : children)
                if (c != pid) kill(c, SIGTERM);
        }
    }
    return rc;
}
