"""Multi-GPU seams of the linear-layer path (one process per GPU, torch.distributed for the plumbing).

The reference is single-GPU (no NCCL/MPI anywhere in it); what follows is the host logic a
data-parallel driver around its `ModelBF16` needs for THIS path:

  * tokens shard across ranks (every per-layer GEMM is independent along M), the dW buckets are
    summed across ranks once per optimizer step -- a sum, not a mean: the reference never divides
    by the number of micro-batches (cuda/crossentropy.cu scales by 1/BT only);
  * the LM head [K, V] shards along the vocabulary in whole 256-column tiles; cross-entropy then
    needs the row maximum and the row sum-of-exponentials across ranks (two small all-reduces)
    and the target logit from the rank that owns it.

The exchange logic is device-agnostic torch.distributed (gloo ranks on CPU in the tests, NCCL on GPUs); the
GEMMs go through `linear.matmul_forward / matmul_backward` and the per-shard cross-entropy steps through
this library's CUDA kernels (`linear.ce_shard_*`).
"""
import torch
import torch.distributed as dist

VOCAB_TILE = 256  # LM-head columns per tile of the widest GEMM tile


def shard_tokens(n_microbatches, world, rank):
    """Micro-batches [start, start+count) of an optimizer step owned by `rank` (contiguous, sizes
    differ by at most one).  The reference's accumulation loop (llama2-mistral/src/main.cpp:159-179)
    runs `accum` micro-batches per step; data parallelism deals them out."""
    if world <= 0 or not (0 <= rank < world) or n_microbatches < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(n_microbatches, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def vocab_shards(vocab, world, tile=VOCAB_TILE):
    """[(start, size)] per rank: whole tiles, as even as the tile count allows; the last shard
    absorbs the ragged tail.  V = 128256 on 8 ranks gives 501 tiles -> 63,63,63,63,63,62,62,62."""
    if vocab <= 0 or world <= 0:
        raise ValueError("bad vocabulary shard request")
    tiles = -(-vocab // tile)
    base, extra = divmod(tiles, world)
    out, start = [], 0
    for r in range(world):
        n = (base + (1 if r < extra else 0)) * tile
        n = max(0, min(n, vocab - start))
        out.append((start, n))
        start += n
    return out


class GradBuckets:
    """dW of every projection as views into one flat buffer, so that one collective sums them all.
    `shapes` is [(K, N), ...] in the order the backward pass produces them."""

    def __init__(self, shapes, dtype, device):
        self.shapes = list(shapes)
        total = sum(k * n for k, n in self.shapes)
        self.flat = torch.zeros(total, dtype=dtype, device=device)
        self.views, off = [], 0
        for k, n in self.shapes:
            self.views.append(self.flat[off:off + k * n].view(k, n))
            off += k * n

    def zero(self):
        self.flat.zero_()

    def all_reduce(self, group=None):
        """Sum over ranks (the reference accumulates micro-batch gradients by summation)."""
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
        return self.flat


class CudaShardOps:
    """The four per-shard steps of the vocabulary-parallel cross-entropy as this library's CUDA kernels
    (csrc/ce_shard.cuh).  CUDA tensors only: there is no host implementation in the package."""

    @staticmethod
    def stats(logits_local, targets, vocab_start):
        from . import linear
        return linear.ce_shard_stats(logits_local, targets, vocab_start)

    @staticmethod
    def rescale(local_max, global_max, row_sum):
        from . import linear
        return linear.ce_shard_rescale(local_max, global_max, row_sum)

    @staticmethod
    def loss(global_max, global_sum, target_logit):
        from . import linear
        return linear.ce_shard_loss(global_max, global_sum, target_logit)

    @staticmethod
    def backward(logits_local, targets, vocab_start, global_max, global_sum, scale, out=None):
        from . import linear
        return linear.ce_shard_backward(logits_local, targets, vocab_start, global_max, global_sum, scale, out=out)


def vocab_parallel_cross_entropy(logits_local, targets, vocab_start, group=None, ops=CudaShardOps, in_place=False,
                                 exchange=True, stats=None):
    """Cross-entropy over a vocabulary that is split across ranks.

    logits_local [BT, V_r] (bf16) are this rank's columns [vocab_start, vocab_start + V_r) of the LM-head
    output; targets [BT] (int32) are global token ids.  Returns (loss_rows fp32 [BT], dlogits_local) with
    dlogits = (softmax - onehot) / BT restricted to this rank's columns -- the same scaling as the
    reference's crossentropy_softmax_backward (cuda/crossentropy.cu:50-64,124-132).
    Communication: all-reduce MAX of the row maxima, then one all-reduce SUM of [sum-exp, target logit].
    `ops` supplies the four per-shard steps: this library's CUDA kernels unless a test passes a host
    restatement to exercise the exchange without a GPU.  in_place=True writes dlogits over the logits (the
    CUDA kernels allow it; no second [BT, V_r] buffer).  exchange=False treats the local columns as the
    whole vocabulary even inside a process group (a single-GPU baseline run on every rank).
    stats = (row_max, row_sum, row_target) of the local columns when the LM-head GEMM has already formed them in its
    epilogue (linear.forward_ce_stats): the pass over the logits that computes them is then skipped."""
    bt = logits_local.shape[0]
    multi = exchange and dist.is_initialized() and dist.get_world_size(group) > 1
    local_max, row_sum, tgt = stats if stats is not None else ops.stats(logits_local, targets, vocab_start)
    global_max = local_max.clone()
    if multi:
        dist.all_reduce(global_max, op=dist.ReduceOp.MAX, group=group)
    ops.rescale(local_max, global_max, row_sum)
    packed = torch.stack([row_sum, tgt])
    if multi:
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    global_sum, tgt_logit = packed[0].contiguous(), packed[1].contiguous()
    loss_rows = ops.loss(global_max, global_sum, tgt_logit)
    if in_place:
        d = ops.backward(logits_local, targets, vocab_start, global_max, global_sum, 1.0 / bt, out=logits_local)
    else:
        d = ops.backward(logits_local, targets, vocab_start, global_max, global_sum, 1.0 / bt)
    return loss_rows, d


def reduce_input_gradient(dx_partial, group=None):
    """dX of a vocabulary-sharded LM head: every rank holds dlogits_r @ W_r^T, the sum over ranks is
    the gradient of the (replicated) final hidden state."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(dx_partial, op=dist.ReduceOp.SUM, group=group)
    return dx_partial
