"""CPU restatement of the reference's softmax cross-entropy for the vocabulary-sharded LM head.

TEST INFRASTRUCTURE ONLY: imported by tests/ (and nothing in the product path).

Follows cuda/crossentropy.cu of chriskuchar/llms-from-scratch-cuda:
  * forward, bf16 overload (:96-122): per row, max over V; e = bf16(exp(l - max)) written in place of the
    logits, sum accumulated from the unrounded e in fp32; p = bf16(float(e) / sum); loss = -log(float(p[target])).
  * backward, bf16 overload (:124-132, scale = loss_scale / BT at :155): dlogits = bf16((float(p) - onehot) * scale).
`reference_bf16` reproduces that rounding sequence; `exact` is the same mathematics in float64 with no
intermediate rounding (what the sharded kernels are compared against: they round dlogits once and the loss
not at all).  `HostShardOps` restates the four per-shard steps of the sharded algorithm (stats / rescale /
loss / backward) on CPU tensors so that the exchange logic can run on gloo ranks without a GPU.

Parity unpinned by the reference itself: it ships no test or golden vector for cross-entropy.  The pin is
tests/test_ce_shard_gpu.py::test_against_reference_kernels_live, which runs the reference's own, unmodified
kernels (compiled from its checkout into oracle/_ref) next to the sharded ones on the same inputs.
"""
import numpy as np
import torch


def _bf16(x):
    return x.to(torch.bfloat16).to(torch.float32)


def exact(logits, targets):
    """float64 loss rows and dlogits = (softmax - onehot) / BT for logits [BT, V] (any float dtype)."""
    l = logits.double()
    bt = l.shape[0]
    loss = torch.logsumexp(l, dim=1) - l.gather(1, targets.long()[:, None]).squeeze(1)
    d = torch.softmax(l, dim=1)
    d[torch.arange(bt), targets.long()] -= 1.0
    return loss, d / bt


def reference_bf16(logits_bf16, targets, loss_scale=1.0):
    """The reference's own rounding sequence (bf16 overloads): returns (loss rows fp32, dlogits bf16)."""
    l = logits_bf16.to(torch.float32)
    bt = l.shape[0]
    m = l.max(dim=1).values
    e32 = torch.exp(l - m[:, None])                    # expf in fp32
    s = e32.sum(dim=1, dtype=torch.float32)            # the sum uses the unrounded exponentials
    e = _bf16(e32)                                     # stored as bf16
    p = _bf16(e / s[:, None])                          # normalised from the stored value, stored as bf16
    loss = -torch.log(p.gather(1, targets.long()[:, None]).squeeze(1))
    ind = torch.zeros_like(p)
    ind[torch.arange(bt), targets.long()] = 1.0
    d = ((p - ind) * np.float32(loss_scale / bt)).to(torch.bfloat16)
    return loss, d


class HostShardOps:
    """The four per-shard steps on CPU tensors (float64 inside), mirroring csrc/ce_shard.cuh."""

    @staticmethod
    def stats(logits_local, targets, vocab_start):
        x = logits_local.double()
        bt, v_r = x.shape
        if v_r == 0:
            z = torch.zeros(bt, dtype=torch.float32)
            return torch.full((bt,), -float("inf"), dtype=torch.float32), z, z.clone()
        m = x.max(dim=1).values
        s = torch.exp(x - m[:, None]).sum(dim=1)
        local = targets.long() - vocab_start
        mine = (local >= 0) & (local < v_r)
        t = torch.where(mine, x.gather(1, local.clamp(0, v_r - 1)[:, None]).squeeze(1), torch.zeros_like(m))
        return m.float(), s.float(), t.float()

    @staticmethod
    def rescale(local_max, global_max, row_sum):
        f = torch.where(torch.isinf(local_max), torch.zeros_like(local_max), torch.exp(local_max - global_max))
        row_sum.mul_(f)
        return row_sum

    @staticmethod
    def loss(global_max, global_sum, target_logit):
        return torch.log(global_sum) + global_max - target_logit

    @staticmethod
    def backward(logits_local, targets, vocab_start, global_max, global_sum, scale):
        x = logits_local.double()
        bt, v_r = x.shape
        d = torch.exp(x - global_max.double()[:, None]) / global_sum.double()[:, None]
        local = targets.long() - vocab_start
        mine = (local >= 0) & (local < v_r)
        if v_r > 0:
            d[mine, local[mine]] -= 1.0
        return (d * scale).to(logits_local.dtype)
