"""World-size-2 (gloo, CPU) tests of the multi-GPU host logic: token sharding, dW bucket
all-reduce and the vocabulary-parallel cross-entropy exchange."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _load_dist():
    import importlib.util
    path = os.path.join(ROOT, "llms-from-scratch-cuda_b200", "dist.py")
    spec = importlib.util.spec_from_file_location("b200_dist_under_test", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_shard_tokens_partitions_every_microbatch():
    d = _load_dist()
    for n in (0, 1, 7, 16, 17):
        for world in (1, 2, 3, 8):
            got = [d.shard_tokens(n, world, r) for r in range(world)]
            covered = [i for s, c in got for i in range(s, s + c)]
            assert covered == list(range(n))
            sizes = [c for _, c in got]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        d.shard_tokens(4, 2, 2)


def test_vocab_shards_are_tile_granular():
    d = _load_dist()
    sh = d.vocab_shards(128256, 8)
    assert sum(n for _, n in sh) == 128256
    assert [s for s, _ in sh] == [sum(n for _, n in sh[:i]) for i in range(8)]
    assert all(n % 256 == 0 for _, n in sh)          # 128256 = 501 * 256
    assert max(n for _, n in sh) - min(n for _, n in sh) == 256
    sh = d.vocab_shards(32000, 8)
    assert sum(n for _, n in sh) == 32000 and all(n % 256 == 0 for _, n in sh)
    sh = d.vocab_shards(1000, 3)                      # ragged tail lands in the last non-empty shard
    assert sum(n for _, n in sh) == 1000 and sh[0][1] % 256 == 0
    sh = d.vocab_shards(300, 4)                       # more ranks than tiles: empty shards are legal
    assert sum(n for _, n in sh) == 300 and sh[-1][1] == 0


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        d = _load_dist()
        torch.manual_seed(123)  # same data on every rank
        bt, k, v = 24, 16, 1000
        x = torch.randn(bt, k, dtype=torch.float64)
        w = torch.randn(k, v, dtype=torch.float64) * 0.3
        targets = torch.randint(0, v, (bt,))
        # full-vocabulary reference
        logits = x @ w
        ref_loss = torch.logsumexp(logits, dim=1) - logits.gather(1, targets[:, None]).squeeze(1)
        ref_d = torch.softmax(logits, dim=1)
        ref_d[torch.arange(bt), targets] -= 1
        ref_d /= bt
        ref_dx = ref_d @ w.T
        # sharded
        start, size = d.vocab_shards(v, world)[rank]
        w_r = w[:, start:start + size].contiguous()
        from oracle.ce_oracle import HostShardOps  # host restatement of the per-shard kernels: no GPU here
        loss_rows, d_local = d.vocab_parallel_cross_entropy((x @ w_r).float(), targets, start, ops=HostShardOps)
        dx = d.reduce_input_gradient(d_local.double() @ w_r.T)
        ok_loss = torch.allclose(loss_rows.double(), ref_loss, atol=1e-4)
        ok_d = torch.allclose(d_local.double(), ref_d[:, start:start + size], atol=1e-6)
        ok_dx = torch.allclose(dx, ref_dx, atol=1e-5)
        # the same with the per-shard statistics handed in (as the LM-head GEMM's epilogue delivers them): the
        # statistics pass is skipped, the exchange and the result are unchanged
        logits_r = (x @ w_r).float()
        pre = HostShardOps.stats(logits_r, targets, start)
        loss2, d2 = d.vocab_parallel_cross_entropy(logits_r, targets, start, ops=HostShardOps, stats=pre)
        ok_loss = ok_loss and torch.equal(loss2, loss_rows)
        ok_d = ok_d and torch.equal(d2, d_local)
        # dW buckets: every rank contributes rank+1; the sum is world*(world+1)/2
        b = d.GradBuckets([(4, 6), (3, 5)], torch.float32, "cpu")
        for view in b.views:
            view.fill_(float(rank + 1))
        b.all_reduce()
        ok_b = bool((b.flat == world * (world + 1) / 2).all()) and b.views[1].shape == (3, 5)
        # token sharding covers the step once
        s, c = d.shard_tokens(16, world, rank)
        counts = torch.tensor([c])
        dist.all_reduce(counts)
        q.put((rank, ok_loss, ok_d, ok_dx, ok_b, int(counts.item()) == 16))
    finally:
        dist.destroy_process_group()


def test_world_size_two_exchange():
    world, port = 2, 29517 + (os.getpid() % 200)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in results:
        assert all(r[1:]), r
