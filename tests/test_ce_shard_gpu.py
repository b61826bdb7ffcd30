"""GPU parity tests of the vocabulary-sharded cross-entropy kernels (csrc/ce_shard.cuh), called through the
C ABI, against the float64 restatement in oracle/ce_oracle.py and the reference's own crossentropy.cu.

Tolerances: loss rows are fp32 -> |loss - loss64| <= 2e-5 * max(1, |loss64|); dlogits is bf16 ->
max|d - d64| / max|d64| <= 1e-2 (the bf16 tolerance of the north star)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _single_rank(pkg, logits, targets, shards):
    """All shards on one GPU; the exchange between ranks is done here with torch on [rows] vectors."""
    stats = [pkg.ce_shard_stats(logits[:, a:a + n], targets, a) for a, n in shards]
    gmax = torch.stack([s[0] for s in stats]).max(dim=0).values
    sums, tgt = [], []
    for lm, sm, tg in stats:
        pkg.ce_shard_rescale(lm, gmax, sm)
        sums.append(sm)
        tgt.append(tg)
    gsum = torch.stack(sums).sum(dim=0)
    gtgt = torch.stack(tgt).sum(dim=0)
    loss = pkg.ce_shard_loss(gmax, gsum, gtgt)
    d = torch.empty_like(logits)
    for a, n in shards:
        pkg.ce_shard_backward(logits[:, a:a + n], targets, a, gmax, gsum, 1.0 / logits.shape[0], out=d[:, a:a + n])
    torch.cuda.synchronize()
    return loss, d


def _check(loss, d, logits, targets):
    from oracle import ce_oracle
    loss64, d64 = ce_oracle.exact(logits.cpu(), targets.cpu())
    assert ((loss.double().cpu() - loss64).abs() <= 2e-5 * loss64.abs().clamp(min=1.0)).all()
    err = (d.double().cpu() - d64).abs().max() / d64.abs().max()
    assert err <= 1e-2, err


@pytest.mark.parametrize("rows,vocab", [(512, 32000), (1000, 1003), (37, 8), (256, 128256)])
def test_one_shard_against_float64(pkg, handle, rows, vocab):
    g = torch.Generator(device=DEV).manual_seed(rows + vocab)
    logits = (3.0 * torch.randn(rows, vocab, device=DEV, generator=g)).to(torch.bfloat16)
    targets = torch.randint(0, vocab, (rows,), device=DEV, generator=g, dtype=torch.int32)
    loss, d = _single_rank(pkg, logits, targets, [(0, vocab)])
    _check(loss, d, logits, targets)


def test_ragged_and_empty_shards_combine(pkg, handle):
    g = torch.Generator(device=DEV).manual_seed(7)
    rows, vocab = 300, 5000
    logits = (4.0 * torch.randn(rows, vocab, device=DEV, generator=g)).to(torch.bfloat16)
    logits[5, 4999] = 60.0   # a row whose maximum sits in the last, ragged shard
    logits[6, :] = -30.0     # a flat row
    targets = torch.randint(0, vocab, (rows,), device=DEV, generator=g, dtype=torch.int32)
    targets[5] = 4999
    shards = [(0, 2048), (2048, 0), (2048, 2047), (4095, 905)]  # unaligned starts, one empty shard
    loss, d = _single_rank(pkg, logits, targets, shards)
    _check(loss, d, logits, targets)
    loss1, d1 = _single_rank(pkg, logits, targets, [(0, vocab)])
    assert torch.allclose(loss, loss1, atol=2e-5)
    assert (d.float() - d1.float()).abs().max() <= 2.0 ** -8 * d1.float().abs().max()


def test_masked_columns_and_fully_masked_shard(pkg, handle):
    """Logits of -inf (masked vocabulary entries): a shard whose columns are all masked, and rows in which
    one lane's share of the columns is masked, must contribute zero -- not exp(-inf - -inf) = NaN."""
    g = torch.Generator(device=DEV).manual_seed(19)
    rows, vocab = 128, 4096
    logits = (2.0 * torch.randn(rows, vocab, device=DEV, generator=g)).to(torch.bfloat16)
    logits[:, 1024:2048] = float("-inf")          # the second of four shards is masked entirely
    logits[3, :1024] = float("-inf")              # a row masked at the start (the running maximum is still -inf)
    logits[4, ::2] = float("-inf")
    targets = torch.randint(2048, vocab, (rows,), device=DEV, generator=g, dtype=torch.int32)
    targets[4] = 2049                             # an unmasked column of the row with every second one masked
    shards = [(0, 1024), (1024, 1024), (2048, 1024), (3072, 1024)]
    loss, d = _single_rank(pkg, logits, targets, shards)
    assert torch.isfinite(loss).all() and torch.isfinite(d.float()).all()
    _check(loss, d, logits, targets)
    assert (d[:, 1024:2048] == 0).all()


def test_backward_default_output_follows_a_strided_view(pkg, handle):
    g = torch.Generator(device=DEV).manual_seed(23)
    rows, vocab, ld = 32, 512, 768
    big = (2.0 * torch.randn(rows, ld, device=DEV, generator=g)).to(torch.bfloat16)
    view = big[:, :vocab]
    targets = torch.randint(0, vocab, (rows,), device=DEV, generator=g, dtype=torch.int32)
    lm, sm, tg = pkg.ce_shard_stats(view, targets, 0)
    loss = pkg.ce_shard_loss(lm, sm, tg)
    d = pkg.ce_shard_backward(view, targets, 0, lm, sm, 1.0 / rows)   # no out=: allocated to match the view
    torch.cuda.synchronize()
    _check(loss, d, view.contiguous(), targets)


def test_backward_in_place_and_strided(pkg, handle):
    g = torch.Generator(device=DEV).manual_seed(11)
    rows, vocab, ld = 64, 1536, 2048
    big = torch.zeros(rows, ld, device=DEV, dtype=torch.bfloat16)
    big[:, :vocab] = (2.0 * torch.randn(rows, vocab, device=DEV, generator=g)).to(torch.bfloat16)
    view = big[:, :vocab]
    keep = view.clone()
    targets = torch.randint(0, vocab, (rows,), device=DEV, generator=g, dtype=torch.int32)
    lm, sm, tg = pkg.ce_shard_stats(view, targets, 0)
    loss = pkg.ce_shard_loss(lm, sm, tg)
    pkg.ce_shard_backward(view, targets, 0, lm, sm, 1.0 / rows, out=view)  # in place, row pitch > columns
    torch.cuda.synchronize()
    _check(loss, view, keep, targets)
    assert (big[:, vocab:] == 0).all()


def test_against_reference_kernels_live(pkg, handle, ref_lib):
    """The reference's own crossentropy.cu (bf16 overloads) on the same inputs.  Its row count must be a
    multiple of 256: its forward kernel has no bounds check on the row index (cuda/crossentropy.cu:98)."""
    if not hasattr(ref_lib, "ref_crossentropy_forward_bf16"):
        pytest.skip("oracle/_ref was built without the reference's crossentropy.cu")
    from oracle import ce_oracle
    g = torch.Generator(device=DEV).manual_seed(3)
    B, T, V = 2, 256, 4096
    rows = B * T
    logits = (3.0 * torch.randn(rows, V, device=DEV, generator=g)).to(torch.bfloat16)
    targets = torch.randint(0, V, (rows,), device=DEV, generator=g, dtype=torch.int32)
    ours_loss, ours_d = _single_rank(pkg, logits, targets, [(0, 2048), (2048, 2048)])
    probs = logits.clone()
    ref_loss = torch.empty(rows, device=DEV, dtype=torch.float32)
    ref_lib.ref_crossentropy_forward_bf16(ref_loss.data_ptr(), probs.data_ptr(), targets.data_ptr(), B, T, V)
    ref_lib.ref_crossentropy_backward_bf16(probs.data_ptr(), probs.data_ptr(), targets.data_ptr(), B, T, V, 1.0)
    torch.cuda.synchronize()
    # the reference takes -log of a probability that went through two bf16 roundings (the stored exponential,
    # then the stored quotient): up to 2 * 2^-8 relative in p, i.e. 8e-3 in the loss
    assert (ours_loss - ref_loss).abs().max() <= 8e-3
    assert (ours_d.float() - probs.float()).abs().max() <= 1e-2 * probs.float().abs().max()
    # the CPU restatement of the reference's rounding sequence is pinned by the reference's own output
    o_loss, o_d = ce_oracle.reference_bf16(logits.cpu(), targets.cpu())
    assert (o_loss - ref_loss.cpu()).abs().max() <= 1e-5
    mism = (o_d.float() != probs.cpu().float()).float().mean().item()
    assert mism <= 0.01, mism                                   # expf vs torch.exp: rare one-ulp flips
    assert (o_d.float() - probs.cpu().float()).abs().max() <= 2.0 ** -8 * probs.float().abs().max().item()


@pytest.mark.parametrize("rows,K,V,shards", [(1024, 768, 32000, [(0, 32000)]),          # the 125M LM head, one rank
                                               (512, 256, 128256, [(0, 64256), (64256, 64000)]),   # LLaMA-3 vocabulary, two shards
                                               (300, 320, 2312, [(0, 1032), (1032, 1280)]),      # ragged rows and widths
                                               (130, 64, 520, [(0, 520)])])
def test_statistics_from_the_lm_head_epilogue(pkg, handle, rows, K, V, shards):
    """b200_linear_forward_ce_stats_bf16: the logits are the plain product's, and (row max, sum exp, target logit)
    equal what b200_ce_shard_stats_bf16 reads back from them -- maximum and target logit exactly, the sum to fp32
    rounding; the loss and dlogits that follow meet the float64 oracle (oracle/ce_oracle.py::exact) on the stored logits."""
    g = torch.Generator(device=DEV).manual_seed(8642)
    dt = torch.bfloat16
    x = torch.randn(rows, K, device=DEV, generator=g).to(dt)
    w = (torch.randn(K, V, device=DEV, generator=g) * (3.0 / K ** 0.5)).to(dt)
    targets = torch.randint(0, V, (rows,), device=DEV, generator=g, dtype=torch.int32)
    logits = torch.full((rows, V), float("nan"), device=DEV, dtype=dt)
    plain = torch.empty(rows, V, device=DEV, dtype=dt)
    fused = []
    for a, n in shards:
        fused.append(pkg.forward_ce_stats(handle, logits[:, a:a + n], x, w[:, a:a + n], rows, n, K, targets, a))
        pkg.gemm_ld(handle, pkg.FWD_NN, 0, plain[:, a:a + n], x, w[:, a:a + n], rows, n, K)
    handle.sync()
    # the same products (where the plain path splits the contraction, fp32 partial sums are added in another order)
    assert ((logits.double() - plain.double()).abs().max() / plain.double().abs().max()).item() <= 4e-3
    for (a, n), (fm, fs, ft) in zip(shards, fused):
        sm, ss, st = pkg.ce_shard_stats(logits[:, a:a + n], targets, a)
        torch.cuda.synchronize()
        assert torch.equal(fm, sm) and torch.equal(ft, st)
        assert ((fs - ss).abs() <= 1e-5 * ss.abs()).all(), ((fs - ss).abs() / ss).max()
    # the rest of the sharded cross-entropy on the fused statistics
    gmax = torch.stack([f[0] for f in fused]).max(dim=0).values
    for fm, fs, _ in fused:
        pkg.ce_shard_rescale(fm, gmax, fs)
    gsum = torch.stack([f[1] for f in fused]).sum(dim=0)
    gtgt = torch.stack([f[2] for f in fused]).sum(dim=0)
    loss = pkg.ce_shard_loss(gmax, gsum, gtgt)
    d = torch.empty_like(logits)
    for a, n in shards:
        pkg.ce_shard_backward(logits[:, a:a + n], targets, a, gmax, gsum, 1.0 / rows, out=d[:, a:a + n])
    torch.cuda.synchronize()
    _check(loss, d, logits, targets)


def test_bad_arguments(pkg, handle):
    logits = torch.zeros(4, 8, device=DEV, dtype=torch.bfloat16)
    targets = torch.zeros(4, device=DEV, dtype=torch.int32)
    with pytest.raises(pkg.LinearError):
        pkg.ce_shard_stats(logits.float(), targets, 0)          # wrong dtype
    with pytest.raises(pkg.LinearError):
        pkg.ce_shard_stats(logits.cpu(), targets.cpu(), 0)      # no host path
    with pytest.raises(pkg.LinearError):
        pkg.ce_shard_stats(logits, targets.long(), 0)           # targets must be int32
    with pytest.raises(pkg.LinearError):
        pkg.ce_shard_stats(logits, targets, -1)                 # negative column offset


def _two_rank_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import importlib
        import __graft_entry__ as ge
        pkg = ge.load_package()
        d = importlib.import_module(pkg.__name__ + ".dist")
        dev = torch.device("cuda", rank)
        g = torch.Generator(device=dev).manual_seed(99)  # same data on every rank
        bt, k, v = 2048, 768, 32000
        x = torch.randn(bt, k, device=dev, generator=g).to(torch.bfloat16)
        w = (0.05 * torch.randn(k, v, device=dev, generator=g)).to(torch.bfloat16)
        targets = torch.randint(0, v, (bt,), device=dev, generator=g, dtype=torch.int32)
        start, size = d.vocab_shards(v, world)[rank]
        w_r = w[:, start:start + size].contiguous()
        h = pkg.Handle()
        logits_r = torch.empty(bt, size, device=dev, dtype=torch.bfloat16)
        pkg.matmul_forward(h, logits_r, x, w_r, bt, size, k)          # the shard's LM-head GEMM
        loss_rows, d_r = d.vocab_parallel_cross_entropy(logits_r, targets, start)
        dx_part = torch.empty(bt, k, device=dev, dtype=torch.bfloat16)
        dw_r = torch.zeros(k, size, device=dev, dtype=torch.bfloat16)
        pkg.matmul_backward(h, dx_part, dw_r, d_r, x, w_r, bt, size, k)
        h.sync()
        dx = d.reduce_input_gradient(dx_part.float())
        # full-vocabulary check on every rank (float64 on the device)
        logits = x.double() @ w.double()
        ref_loss = torch.logsumexp(logits, dim=1) - logits.gather(1, targets.long()[:, None]).squeeze(1)
        ref_d = torch.softmax(logits, dim=1)
        ref_d[torch.arange(bt, device=dev), targets.long()] -= 1
        ref_d /= bt
        ref_dx = ref_d @ w.double().T
        ref_dw = x.double().T @ ref_d[:, start:start + size]
        ok_loss = bool(((loss_rows.double() - ref_loss).abs() <= 2e-2).all())  # logits themselves are bf16
        ok_mean = abs(loss_rows.double().mean().item() - ref_loss.mean().item()) <= 2e-3
        ok_dx = ((dx.double() - ref_dx).abs().max() / ref_dx.abs().max()).item() <= 2e-2
        ok_dw = ((dw_r.double() - ref_dw).abs().max() / ref_dw.abs().max()).item() <= 2e-2
        q.put((rank, ok_loss, ok_mean, ok_dx, ok_dw))
    finally:
        dist.destroy_process_group()


def test_two_ranks_nccl_lm_head_and_cross_entropy():
    """Config 4 in small: the LM head sharded by vocabulary over two GPUs, one process each."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, 29600 + (os.getpid() % 200)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_two_rank_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r in results:
        assert all(r[1:]), r
