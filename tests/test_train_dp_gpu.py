"""The data-parallel training driver (csrc/train_dp.cpp: the reference's own ModelBF16 objects, this library's
GEMMs, NCCL) on two GPUs against the same driver on one: same token stream, same number of micro-batches
per step, gradients summed across ranks once per step -- the loss of every step must agree."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_two_ranks_follow_one_rank():
    from oracle import train_dropin
    if not train_dropin.dp_binary():
        pytest.skip("oracle/_ref/train_dp_b200_* not built (reference checkout absent at build time)")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = train_dropin.data_parallel((1, 2), steps=3, batch=16, accum=4)
    one, two = res[1], res[2]
    assert one["rc"] == 0 and two["rc"] == 0, (one["tail"], two["tail"])
    assert set(one["losses"]) == set(two["losses"]) == {1, 2, 3}
    assert one["losses"][1] > 10.0                      # ln(32000) = 10.37 at initialisation
    for step in (1, 2, 3):
        # step 1 sees identical weights: only the order of the bf16 gradient sums differs (loss unaffected);
        # later steps differ by that rounding through one or two optimizer updates
        tol = 1e-3 if step == 1 else 1e-2
        assert abs(one["losses"][step] - two["losses"][step]) <= tol * one["losses"][step], (step, one["losses"], two["losses"])
    # The reference's optimizer step (gradient norm + update, ~9 s per step on a B200) is serial and identical on
    # every rank; with only 4 micro-batches of ~1.7 s per step, two ranks can gain 1.27x at most.
    assert two["tokens_per_s"] > 1.15 * one["tokens_per_s"], (one["tokens_per_s"], two["tokens_per_s"])
