"""The drop-in claim end to end, on the reference README's overfit recipe (README.md:76-91: B=1, T=512, one batch,
lr 3e-4, warmup 20, 200 steps; a seeded synthetic 513-token file stands in for the corpus slice).

1. The reference's unmodified training program, relinked against this library (no cuBLAS), follows the reference
   build's loss curve (the program prints four decimals).
2. The same recipe through the package's driver at one rank, linked once against the reference's own matmul.cu
   (cuBLAS) and once against this library, prints eight decimals: the whole curve down to step 200 is compared
   with the reference link's own run-to-run spread measured beside it."""
import pytest

pytestmark = pytest.mark.gpu


def test_reference_program_relinked_follows_the_reference_build():
    from oracle import train_dropin
    ref, ours = train_dropin.binaries()
    if not ref or not ours:
        pytest.skip("oracle/_ref/train_* not built (reference checkout absent at build time)")
    res = train_dropin.overfit(steps=60, repeats_ref=2)
    a, b = (r["losses"] for r in res["reference"])
    o = res["b200"]["losses"]
    assert res["b200"]["rc"] == 0 and all(r["rc"] == 0 for r in res["reference"]), res["b200"]["tail"]
    assert set(o) == set(a) and 60 in o and 1 in o
    for step in sorted(o):
        ref_mid = 0.5 * (a[step] + b[step])
        spread = abs(a[step] - b[step])  # the reference's own run-to-run spread (float atomics in its kernels)
        # 1 % of the loss, the spread of the reference's own two runs, and the print resolution
        assert abs(o[step] - ref_mid) <= 0.01 * ref_mid + 2 * spread + 1e-4, (step, o[step], a[step], b[step])
    assert o[1] > 10.0 and o[60] < 0.05  # it starts at ln(32000) and is deep into the overfit by step 60


def test_step_200_loss_within_one_percent_at_eight_digits():
    from oracle import train_dropin
    ours, ref = train_dropin.dp_binaries()
    if not ref or not ours:
        pytest.skip("oracle/_ref/train_dp_* not built (reference checkout absent at build time)")
    res = train_dropin.overfit_digits(steps=200, repeats_ref=3, repeats_ours=2)
    refs = [r["losses"] for r in res["reference"]]
    mine = [r["losses"] for r in res["b200"]]
    assert all(r["rc"] == 0 for r in res["reference"] + res["b200"]), res["b200"][0]["tail"]
    assert all(set(x) == set(range(1, 201)) for x in refs + mine)
    report = []
    last_resolved = None
    for step in range(1, 201):
        rv = [x[step] for x in refs]
        ov = [x[step] for x in mine]
        ref_mid, spread = sum(rv) / len(rv), max(rv) - min(rv)
        ours_mid, ours_spread = sum(ov) / len(ov), max(ov) - min(ov)
        # within 1 % of the reference link, up to what either link moves from one run to the next
        # (float atomics in the reference's rmsnorm / attention / embedding kernels, linked into both)
        assert abs(ours_mid - ref_mid) <= 0.01 * ref_mid + spread + ours_spread, (step, rv, ov)
        if ref_mid >= 100 * spread:
            last_resolved = step  # here the reference's own spread is below the 1 % under test
        if step in (1, 10, 20, 30, 50, 100, 150, 200):
            report.append((step, rv, ov))
    print("overfit, 8 digits (step, reference link runs, this library runs):", report)
    print("last step at which the reference link's spread is below 1 %% of its loss: %s" % last_resolved)
    assert last_resolved is not None and last_resolved >= 5
    assert refs[0][1] > 10.0 and all(x[200] < 1e-3 for x in refs + mine)
