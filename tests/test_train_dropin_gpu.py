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
    res = train_dropin.overfit(steps=60, repeats_ref=3)
    refs = [r["losses"] for r in res["reference"]]
    a = refs[0]
    o = res["b200"]["losses"]
    assert res["b200"]["rc"] == 0 and all(r["rc"] == 0 for r in res["reference"]), res["b200"]["tail"]
    assert set(o) == set(a) and 60 in o and 1 in o
    for step in sorted(o):
        v = [r[step] for r in refs]
        ref_mid = sum(v) / len(v)
        # the reference's own run-to-run spread (float atomics in its kernels): three runs, because on the steepest
        # steps of the curve (7.7 -> 0.27 between steps 10 and 30) two runs can agree by chance to 0.2 % while a third
        # lies 1 % away
        spread = max(v) - min(v)
        # 1 % of the loss, twice that spread, and the print resolution
        assert abs(o[step] - ref_mid) <= 0.01 * ref_mid + 2 * spread + 1e-4, (step, o[step], v)
    assert o[1] > 10.0 and o[60] < 0.05  # it starts at ln(32000) and is deep into the overfit by step 60


def _curve_stats(runs, step):
    v = [x[step] for x in runs]
    return sum(v) / len(v), max(v) - min(v)


def test_step_200_loss_within_one_percent_at_eight_digits():
    """Three links of the same driver, 200 steps each: the reference's matmul.cu (cuBLAS) three times -- its kernels use
    float atomics, so its own curve moves from run to run; that spread is the resolution of any comparison --, this
    library's linear layers twice, and this library's linear layers plus its attention / SwiGLU / RMSNorm /
    cross-entropy drop-ins twice.  The linear-layer link must stay within 1 % of the reference link at every step,
    up to twice the two links' own spreads (three and two runs underestimate a range).  The layer drop-ins compute
    attention and the RMSNorm weight gradient in fp32 where the reference rounds to bf16 in between, so that link's
    trajectory differs by more on the steep part of the overfit: it is held to 10 % (plus 1e-3 absolute).  Both bounds apply
    at every step at which the reference link's loss is above 0.01 (eleven orders of the curve: 10.5 down to 0.01); in the
    memorised tail below that, where the reference link's own runs differ by tens of percent, both links must have
    converged below 0.01 as well.  The curves are printed."""
    from oracle import train_dropin
    layers_bin, ref = train_dropin.dp_binaries()
    if not ref or not layers_bin or not train_dropin.dp_gemm_binary():
        pytest.skip("oracle/_ref/train_dp_* not built (reference checkout absent at build time)")
    res = train_dropin.overfit_digits(steps=200, repeats_ref=3, repeats_ours=2)
    runs = {k: [r["losses"] for r in v] for k, v in res.items()}
    for k, v in res.items():
        assert all(r["rc"] == 0 for r in v), (k, v[0]["tail"])
        assert all(set(x) == set(range(1, 201)) for x in runs[k]), k
    report, worst, last_resolved = [], {"b200": (0.0, 0), "b200_layers": (0.0, 0)}, None
    for step in range(1, 201):
        ref_mid, ref_spread = _curve_stats(runs["reference"], step)
        if ref_mid >= 100 * ref_spread:
            last_resolved = step  # here the reference link's own spread is below the 1 % under test
        for link, pct in (("b200", 0.01), ("b200_layers", 0.10)):
            mid, spread = _curve_stats(runs[link], step)
            excess = abs(mid - ref_mid) - 2 * (ref_spread + spread)
            if ref_mid > 0 and excess / ref_mid > worst[link][0]:
                worst[link] = (excess / ref_mid, step)
            if ref_mid < 1e-2:
                # the memorised tail (loss 1e-2 .. 1e-5): trajectories at this scale are chaotic -- the reference
                # link's own three runs differ by tens of percent there, which two or three runs cannot bound --, so
                # both links are only required to have converged as well
                assert mid < 1e-2, (link, step, [x[step] for x in runs["reference"]], [x[step] for x in runs[link]])
                continue
            floor = 1e-3 if link == "b200_layers" else 0.0
            assert excess <= pct * ref_mid + floor, (link, step, [x[step] for x in runs["reference"]], [x[step] for x in runs[link]])
        if step in (1, 10, 20, 30, 40, 50, 100, 150, 200):
            report.append((step, [x[step] for x in runs["reference"]], [x[step] for x in runs["b200"]],
                           [x[step] for x in runs["b200_layers"]]))
    print("overfit, 8 digits (step, reference link x3, linear layers x2, all layers x2):")
    for row in report:
        print("  ", row)
    print("largest relative deviation beyond twice the spreads (fraction of the loss, step):", worst)
    print("last step at which the reference link's spread is below 1 %% of its loss: %s" % last_resolved)
    assert last_resolved is not None and last_resolved >= 5
    assert runs["reference"][0][1] > 10.0
    assert all(x[200] < 1e-3 for k in runs for x in runs[k])
