"""The drop-in claim end to end: the reference's unmodified training program, relinked against this
library (no cuBLAS), follows the reference build's loss curve on the README's overfit recipe."""
import pytest

pytestmark = pytest.mark.gpu


def test_overfit_loss_curve_matches_reference_build():
    from oracle import train_dropin
    ref, ours = train_dropin.binaries()
    if not ref or not ours:
        pytest.skip("oracle/_ref/train_* not built (reference checkout absent at build time)")
    res = train_dropin.overfit(steps=200, repeats_ref=2)
    a, b = (r["losses"] for r in res["reference"])
    o = res["b200"]["losses"]
    assert res["b200"]["rc"] == 0 and all(r["rc"] == 0 for r in res["reference"]), res["b200"]["tail"]
    assert set(o) == set(a) and 200 in o and 1 in o
    for step in sorted(o):
        ref_mid = 0.5 * (a[step] + b[step])
        spread = abs(a[step] - b[step])  # the reference's own run-to-run spread (float atomics in its kernels)
        if ref_mid > 0.05:
            # 1 % where the curve is flat (the first steps); 3 % on the steep part of the overfit, where two
            # runs of the reference itself differ by 0.5 % and a different fp32 summation order inside the
            # GEMMs moves the trajectory a little further (seen: 1.5 % at step 30)
            tol = 0.01 if step <= 5 else 0.03
            assert abs(o[step] - ref_mid) <= tol * ref_mid + spread, (step, o[step], a[step], b[step])
        else:
            # the program prints four decimals; this deep into the overfit the curve is chaotic at that
            # resolution (bf16 weights, different summation order): agree to three printed units
            assert abs(o[step] - ref_mid) <= 3.5e-4 + spread, (step, o[step], a[step], b[step])
    assert o[1] > 10.0 and o[200] <= 2e-4  # it starts at ln(32000) and it has overfitted by step 200
