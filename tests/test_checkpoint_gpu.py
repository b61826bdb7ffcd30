"""On-disk compatibility with the reference: the checkpoint file (llama2-mistral/src/main.cpp:212-254: fp32 master
weights, magic, step, the two AdamW moments) and the token file (dataloader.cpp:6-30: raw int32 ids).  The package's
driver writes a checkpoint that the reference's own program resumes from, and the other way round; a program that
continues from the other's file must print the loss it prints when continuing from its own."""
import pytest

pytestmark = pytest.mark.gpu

N_PARAMS = 124_668_672  # llama2-mistral 125M (README.md:15 of the reference)


def test_checkpoints_and_token_files_interoperate():
    from oracle import train_dropin
    ref, _ = train_dropin.binaries()
    ours, _ = train_dropin.dp_binaries()
    if not ref or not ours:
        pytest.skip("oracle/_ref/train_ref_* / train_dp_b200_* not built (reference checkout absent at build time)")
    res = train_dropin.checkpoint_roundtrip()
    assert res["token_file_bytes"] == (3 * 512 + 1) * 4
    losses = {}
    for writer in ("driver", "reference"):
        e = res[writer]
        assert e["write"]["rc"] == 0, e["write"]["tail"]
        assert "DataLoader: 1537 tokens" in e["write"]["stdout"]          # both programs read the same token file
        assert e["bytes"] == 3 * N_PARAMS * 4 + 8, (writer, e["bytes"])    # weights + magic + step + two moments
        for reader in ("resume_reference", "resume_driver"):
            r = e[reader]
            assert r["rc"] == 0, r["tail"]
            assert "Restored optimizer state from step 2" in r["stdout"], r["tail"]
            assert set(r["losses"]) == {3}, r["losses"]                    # the step counter continues
            losses[(writer, reader)] = r["losses"][3]
    # the two writers ran the same two steps (different GEMM libraries): their files agree to training noise
    for reader in ("resume_reference", "resume_driver"):
        a, b = losses[("driver", reader)], losses[("reference", reader)]
        assert abs(a - b) <= 0.01 * b, losses
    # one file, two readers: the same third step
    for writer in ("driver", "reference"):
        a, b = losses[(writer, "resume_reference")], losses[(writer, "resume_driver")]
        assert abs(a - b) <= 0.01 * b, losses
