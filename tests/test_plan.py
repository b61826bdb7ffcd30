"""Host-side plan selection (pure arithmetic, no GPU): invariants over the BASELINE shapes."""
import itertools

import pytest

MS = [512, 2048, 8192, 16384, 65536]
NKS = [768, 1280, 2048, 4096, 8192, 32000, 128256]


def _dims(which, M, N, K):
    return {0: (M, N, K), 1: (M, K, N), 2: (K, N, M)}[which]


@pytest.mark.parametrize("which", [0, 1, 2])
def test_plan_invariants(pkg, which):
    for M, N, K in itertools.product(MS, NKS, NKS):
        p = pkg.plan_bf16(which, which == 2, M, N, K, 148)
        Mo, No, Kc = _dims(which, M, N, K)
        assert p.bn in (64, 128, 192, 256)
        assert p.cta_pair in (0, 1)
        if p.cta_pair:
            assert p.bn in (128, 256)
        rows = 256 if p.cta_pair else 128
        assert p.tiles == -(-Mo // rows) * -(-No // p.bn)
        kb = -(-Kc // 64)
        assert 1 <= p.splits <= kb
        per = -(-kb // p.splits)
        assert (p.splits - 1) * per < kb  # every range owns at least one block
        assert 0 <= p.dp_tiles <= p.tiles
        assert p.sk_items == (p.tiles - p.dp_tiles) * p.splits
        if p.splits == 1:
            assert p.dp_tiles == p.tiles and p.sk_items == 0
        else:
            slots = 148 // (2 if p.cta_pair else 1)
            assert p.dp_tiles % slots == 0     # only the ragged last wave is cut
            assert p.sk_items <= slots         # and its pieces fit one wave
        assert p.m_fastest in (0, 1)
        if p.cluster_split > 1:
            ctas = 2 if p.cta_pair else 1
            assert p.splits == 1 and p.sk_items == 0
            assert p.cluster_split * ctas <= 8           # portable cluster size
            assert p.cluster_split <= p.bn // 32         # every member owns at least one column group
            assert p.cluster_split <= kb
            assert p.tiles * p.cluster_split * ctas <= 148  # one wave


def test_small_weight_gradients_split_the_token_dimension(pkg):
    # dW of the 125M projections: the output alone gives far fewer tiles than SMs
    for N, K in ((768, 768), (256, 768), (2048, 768), (768, 2048)):
        p = pkg.plan_bf16(2, 1, 8192, N, K, 148)
        ctas = 2 if p.cta_pair else 1
        if p.cluster_split > 1:
            busy = p.tiles * p.cluster_split * ctas
            assert busy >= 48, (N, K, p.bn, p.cta_pair, p.cluster_split)
        else:
            assert p.splits > 1 and p.dp_tiles == 0
            assert p.sk_items * ctas >= 74, (N, K, p.bn, p.cta_pair, p.splits)


def test_unaligned_pitch_goes_to_cuda_core_kernel(pkg):
    assert pkg.plan_bf16(0, 0, 100, 250, 136, 148).bn == 0
    assert pkg.plan_bf16(0, 0, 100, 256, 130, 148).bn == 0
    assert pkg.plan_bf16(0, 0, 101, 256, 136, 148).bn != 0  # M needs no alignment


def test_plan_rejects_bad_arguments(pkg):
    for args in ((3, 0, 8, 8, 8, 148), (0, 0, 0, 8, 8, 148), (0, 0, 8, -1, 8, 148), (0, 0, 8, 8, 8, 0)):
        with pytest.raises(pkg.LinearError):
            pkg.plan_bf16(*args)


def test_plan_for_a_share_of_the_sms(pkg):
    """matmul_backward plans its two products for complementary shares of the GPU: every plan must fit its share."""
    for sms in (8, 32, 48, 64, 84, 100, 116, 140):
        for which in (1, 2):
            for N, K in ((768, 768), (256, 768), (2048, 768), (768, 2048), (32000, 768)):
                p = pkg.plan_bf16(which, which == 2, 8192, N, K, sms)
                ctas = 2 if p.cta_pair else 1
                assert p.est_ns > 0
                if p.cluster_split > 1:
                    assert p.tiles * p.cluster_split * ctas <= sms, (sms, which, N, K)
                elif p.splits > 1:
                    assert p.sk_items <= sms // ctas, (sms, which, N, K)


def test_estimate_grows_when_sms_are_taken_away(pkg):
    for which in (0, 1, 2):
        for N, K in ((768, 768), (2048, 768), (32000, 768)):
            full = pkg.plan_bf16(which, which == 2, 8192, N, K, 148).est_ns
            third = pkg.plan_bf16(which, which == 2, 8192, N, K, 48).est_ns
            assert third > full, (which, N, K, full, third)


@pytest.mark.parametrize("which", [0, 1, 2])
def test_grouped_plan_never_lets_a_tile_straddle_two_products(pkg, which):
    """Column-concatenated groups (forward, weight gradient): the tile width divides every member's width; the input
    gradient (products concatenated along the contraction) is planned like one product of the summed width; widths
    that are not multiples of 64 fall back to single products (bn = 0)."""
    groups = [(768, 256, 256), (2048, 2048), (1024, 256, 256), (128, 64, 192), (4096, 4096, 4096), (64, 64)]
    for M, Ns in itertools.product([512, 8192, 16384], groups):
        K = 768
        p = pkg.plan_grouped_bf16(which, M, list(Ns), K, 148)
        assert p.bn in (64, 128, 192, 256)
        total = sum(Ns)
        rows = 256 if p.cta_pair else 128
        if which == 1:   # dX = sum_i dY_i W_i^T: output M x K, contraction = the summed widths
            assert p.tiles == -(-M // rows) * -(-K // p.bn)
        else:
            assert all(n % p.bn == 0 for n in Ns), (Ns, p.bn)
            out_rows = M if which == 0 else K
            assert p.tiles == -(-out_rows // rows) * (total // p.bn)
    assert pkg.plan_grouped_bf16(which, 1024, [72, 136], 264, 148).bn == 0      # not multiples of 64
    assert pkg.plan_grouped_bf16(which, 1024, [768], 768, 148).bn == 0          # a group of one is a single product
    with pytest.raises(pkg.LinearError):
        pkg.plan_grouped_bf16(which, 1024, [768, 0], 768, 148)
