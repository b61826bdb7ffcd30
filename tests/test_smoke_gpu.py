"""The entry point's smoke run (one small pass over the GEMMs, the fused attention, a grouped launch and the LM-head
statistics, each against its oracle) as a test, so that it cannot rot unnoticed."""
import pytest

pytestmark = pytest.mark.gpu


def test_smoke_entry_point(pkg):
    import __graft_entry__ as ge
    ge.smoke()
