"""Failure detection of the multi-GPU driver, tested on the host: the ranks of csrc/train_dp.cpp meet on a page of
shared memory before every group of collectives (csrc/rank_rendezvous.h).  A rank that fails, vanishes or never
arrives must make the others leave at that meeting point -- quickly and on their own -- instead of entering a
collective that can never complete.  No GPU is involved: the failures are made on the host."""
import os
import re
import shutil
import subprocess

import pytest

from conftest import ROOT

SRC = os.path.join(ROOT, "tests", "rendezvous_harness.cpp")
INC = os.path.join(ROOT, "llms-from-scratch-cuda_b200", "csrc")


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("g++ not found")
    exe = str(tmp_path_factory.mktemp("rv") / "rendezvous_harness")
    subprocess.run(["g++", "-std=c++17", "-O2", "-I", INC, SRC, "-o", exe], check=True)
    return exe


def _run(exe, *args):
    out = subprocess.run([exe, *[str(a) for a in args]], capture_output=True, text=True, timeout=60)
    ranks = {int(m.group(1)): (int(m.group(2)), int(m.group(3)), float(m.group(4)))
             for m in re.finditer(r"rank (\d+) result (\d+) points (\d+) seconds ([0-9.]+)", out.stdout)}
    failed = int(re.search(r"failed_rank (-?\d+)", out.stdout).group(1))
    return out.returncode, ranks, failed


def test_all_ranks_meet_every_time(harness):
    rc, ranks, failed = _run(harness, "ok", 4, 2000)
    assert rc == 0 and failed == -1
    assert all(r == (0, 2000) for r in [(v[0], v[1]) for v in ranks.values()]) and len(ranks) == 4


@pytest.mark.parametrize("mode", ["fail", "vanish"])
def test_a_rank_that_fails_stops_the_others_between_collectives(harness, mode):
    rc, ranks, failed = _run(harness, mode, 4, 100, 30.0)
    assert rc == 1 and failed == 1
    assert set(ranks) == {0, 2, 3}                       # rank 1 left at point 2 without a report
    for res, points, secs in ranks.values():
        assert res == 1 and points == 2                   # RV_STOPPED, after the two points everybody reached
        assert secs < 5.0                                 # long before the 30 s time limit


def test_a_rank_that_never_arrives_runs_into_the_time_limit(harness):
    rc, ranks, failed = _run(harness, "late", 3, 100, 0.5)
    assert rc == 1 and failed == 1
    assert set(ranks) == {0, 2}
    assert sorted(v[0] for v in ranks.values())[-1] == 2  # somebody's wait ran out (RV_TIMEOUT) ...
    assert all(v[0] in (1, 2) and v[1] == 2 and v[2] < 2.5 for v in ranks.values())  # ... and all left at once
