"""Pins the CPU oracle (the C restatement in oracle/qmm_oracle.c) to outputs
of the unmodified reference library: the committed fixtures in
tests/golden/golden.npz (made by tests/golden/make_golden.py), and - when a
build of the reference is present under oracle/_ref - the reference itself on
further seeded problems.  The oracle must reproduce them bit for bit."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

from cases import CASES  # noqa: E402
from onednn_b200 import workloads as W  # noqa: E402
from oracle import oracle as O  # noqa: E402

GOLDEN = np.load(os.path.join(HERE, "golden", "golden.npz"))


@pytest.mark.parametrize("name", sorted(CASES))
def test_port_reproduces_reference_fixture(name):
    p = CASES[name]()
    got = O.run_port(p).view(np.uint8).reshape(-1)
    want = GOLDEN[name]
    assert got.shape == want.shape
    assert np.array_equal(got, want), "%d of %d bytes differ" % (int((got != want).sum()), want.size)
    assert GOLDEN[name + "__impl"].tobytes().decode().startswith("ref")


def test_row_subset_equals_full_rows():
    p = W.int8_postops(40, 256, 72)
    full = O.run_port(p)
    rows = np.array([0, 7, 39])
    sub = O.run_port(p, rows=rows)
    assert np.array_equal(sub[rows], full[rows])
    assert np.array_equal(O.run_port(p.take_rows(rows)), full[rows])


def test_grouped_offsets_validation():
    p = W.moe_grouped(20, 32, 16, 3, sizes=[5, 5, 10])
    p.offsets = np.array([5, 3, 20], np.int32)
    with pytest.raises(RuntimeError):
        O.run_port(p)


REF_CASES = {
    "int8_zp": lambda: W.int8_zp(31, 96, 50, seed=1),
    "int8_zp_scaled": lambda: W.int8_zp(17, 64, 33, per_n_scales=True, seed=2),
    "fp8": lambda: W.fp8_prefill(9, 80, 24, seed=3),
    "int4": lambda: W.int4_decode(4, 384, 96, seed=4),
    "int4_g32": lambda: W.int4_decode(2, 128, 32, group=32, seed=5),
    "postops": lambda: W.int8_postops(13, 64, 40, seed=6),
    "moe": lambda: W.moe_grouped(50, 64, 24, 7, seed=7),
}


@pytest.mark.skipif(not O.ref_available(), reason="no build of the reference under oracle/_ref")
@pytest.mark.parametrize("name", sorted(REF_CASES))
def test_port_matches_reference_library(name):
    p = REF_CASES[name]()
    want, impl, _ = O.run_ref(p, pin_ref=True)
    assert impl.startswith("ref")
    got = O.run_port(p)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
