"""The row checker itself (oracle/parity.py), on CPU: oracle rows pass, the fp64 evaluation agrees
with the oracle to within the output type's rounding, and a planted error is found."""
import numpy as np
import pytest

from onednn_b200 import workloads as W
from oracle import oracle as O
from util import check_rows, exact_rows_f64, _ulp16

CASES = {
    "fp8": lambda: W.fp8_prefill(24, 256, 96),
    "int4": lambda: W.int4_decode(6, 512, 128),
    "int4_no_zp_f32": lambda: W.int4_decode(3, 256, 64, with_zp=False, dst_dt=W.F32),
    "moe": lambda: W.moe_grouped(40, 128, 64, 6, sizes=[0, 17, 0, 3, 20, 0]),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_checker_accepts_the_oracle_and_finds_a_planted_error(name):
    p = CASES[name]()
    want = O.run_port(p)
    rows = np.arange(p.M)
    res = check_rows(p, want.copy(), rows, True)
    assert res["ok"] and res["beyond_strict"] == 0 and res["rows"] == p.M
    # the fp64 evaluation and the oracle agree to the rounding of the output type
    exact = exact_rows_f64(p, rows)
    wv = W.to_f32(want.reshape(p.M, -1), p.dst_dt).astype(np.float64)
    unit = 1e-5 * np.abs(wv) + 1e-6 if p.dst_dt == W.F32 else _ulp16(want.reshape(p.M, -1), p.dst_dt)
    assert (np.abs(wv - exact) <= unit + 1e-4 * np.abs(exact).max()).all()
    # a value far from both the reference and the fp64 result is reported
    bad = want.copy().reshape(p.M, -1)
    if p.dst_dt == W.F32:
        bad[p.M - 1, 3] = bad[p.M - 1, 3] * 1.5 + 1.0
    else:
        bad[p.M - 1, 3] = bad[p.M - 1, 3] + 64  # many ulps in the 16-bit pattern
    res = check_rows(p, bad, rows, True)
    assert not res["ok"] and res["beyond_strict"] >= 1 and not res["strict_misses_explained"]
