"""GPU parity at the full sizes of the five benchmark configurations.

The CPU oracle needs minutes to hours for a whole result at these sizes, so it
computes a seeded subset of dst rows (every dst row depends on one src row
only: first and last rows, tile boundaries, first/last row of experts) and
those rows of the GPU result are compared with it.  Two size-independent
properties cover the rest of the result: a second execution gives the same
bits, and rows of the src that are equal give equal dst rows."""
import numpy as np
import pytest

from onednn_b200 import workloads as W
from onednn_b200.runner import run_problem
from oracle import oracle as O
from util import assert_parity, summation_slack

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(900)]


def _check_rows(p, got, rows, slack_rows=None, what=""):
    rows = np.unique(np.asarray(rows, dtype=np.int64))
    want = O.run_port(p, rows=rows)
    g = got.reshape(p.M, -1)[rows]
    w = want.reshape(p.M, -1)[rows]
    assert_parity(g, w, p.dst_dt, what, slack_rows)


def _dense_slack(p, rows):
    return summation_slack(p.take_rows(rows))


def test_cfg2_fp8_prefill_full_size(gpu):
    eng, strm = gpu
    p = W.fp8_prefill()  # 4096 x 4096 x 14336
    # duplicate a src row: equal rows must give equal dst rows
    src = p.src.data.reshape(p.M, p.K)
    src[3001] = src[17]
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:fp8"
    rows = np.array([0, 17, 255, 256, 2047, 3001, 4095])
    _check_rows(p, got, rows, _dense_slack(p, np.unique(rows)), "fp8 prefill, %d rows" % len(rows))
    g = got.reshape(p.M, -1)
    assert np.array_equal(g[17], g[3001])
    got2, _ = run_problem(p, eng, strm)
    assert np.array_equal(got, got2)


def test_cfg4_int8_postops_full_size(gpu):
    eng, strm = gpu
    p = W.int8_postops()  # 2048 x 4096 x 11008
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:int8"
    rows = np.array([0, 1, 255, 256, 1023, 2047])
    _check_rows(p, got, rows, None, "int8 post-ops, %d rows" % len(rows))
    got2, _ = run_problem(p, eng, strm)
    assert np.array_equal(got, got2)


@pytest.mark.parametrize("M", [1, 8, 32])
def test_cfg3_int4_decode_full_size(gpu, M):
    eng, strm = gpu
    p = W.int4_decode(M)  # K = 8192, N = 28672, groups of 128
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:woq4"
    rows = np.unique(np.array([0, M // 2, M - 1]))
    _check_rows(p, got, rows, _dense_slack(p, rows), "int4 decode M=%d" % M)
    got2, _ = run_problem(p, eng, strm)
    assert np.array_equal(got, got2)


def test_cfg5_moe_full_size(gpu):
    eng, strm = gpu
    p = W.moe_grouped()  # 8192 rows, 64 experts, K = 4096, N = 14336
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:grouped"
    ends = p.offsets.astype(np.int64)
    begins = np.concatenate([[0], ends[:-1]])
    rows = []
    for g in (0, 1, 7, 31, 63):  # first and last row of a few experts, and a row-block boundary
        if ends[g] > begins[g]:
            rows += [begins[g], ends[g] - 1]
    rows += [255, 256]
    rows = np.unique(np.array(rows))
    # summation slack of these rows only (the whole-problem helper would widen 3.8 GB of weights)
    src = W.to_f32(p.src.data.reshape(p.M, p.K)[rows], p.src.dt).astype(np.float64)
    sc = np.abs(p.quant["wei_scale"].data.reshape(p.groups, p.N).astype(np.float64))
    slack = np.zeros((len(rows), p.N))
    for i, r in enumerate(rows):
        g = int(np.searchsorted(ends, r, side="right"))
        slack[i] = (np.abs(src[i]) @ np.abs(p.wei.data[g].astype(np.float32)).astype(np.float64)) * sc[g]
    _check_rows(p, got, rows, 4.0 * 2.0 ** -24 * slack, "moe, %d rows" % len(rows))
