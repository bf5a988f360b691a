"""GPU parity at the full sizes of the five benchmark configurations.

The CPU oracle needs minutes to hours for a whole result at these sizes, so it
computes a subset of dst rows (every dst row depends on one src row only):
at least one row of EVERY row tile of the kernels (256 rows; 128 where the
kernel uses that), the rows on both sides of tile boundaries, and eight
seeded random rows; for the grouped problem the first, the last and a middle
row of every non-empty expert.  Those rows of the GPU result are compared
with it under the rules of oracle/parity.py.  For floating-point results the
test also prints how many elements lie beyond the STRICT rule (1 ulp of the
output type, no summation slack) and requires each of them to be explained by
an fp64 evaluation of the same row: the GPU value may not be farther from the
fp64 result than the reference's own value is (plus one ulp).  Two
size-independent properties cover the rest of the result: a second execution
gives the same bits, and equal src rows give equal dst rows."""
import numpy as np
import pytest

from onednn_b200 import workloads as W
from onednn_b200.runner import run_problem
from util import check_rows

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(1500)]


def tile_rows(M, tile, seed, extra=()):
    """One seeded row out of every `tile` rows, both rows of every tile boundary that `extra` names,
    the first and the last row, and eight seeded random rows."""
    r = np.random.Generator(np.random.PCG64(seed))
    rows = [0, M - 1] + list(extra)
    for t0 in range(0, M, tile):
        rows.append(int(r.integers(t0, min(M, t0 + tile))))
    rows += [int(x) for x in r.integers(0, M, 8)]
    return np.unique(np.array([x for x in rows if 0 <= x < M], dtype=np.int64))


def report(what, res):
    print("%s: %d rows, %s; beyond the strict rule: %d (explained by fp64: %s)" % (
        what, res["rows"], res["msg"], res["beyond_strict"], res["strict_misses_explained"]))
    assert res["ok"], (what, res)
    assert res["strict_misses_explained"], (what, res)


def test_cfg1_int8_zp_full_size(gpu):
    eng, strm = gpu
    for per_n in (False, True):  # run A: s32 dst, bit-exact; run B: per-column scales, f32 dst
        p = W.int8_zp(per_n_scales=per_n)  # 256 x 1024 x 1024: the whole result is checked
        got, impl = run_problem(p, eng, strm)
        assert impl == "cuda:tcgen05:int8"
        report("int8 zero-point, %s dst" % ("f32" if per_n else "s32"), check_rows(p, got, np.arange(p.M), False))


def test_cfg2_fp8_prefill_full_size(gpu):
    eng, strm = gpu
    p = W.fp8_prefill()  # 4096 x 4096 x 14336
    # duplicate a src row: equal rows must give equal dst rows
    src = p.src.data.reshape(p.M, p.K)
    src[3001] = src[17]
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:fp8"
    rows = tile_rows(p.M, 256, 1, extra=(17, 255, 256, 2047, 2048, 3001))
    assert len(rows) >= 24
    report("fp8 prefill", check_rows(p, got, rows, True))
    g = got.reshape(p.M, -1)
    assert np.array_equal(g[17], g[3001])
    got2, _ = run_problem(p, eng, strm)
    assert np.array_equal(got, got2)


def test_cfg4_int8_postops_full_size(gpu):
    eng, strm = gpu
    p = W.int8_postops()  # 2048 x 4096 x 11008
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:int8"
    rows = tile_rows(p.M, 256, 2, extra=(1, 255, 256, 1023, 1024))
    assert len(rows) >= 16
    report("int8 post-ops", check_rows(p, got, rows, False))
    got2, _ = run_problem(p, eng, strm)
    assert np.array_equal(got, got2)


@pytest.mark.parametrize("M", [1, 8, 32])
def test_cfg3_int4_decode_full_size(gpu, M):
    eng, strm = gpu
    p = W.int4_decode(M)  # K = 8192, N = 28672, groups of 128
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:woq4"
    rows = np.unique(np.array([0, M // 3, M // 2, M - 1]))
    report("int4 decode M=%d" % M, check_rows(p, got, rows, True))
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
    for g in range(p.groups):  # first, last and a middle row of every non-empty expert
        if ends[g] > begins[g]:
            rows += [begins[g], (begins[g] + ends[g]) // 2, ends[g] - 1]
    rows += [255, 256]  # a row-block boundary inside the largest expert
    report("moe", check_rows(p, got, np.array(rows), True))
    got2, _ = run_problem(p, eng, strm)
    assert np.array_equal(got, got2)
