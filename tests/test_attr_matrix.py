"""The attribute combinations of the reference's own matmul test inputs
(tests/attr_matrix.py): on the CPU the C restatement must reproduce the live
reference bit for bit (where the reference library is built); on the GPU every
implementation that accepts a problem must match the C restatement."""
import numpy as np
import pytest

from attr_matrix import CASES
from onednn_b200 import workloads as W
from oracle import oracle as O
from util import assert_parity, summation_slack, summation_slack_grouped


@pytest.mark.parametrize("name", sorted(CASES))
def test_restatement_matches_the_live_reference(name):
    if not O.ref_available():
        pytest.skip("reference library not built")
    p = CASES[name]()
    want, impl, _ = O.run_ref(p, pin_ref=True)
    assert impl.startswith("ref"), impl
    got = O.run_port(p)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), \
        "%s: C restatement differs from %s" % (name, impl)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_every_accepting_implementation_matches(gpu, name):
    from onednn_b200 import api
    from onednn_b200.runner import Prepared
    eng, strm = gpu
    p = CASES[name]()
    want = O.run_port(p)
    r = Prepared(p, eng)
    seen = []
    while True:
        impl = r.pd.impl_info_str()
        seen.append(impl)
        run = Prepared(p, eng, impl=impl).upload()
        run.execute(strm)
        strm.wait()
        slack = None
        if not impl.startswith("cuda:ref") and p.src.dt not in (W.S8, W.U8):
            slack = summation_slack_grouped(p) if p.offsets is not None else summation_slack(p)
        assert_parity(run.download(), want, p.dst_dt, "%s via %s" % (name, impl), slack)
        if not r.pd.next_impl():
            break
    assert seen[-1].startswith("cuda:ref"), seen
