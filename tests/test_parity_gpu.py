"""GPU parity: every workload type through the C API against the CPU oracle
on the same seeded inputs (sizes the oracle finishes in seconds)."""
import numpy as np
import pytest

from onednn_b200 import workloads as W
from onednn_b200.runner import run_problem
from oracle import oracle as O
from util import assert_parity

pytestmark = pytest.mark.gpu

CASES = {
    "int8_zp_s32_full": lambda: W.int8_zp(256, 1024, 1024),
    "int8_zp_f32_per_n": lambda: W.int8_zp(256, 1024, 1024, per_n_scales=True),
    "int8_zp_ragged": lambda: W.int8_zp(37, 200, 77),
    "fp8_small": lambda: W.fp8_prefill(96, 512, 384),
    "fp8_ragged": lambda: W.fp8_prefill(33, 136, 72),
    "int4_m1": lambda: W.int4_decode(1, 1024, 512),
    "int4_m8": lambda: W.int4_decode(8, 1024, 512),
    "int4_m32": lambda: W.int4_decode(32, 512, 256),
    "int4_u4_u8zp": lambda: W.int4_decode(3, 512, 256, wei_dt=W.U4, zp_dt=W.U8),
    "int8w_decode": lambda: W.int4_decode(4, 512, 256, wei_dt=W.S8, zp_dt=W.S8),
    "int8_postops": lambda: W.int8_postops(64, 512, 256),
    "int8_postops_ragged": lambda: W.int8_postops(19, 96, 50),
    "moe_small": lambda: W.moe_grouped(96, 256, 128, 8),
    "moe_empty_groups": lambda: W.moe_grouped(40, 128, 64, 6, sizes=[0, 17, 0, 3, 20, 0]),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_ref_kernels_match_oracle(gpu, name):
    eng, strm = gpu
    p = CASES[name]()
    want = O.run_port(p)
    got, impl = run_problem(p, eng, strm, impl="ref")
    assert impl.startswith("cuda:ref")
    assert_parity(got, want, p.dst_dt, name)


@pytest.mark.parametrize("name", sorted(CASES))
def test_default_impl_matches_oracle(gpu, name):
    eng, strm = gpu
    p = CASES[name]()
    want = O.run_port(p)
    got, impl = run_problem(p, eng, strm)
    assert_parity(got, want, p.dst_dt, "%s via %s" % (name, impl))


def test_grouped_bad_offsets_reports_invalid_arguments(gpu):
    """Non-monotone offsets: the reference returns invalid_arguments
    (ref_grouped_gemm.cpp:164-213); here the status surfaces at wait()."""
    from onednn_b200 import api
    from onednn_b200.runner import Prepared
    eng, strm = gpu
    p = W.moe_grouped(40, 128, 64, 4, sizes=[10, 10, 10, 10])
    p.offsets = np.array([10, 5, 30, 40], np.int32)
    r = Prepared(p, eng).upload()
    r.execute(strm)
    with pytest.raises(api.error) as ei:
        strm.wait()
    assert ei.value.status == api.invalid_arguments
    strm.wait()  # the status word is cleared: the stream stays usable
