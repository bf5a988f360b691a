"""dnnl::reorder between plain layouts (tests/reorder_cases.py).

CPU: the C restatement reproduces, bit for bit, the fixtures the reference
library produced (tests/golden/reorder.npz, made by make_golden_reorder.py)
and, where that library is built, its live output.  GPU: the CUDA library
reproduces the restatement bit for bit (element-wise work, one rounding
sequence: no tolerance)."""
import os

import numpy as np
import pytest

from onednn_b200 import workloads as W
from oracle import oracle as O
from reorder_cases import CASES

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = np.load(os.path.join(HERE, "golden", "reorder.npz"))


@pytest.mark.parametrize("name", sorted(CASES))
def test_restatement_matches_the_fixture(name):
    got = O.run_port_reorder(CASES[name]())
    assert np.array_equal(got.view(np.uint8).reshape(-1), GOLDEN[name]), \
        "%s differs from %s" % (name, bytes(GOLDEN[name + "__impl"]).decode())


@pytest.mark.parametrize("name", sorted(CASES))
def test_restatement_matches_the_live_reference(name):
    if not O.ref_available():
        pytest.skip("reference library not built")
    r = CASES[name]()
    want, impl = O.run_ref_reorder(r)
    got = O.run_port_reorder(r)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), "%s: differs from %s" % (name, impl)


def test_restatement_rejects_what_the_reference_has_no_implementation_of():
    r = CASES["compress_f32_to_s4"]()
    r.quant["dst_scale"] = W.Quant(np.array([0.5], np.float32), W.F32, 0)
    with pytest.raises(RuntimeError):
        O.run_port_reorder(r)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_reorder_matches_oracle(gpu, name):
    from onednn_b200.runner import run_reorder
    eng, strm = gpu
    r = CASES[name]()
    want = O.run_port_reorder(r)
    got, impl = run_reorder(r, eng, strm)
    assert impl == "cuda:ref:reorder"
    n = want.view(np.uint8).size
    assert np.array_equal(got.view(np.uint8).reshape(-1)[:n], want.view(np.uint8).reshape(-1)), name


@pytest.mark.gpu
def test_cuda_reorder_feeds_the_matmul(gpu):
    """The canonical flow: quantize f32 weights to s8 with per-column scales by a reorder, then
    run the int8 matmul with the same scales; compared with the oracle run on the oracle's
    own quantized weights."""
    from onednn_b200.runner import run_problem, run_reorder
    eng, strm = gpu
    r = np.random.Generator(np.random.PCG64(77))
    K, N, M = 256, 128, 64
    wf = W.QTensor((r.standard_normal((K, N)) * 0.05).astype(np.float32), W.F32, (K, N))
    sc = (np.abs(wf.data).max(axis=0, keepdims=True) / 127.0).astype(np.float32)
    ro = W.Reorder("quantize", wf, W.S8, quant={"dst_scale": W.Quant(sc, W.F32, 2)})
    wq, _ = run_reorder(ro, eng, strm)
    assert np.array_equal(wq, O.run_port_reorder(ro))
    p = W.int8_zp(M, K, N, dst_dt=W.F32)
    p.wei = W.QTensor(wq.reshape(K, N).copy(), W.S8, (K, N))
    p.quant = {"wei_scale": W.Quant(sc, W.F32, 2)}
    got, impl = run_problem(p, eng, strm)
    want = O.run_port(p)
    assert impl.startswith("cuda:tcgen05:int8"), impl
    assert np.allclose(got, want, rtol=1e-5, atol=0)


@pytest.mark.gpu
def test_cuda_reorder_feeds_the_fp8_matmul(gpu):
    """f32 activations and weights quantized to e4m3 by reorders (common dst scales), then the fp8
    matmul with the same scales; the oracle runs on the oracle's own quantized tensors."""
    from onednn_b200.runner import run_problem, run_reorder
    eng, strm = gpu
    r = np.random.Generator(np.random.PCG64(78))
    M, K, N = 64, 256, 128
    p = W.fp8_prefill(M, K, N)
    quantized = {}
    for name, dims, scale in (("src", (M, K), 0.02), ("wei", (K, N), 0.01)):
        x = W.QTensor(r.standard_normal(dims).astype(np.float32), W.F32, dims)
        ro = W.Reorder(name, x, W.F8_E4M3, quant={"dst_scale": W.Quant(np.array([scale], np.float32), W.F32, 0)})
        q, impl = run_reorder(ro, eng, strm)
        assert impl == "cuda:ref:reorder"
        assert np.array_equal(q, O.run_port_reorder(ro)), name
        quantized[name] = W.QTensor(q.reshape(dims).copy(), W.F8_E4M3, dims)
    p.src, p.wei = quantized["src"], quantized["wei"]
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:fp8", impl
    from util import assert_parity, summation_slack
    assert_parity(got, O.run_port(p), p.dst_dt, "fp8 matmul on reorder-quantized tensors", summation_slack(p))


def test_reorder_descriptor_checks(host_engine):
    """Creation-time validation on a device-less engine: the error codes of
    src/common/reorder.cpp:67-150 and the combinations the implementation list covers."""
    import ctypes as C
    from onednn_b200 import api
    md, tag, eng = api.memory.desc, api.tag, host_engine

    def status(src_md, dst_md, attr=None):
        try:
            api.reorder.primitive_desc(eng, src_md, eng, dst_md, attr)
        except api.error as e:
            return e.status
        return api.success

    def attr_with(fn):
        a = api.primitive_attr()
        fn(a)
        return a

    f32, s8 = md((8, 16), W.F32, tag.ab), md((8, 16), W.S8, tag.ab)
    h = C.c_void_p()
    assert api.lib().dnnl_reorder_primitive_desc_create(C.byref(h), None, None, None, None, None) == api.invalid_arguments
    pd = api.reorder.primitive_desc(eng, f32, eng, s8, attr_with(lambda a: a.set_scales(api.ARG_DST, 2, (), W.F32)))
    assert pd.impl_info_str() == "cuda:ref:reorder" and not pd.next_impl()
    assert pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_SCALES | api.ARG_DST).get_dims() == (1, 16)
    assert pd.src_desc() == f32 and pd.dst_desc() == s8
    # dims must agree; format_tag::any is not a layout to reorder into
    assert status(f32, md((8, 12), W.S8, tag.ab)) == api.invalid_arguments
    assert status(f32, md((8, 16), W.S8, tag.any)) == api.invalid_arguments
    # zero-points only on integer tensors; a scale for s4 sources needs a mask; dst scales take no groups
    assert status(f32, s8, attr_with(lambda a: a.set_zero_points(api.ARG_SRC, 0, (), W.S32))) == api.invalid_arguments
    assert status(s8, f32, attr_with(lambda a: a.set_zero_points(api.ARG_SRC, 0, (), W.S32))) == api.success
    s4 = md((8, 16), W.S4, tag.ab)
    assert status(s4, f32, attr_with(lambda a: a.set_scales(api.ARG_SRC, 0, (), W.F32))) == api.invalid_arguments
    assert status(s4, f32, attr_with(lambda a: a.set_scales(api.ARG_SRC, 3, (4, 1), W.BF16))) == api.success
    assert status(s4, f32, attr_with(lambda a: a.set_scales(api.ARG_SRC, 3, (3, 1), W.BF16))) == api.invalid_arguments
    assert status(f32, s8, attr_with(lambda a: a.set_scales(api.ARG_DST, 3, (4, 1), W.F32))) == api.invalid_arguments
    # outside the implementation list: 4-bit targets with arithmetic or from other types, 4-bit to integers
    assert status(f32, s4) == api.success
    assert status(f32, s4, attr_with(lambda a: a.set_scales(api.ARG_DST, 0, (), W.F32))) == api.unimplemented
    assert status(md((8, 16), W.BF16, tag.ab), s4) == api.unimplemented
    assert status(s4, s8) == api.unimplemented
    # a 4-bit tensor whose rows do not end on a byte has no plain descriptor in the first place
    with pytest.raises(api.error):
        md((8, 15), W.S4, tag.ab)
