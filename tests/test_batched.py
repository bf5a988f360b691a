"""Batched (ndims > 2) matmul: the reference's broadcast rules for batch dims
(src/common/matmul.cpp:630-744); each matrix of the batch must equal the 2D
problem's result from the oracle."""
import numpy as np
import pytest

from onednn_b200 import workloads as W
from oracle import oracle as O
from util import assert_parity, summation_slack


def _batched_desc(api, eng, B, wei_b, p, attr):
    src_md = api.memory.desc((B, p.M, p.K), p.src.dt, (p.M * p.K, p.K, 1))
    wei_md = api.memory.desc((wei_b, p.K, p.N), p.wei.dt, (p.K * p.N, p.N, 1))
    dst_md = api.memory.desc((B, p.M, p.N), p.dst_dt, (p.M * p.N, p.N, 1))
    bias_md = api.memory.desc((1, 1, p.N), p.bias.dt, (p.N, p.N, 1)) if p.bias is not None else None
    return src_md, wei_md, dst_md, bias_md, api.matmul.primitive_desc(eng, src_md, wei_md, dst_md, bias_md, attr)


def _attr(api, p, nd):
    """The 2D problem's attributes with their masks moved to the last two of nd dims."""
    attr = api.primitive_attr()
    if p.apply_to_int or p.fpmath:
        attr.set_fpmath_mode(p.fpmath, p.apply_to_int)
    arg_of = {"src": api.ARG_SRC, "wei": api.ARG_WEIGHTS, "dst": api.ARG_DST}
    keys = {}
    for name, q in p.quant.items():
        arg = arg_of[name[:3]]
        groups = tuple(q.groups) if tuple(q.groups) != (1, 1) else ()
        mask = q.mask << (nd - 2)
        if name.endswith("scale"):
            attr.set_scales(arg, mask, groups, q.dt)
            keys[name] = api.ARG_ATTR_SCALES | arg
        else:
            attr.set_zero_points(arg, mask, groups, q.dt)
            keys[name] = api.ARG_ATTR_ZERO_POINTS | arg
    return attr, keys


def test_batched_descriptor_rules(host_engine):
    from onednn_b200 import api
    eng = host_engine
    p = W.int8_zp(32, 64, 48)
    attr, _ = _attr(api, p, 3)
    *_, pd = _batched_desc(api, eng, 3, 1, p, attr)
    assert pd.impl_info_str() == "cuda:tcgen05:int8"
    assert tuple(pd.query_md(api.QUERY_DST_MD, 0).get_dims()) == (3, 32, 48)
    # batch dims must match or be 1
    with pytest.raises(api.error):
        _batched_desc(api, eng, 3, 2, p, attr)
    # a parameter that varies along the batch is not built
    bad = api.primitive_attr()
    bad.set_scales(api.ARG_WEIGHTS, 0b101, (), W.F32)
    with pytest.raises(api.error) as ei:
        _batched_desc(api, eng, 3, 3, W.int8_zp(32, 64, 48, per_n_scales=True), bad)
    assert ei.value.status == api.unimplemented


BATCHED = {
    "int8_s32_weights_broadcast": (lambda s: W.int8_zp(70, 256, 192, seed=s), 3, 1),
    "int8_f32_per_n_scales": (lambda s: W.int8_zp(33, 128, 64, per_n_scales=True, seed=s), 2, 2),
    "fp8_bias": (lambda s: W.fp8_prefill(40, 256, 128, seed=s), 2, 1),
    "int4_decode": (lambda s: W.int4_decode(4, 512, 256, seed=s), 3, 3),
}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(BATCHED))
def test_batched_matches_the_2d_oracle(gpu, name):
    from onednn_b200 import api
    eng, strm = gpu
    make, B, wei_b = BATCHED[name]
    ps = [make(100 + b) for b in range(B)]
    p0 = ps[0]
    if wei_b == 1:  # one weight matrix (and its parameters) for the whole batch
        for p in ps[1:]:
            p.wei, p.bias = p0.wei, p0.bias
            for k in p0.quant:
                p.quant[k] = p0.quant[k]
    else:  # per-tensor / per-column parameters are shared by the batch
        for p in ps[1:]:
            p.bias = p0.bias
            for k in p0.quant:
                p.quant[k] = p0.quant[k]
    attr, keys = _attr(api, p0, 3)
    src_md, wei_md, dst_md, bias_md, pd = _batched_desc(api, eng, B, wei_b, p0, attr)
    prim = api.matmul(pd)

    def mem(md, arrays):
        m = api.memory(md, eng)
        m.write(np.concatenate([np.ascontiguousarray(a).view(np.uint8).reshape(-1) for a in arrays]), 0)
        return m

    args = {api.ARG_SRC: mem(src_md, [p.src.data for p in ps]),
            api.ARG_WEIGHTS: mem(wei_md, [p.wei.data for p in ps[:wei_b]]),
            api.ARG_DST: mem(dst_md, [np.zeros(dst_md.get_size(0), np.uint8)])}
    if bias_md is not None:
        args[api.ARG_BIAS] = mem(bias_md, [p0.bias.data])
    for qname, key in keys.items():
        args[key] = mem(pd.query_md(api.QUERY_EXEC_ARG_MD, key), [p0.quant[qname].data])
    prim.execute(strm, args)
    strm.wait()
    got = args[api.ARG_DST].read(np.uint8, 0).view(W.NP_STORAGE[p0.dst_dt]).reshape(B, p0.M, p0.N)
    impl = pd.impl_info_str()
    for b, p in enumerate(ps):
        slack = None if p.src.dt in (W.S8, W.U8) else summation_slack(p)
        assert_parity(got[b], O.run_port(p), p.dst_dt, "%s batch %d via %s" % (name, b, impl), slack)
