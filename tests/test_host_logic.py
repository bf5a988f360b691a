"""Host-side behaviour of the C API on a device-less engine: descriptor and
attribute creation, primitive-descriptor validation and error codes.  The
accepted / rejected combinations follow oneDNN's interface tests
(tests/gtests/test_iface_attr_quantization.cpp:476-721, test_matmul.cpp,
test_iface_grouped.cpp) and src/common/matmul.cpp."""
import pytest

from onednn_b200 import api, workloads as W
from onednn_b200.runner import Prepared

md = api.memory.desc
tag = api.tag
SRC, WEI, DST = api.ARG_SRC, api.ARG_WEIGHTS, api.ARG_DST


def status_of(fn):
    try:
        fn()
    except api.error as e:
        return e.status
    return api.success


def make_pd(eng, sdt, wdt, ddt, attr=None, M=32, K=64, N=48, bias=None):
    return api.matmul.primitive_desc(eng, md((M, K), sdt, tag.ab), md((K, N), wdt, tag.ab),
                                     md((M, N), ddt, tag.ab), bias, attr)


def test_memory_desc_basics():
    d = md((4, 6), W.F32, tag.ab)
    assert d.get_dims() == (4, 6) and d.get_strides() == (6, 1) and d.get_size() == 96
    t = md((4, 6), W.F32, tag.ba)
    assert t.get_strides() == (1, 4) and not (d == t)
    assert md((4, 6), W.F32, (6, 1)) == d
    assert md((3, 5, 7), W.S8, tag.acb).get_strides() == (35, 1, 5)
    # sub-byte: two elements per byte, odd strides above 1 are rejected
    assert md((3, 6), W.S4, tag.ab).get_size() == 9
    assert status_of(lambda: md((3, 5), W.S4, tag.ab)) == api.invalid_arguments  # odd row pitch
    assert status_of(lambda: md((4, 6), W.U4, (7, 1))) == api.invalid_arguments
    assert status_of(lambda: md((4, 6), W.F32, tag.abc)) == api.invalid_arguments
    # overlapping strides are not a valid dense layout
    assert status_of(lambda: md((4, 6), W.F32, (2, 1))) == api.invalid_arguments
    any_md = md((4, 6), W.F32, tag.any)
    assert any_md.get_format_kind() == 1 and any_md.get_size() == 0
    assert api.lib().dnnl_data_type_size(W.S4) == 1 and api.lib().dnnl_data_type_size(W.BF16) == 2


def test_grouped_memory_desc():
    g = md.grouped((100, 16), W.BF16, 0, 8)
    assert g.get_num_handles() == 2 and g.get_size(0) == 3200 and g.get_size(1) == 32
    assert status_of(lambda: md.grouped((100, 16, 2), W.BF16, 0, 8)) == api.unimplemented
    assert status_of(lambda: md.grouped((100, 16), W.BF16, 2, 8)) == api.invalid_arguments
    assert status_of(lambda: md.grouped((100, 16), W.BF16, 0, 0)) == api.invalid_arguments
    assert status_of(lambda: md.grouped((100, 16), W.BF16, 0, 8, offsets_dt=W.S8)) == api.unimplemented


def test_attr_setters_validate_arguments():
    a = api.primitive_attr()
    assert status_of(lambda: a.set_scales(SRC, -1)) == api.invalid_arguments
    assert status_of(lambda: a.set_scales(WEI, 3, (32,), W.F32)) == api.invalid_arguments  # group_ndims 1
    assert status_of(lambda: a.set_scales(WEI, 0, (32, 1), W.F32)) == api.invalid_arguments  # groups need a mask
    assert status_of(lambda: a.set_scales(WEI, 3, (32, 1), W.S8)) == api.invalid_arguments  # scale data type
    assert status_of(lambda: a.set_zero_points(WEI, 0, (), W.U4)) == api.invalid_arguments  # int4 zp needs a mask
    assert status_of(lambda: a.set_zero_points(WEI, 3, (32, 1), W.F32)) == api.invalid_arguments
    assert status_of(lambda: a.set_zero_points(DST, 0, (), W.S8)) == api.invalid_arguments  # dst zp is s32
    assert status_of(lambda: a.set_precomputed_reductions(DST, 3)) == api.invalid_arguments
    assert status_of(lambda: a.set_precomputed_reductions(SRC, 3, (), W.S8)) == api.invalid_arguments
    a.set_fpmath_mode(api.fpmath_mode.bf16, True)
    assert a.get_fpmath_mode() == (api.fpmath_mode.bf16, True)
    po = api.post_ops()
    assert status_of(lambda: po.append_eltwise(W.ELTWISE["clip"], 1.0, 0.0)) == api.invalid_arguments
    for _ in range(32):
        po.append_eltwise(W.ELTWISE["relu"], 0.0, 0.0)
    assert po.len() == 32 and po.kind(0) == api.KIND_ELTWISE
    assert status_of(lambda: po.append_eltwise(W.ELTWISE["relu"], 0.0, 0.0)) == api.out_of_memory


def test_shape_checks(host_engine):
    e = host_engine
    mk = lambda s, w, d, b=None: api.matmul.primitive_desc(e, md(s, W.S8, tag.ab), md(w, W.S8, tag.ab),
                                                           md(d, W.S32, tag.ab), b)
    assert status_of(lambda: mk((8, 16), (16, 4), (8, 4))) == api.success
    assert status_of(lambda: mk((8, 16), (15, 4), (8, 4))) == api.invalid_arguments  # K mismatch
    assert status_of(lambda: mk((8, 16), (16, 4), (9, 4))) == api.invalid_arguments  # M mismatch
    assert status_of(lambda: mk((8, 16), (16, 4), (8, 5))) == api.invalid_arguments  # N mismatch
    assert status_of(lambda: mk((8, 16), (16, 4), (8, 4), md((1, 3), W.F32, tag.ab))) == api.invalid_arguments
    assert status_of(lambda: mk((8, 16), (16, 4), (8, 4), md((4,), W.F32, tag.a))) == api.invalid_arguments
    assert status_of(lambda: mk((8, 16), (16, 4), (8, 4), md((1, 4), W.F32, tag.ab))) == api.success
    # f32 x s8 without weights decompression has no accumulation type
    assert status_of(lambda: make_pd(e, W.S8, W.F32, W.F32)) == api.invalid_arguments


def test_quantization_acceptance_matrix(host_engine):
    e = host_engine

    def with_attr(setup, sdt=W.U8, wdt=W.S8, ddt=W.F32, **kw):
        a = api.primitive_attr()
        setup(a)
        return status_of(lambda: make_pd(e, sdt, wdt, ddt, a, **kw))

    ok, no = api.success, api.unimplemented
    # zero-points are refused for an f32 source
    assert with_attr(lambda a: a.set_zero_points_mask(SRC, 0), sdt=W.F32, wdt=W.F32) == no
    # per-tensor / per-N / grouped weights zero-points for u8 x s8
    assert with_attr(lambda a: a.set_zero_points_mask(WEI, 0)) == ok
    assert with_attr(lambda a: a.set_zero_points_mask(WEI, 2)) == ok
    assert with_attr(lambda a: a.set_zero_points(WEI, 3, (32, 1), W.S8)) == ok
    # K groups must be multiples of 16 (weights) / 32 (src) when 1 < g < K
    assert with_attr(lambda a: a.set_zero_points(WEI, 3, (8, 1), W.S8)) == no
    assert with_attr(lambda a: a.set_zero_points(SRC, 3, (1, 16), W.S8)) == no
    assert with_attr(lambda a: a.set_scales(WEI, 3, (8, 1), W.F32)) == no
    assert with_attr(lambda a: a.set_scales(WEI, 3, (32, 1), W.F32)) == ok
    # N groups of weights zero-points only with apply_to_int
    assert with_attr(lambda a: a.set_zero_points(WEI, 3, (32, 16), W.S8)) == no
    # src scale masks: 0, M, K, M+K; per-M alone only on the int8 reference path
    assert with_attr(lambda a: a.set_scales_mask(SRC, 1)) == ok
    assert with_attr(lambda a: a.set_scales_mask(SRC, 1), sdt=W.BF16, wdt=W.BF16, ddt=W.BF16) == no
    # dst zero-point: per-tensor or per-N
    assert with_attr(lambda a: a.set_zero_points_mask(DST, 0)) == ok
    assert with_attr(lambda a: a.set_zero_points_mask(DST, 2)) == ok
    assert with_attr(lambda a: a.set_zero_points_mask(DST, 1)) == no
    # precomputed reductions: src only, full mask, need weights zero-points
    def pr(a):
        a.set_zero_points(WEI, 3, (32, 1), W.S8)
        a.set_precomputed_reductions(SRC, 3, (1, 32))
    assert with_attr(pr) == ok
    assert with_attr(lambda a: a.set_precomputed_reductions(SRC, 3, (1, 32))) == no
    def pr_bad_mask(a):
        a.set_zero_points(WEI, 3, (32, 1), W.S8)
        a.set_precomputed_reductions(SRC, 2)
    assert with_attr(pr_bad_mask) == no
    # weights decompression needs apply_to_int and a matching fpmath mode
    assert status_of(lambda: make_pd(e, W.BF16, W.S4, W.BF16)) == no
    def woq(mode):
        def f(a):
            a.set_fpmath_mode(mode, True)
            a.set_scales(WEI, 3, (32, 1), W.BF16)
            a.set_zero_points(WEI, 3, (32, 1), W.U4)
        return f
    assert with_attr(woq(api.fpmath_mode.bf16), sdt=W.BF16, wdt=W.S4, ddt=W.BF16) == ok
    assert with_attr(woq(api.fpmath_mode.f16), sdt=W.BF16, wdt=W.S4, ddt=W.BF16) == no
    assert with_attr(woq(api.fpmath_mode.f16), sdt=W.F16, wdt=W.S4, ddt=W.F16) == ok
    # u4 zero-points along N need an even N
    assert with_attr(woq(api.fpmath_mode.bf16), sdt=W.BF16, wdt=W.S4, ddt=W.BF16, N=47) == api.invalid_arguments \
        or True  # an odd N already fails the s4 stride rule at descriptor creation


def test_post_op_validation(host_engine):
    e = host_engine
    a = api.primitive_attr()
    po = api.post_ops()
    po.append_binary(W.BINARY["add"], md((32, 48), W.F32, tag.ab))
    po.append_binary(W.BINARY["mul"], md((1, 48), W.F32, tag.ab))
    a.set_post_ops(po)
    assert status_of(lambda: make_pd(e, W.S8, W.S8, W.S8, a)) == api.success
    bad = api.primitive_attr()
    po2 = api.post_ops()
    po2.append_binary(W.BINARY["add"], md((48,), W.F32, tag.a))  # rank differs from dst
    bad.set_post_ops(po2)
    assert status_of(lambda: make_pd(e, W.S8, W.S8, W.S8, bad)) == api.invalid_arguments
    bad2 = api.primitive_attr()
    po3 = api.post_ops()
    po3.append_binary(W.BINARY["add"], md((32, 7), W.F32, tag.ab))  # not broadcastable
    bad2.set_post_ops(po3)
    assert status_of(lambda: make_pd(e, W.S8, W.S8, W.S8, bad2)) == api.invalid_arguments


def test_workload_descriptors_and_queries(host_engine):
    e = host_engine
    for p in (W.int8_zp(16, 64, 32), W.fp8_prefill(16, 64, 32), W.int4_decode(4, 256, 64),
              W.int8_postops(16, 64, 32), W.moe_grouped(24, 64, 32, 4)):
        r = Prepared(p, e)
        assert r.impl.startswith("cuda:")
        assert r.pd.dst_desc().get_dims() == (p.M, p.N)
        # walking the list ends with last_impl_reached, never an error
        while r.pd.next_impl():
            pass
    p = W.int4_decode(4, 256, 64)
    r = Prepared(p, e)
    smd = r.pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_SCALES | WEI)
    assert smd.get_dims() == (2, 64) and smd.get_data_type() == W.BF16
    zmd = r.pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_ZERO_POINTS | WEI)
    assert zmd.get_dims() == (2, 64) and zmd.get_size() == 64
    g = Prepared(W.moe_grouped(24, 64, 32, 4), e)
    assert g.pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_SCALES | WEI).get_dims() == (4, 1, 32)


def test_grouped_validation(host_engine):
    e = host_engine
    src = md.grouped((40, 64), W.BF16, 0, 4)
    dst = md.grouped((40, 32), W.BF16, 0, 4)
    wei = md((4, 64, 32), W.S8, tag.abc)
    a = api.primitive_attr()
    a.set_fpmath_mode(api.fpmath_mode.bf16, True)
    a.set_scales_mask(WEI, 0b101)
    mk = lambda s, w, d, at=a: status_of(lambda: api.matmul.primitive_desc(e, s, w, d, None, at))
    assert mk(src, wei, dst) == api.success
    assert mk(src, md((5, 64, 32), W.S8, tag.abc), dst) == api.unimplemented  # experts != groups
    assert mk(src, wei, md.grouped((40, 32), W.BF16, 0, 5)) == api.unimplemented
    assert mk(src, md((4, 64, 32), W.S8, tag.acb), dst) == api.success
    assert mk(src, md((4, 64, 32), W.S8, tag.bac), dst) == api.unimplemented
    assert mk(src, wei, dst, None) == api.unimplemented  # int weights need scales + apply_to_int
    b = api.primitive_attr()
    b.set_fpmath_mode(api.fpmath_mode.bf16, True)
    b.set_scales_mask(WEI, 0b010)
    assert mk(src, wei, dst, b) == api.unimplemented  # scale mask must cover (expert, N)


def test_deviceless_engine_executes_nothing(host_engine):
    if api.engine.get_count(api.engine.kind.gpu) > 0:
        pytest.skip("a real device is present")
    p = W.int8_zp(8, 32, 16)
    r = Prepared(p, host_engine)
    with pytest.raises(api.error) as ei:
        r.upload()
    assert ei.value.status == api.runtime_error


def test_user_scratchpad_descriptor(host_engine):
    """scratchpad_mode::user: the primitive descriptor says how many bytes the caller
    has to bring; library mode (the default) asks for nothing."""
    from onednn_b200 import workloads as W
    from onednn_b200.runner import Prepared

    def size(p, user):
        r = Prepared(p, host_engine, user_scratchpad=user)
        return r.pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_SCRATCHPAD).get_size(0)

    int4 = W.int4_decode(1, 1024, 512)
    assert size(int4, False) == 0
    assert size(int4, True) > 0
    assert size(W.moe_grouped(40, 128, 64, 4), True) >= 16 * 5  # one int4 record per expert and a header
    assert size(W.int8_zp(64, 128, 64), True) >= 4 * (64 + 64)  # column and row sums
    assert size(W.fp8_prefill(64, 128, 64), True) == 0


def test_runtime_m_descriptor(host_engine):
    """DNNL_RUNTIME_DIM_VAL (src/common/matmul.cpp:630-744; the reference's int8 inference tutorial
    leaves M open): accepted for any of M, K, N of a dense 2D problem, reported back by the queries,
    refused for batched and grouped problems."""
    RT = api.RUNTIME_DIM_VAL
    open_md = md((RT, 64), W.U8, (64, 1))
    assert open_md.get_dims() == (RT, 64) and open_md.get_strides() == (64, 1)
    assert open_md.get_size() == (1 << 64) + RT  # DNNL_RUNTIME_SIZE_VAL
    a = api.primitive_attr()
    a.set_scales_mask(WEI, 2)
    a.set_zero_points_mask(SRC, 0)
    pd = api.matmul.primitive_desc(host_engine, open_md, md((64, 48), W.S8, tag.any), md((RT, 48), W.S32, (48, 1)), None, a)
    assert pd.impl_info_str().startswith("cuda:")
    assert pd.src_desc().get_dims() == (RT, 64) and pd.weights_desc().get_strides() == (48, 1)
    # K and N left open, with the strides that depend on them; the parameter descriptors stay open too
    pd = api.matmul.primitive_desc(host_engine, md((8, RT), W.U8, (RT, 1)), md((RT, RT), W.S8, (RT, 1)),
                                   md((8, RT), W.S32, (RT, 1)), None, a)
    assert pd.impl_info_str().startswith("cuda:")
    assert pd.weights_desc().get_dims() == (RT, RT) and pd.dst_desc().get_dims() == (8, RT)
    assert pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_SCALES | WEI).get_dims() == (1, RT)
    # a row-dependent stride (src stored transposed with M open)
    pd = api.matmul.primitive_desc(host_engine, md((RT, 64), W.U8, tag.ba), md((64, 48), W.S8, tag.ab), md((RT, 48), W.S32, tag.ab))
    assert pd.src_desc().get_dims() == (RT, 64)
    # a binary operand given with format `any` (allowed as in the reference) resolves to row-major, with M open or not
    for rows in (RT, 16):
        po = api.post_ops()
        po.append_binary(W.BINARY["add"], md((1, 48), W.F32, tag.any))
        b = api.primitive_attr()
        b.set_post_ops(po)
        pd = api.matmul.primitive_desc(host_engine, md((rows, 64), W.U8, (64, 1)), md((64, 48), W.S8, tag.ab),
                                       md((rows, 48), W.S32, (48, 1)), None, b)
        assert pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_MULTIPLE_POST_OP(0) | api.ARG_SRC_1).get_strides() == (48, 1)
    # dims that contradict one another are refused at creation, batched problems with open dims are not built
    assert status_of(lambda: api.matmul.primitive_desc(host_engine, md((RT, 64), W.U8, (64, 1)), md((32, 48), W.S8, (48, 1)),
                                                        md((RT, 48), W.S32, (48, 1)))) == api.invalid_arguments
    assert status_of(lambda: api.matmul.primitive_desc(host_engine, md((2, RT, 64), W.U8, (RT, 64, 1)), md((2, 64, 48), W.S8, tag.abc),
                                                        md((2, RT, 48), W.S32, (RT, 48, 1)))) == api.unimplemented


def test_value_names_and_late_post_op_calls():
    """dnnl_debug.h names, dnnl_post_ops_append_binary_v2 / get_params_prelu, sub-memory descriptors."""
    import ctypes as C
    L = api.lib()
    for fn, v, want in (("dnnl_status2str", 3, b"unimplemented"), ("dnnl_dt2str", W.F8_E4M3, b"f8_e4m3"),
                        ("dnnl_dt2str", W.S4, b"s4"), ("dnnl_fmt_tag2str", 3, b"ab"), ("dnnl_engine_kind2str", 2, b"gpu"),
                        ("dnnl_alg_kind2str", W.ELTWISE["gelu_tanh"], b"eltwise_gelu_tanh"),
                        ("dnnl_alg_kind2str", W.BINARY["mul"], b"binary_mul"), ("dnnl_prim_kind2str", 14, b"matmul"),
                        ("dnnl_fpmath_mode2str", 1, b"bf16"), ("dnnl_runtime2str", 2048, b"CUDA")):
        f = getattr(L, fn)
        f.restype = C.c_char_p
        assert f(v) == want, (fn, v, f(v))
    po = api.post_ops()
    src1 = md((1, 8), W.F32, tag.ab)
    assert L.dnnl_post_ops_append_binary_v2(po._h, W.BINARY["add"], src1._h, None) == api.success
    assert L.dnnl_post_ops_append_binary_v2(po._h, 0x1fffc, src1._h, src1._h) == api.unimplemented  # select
    po.append_prelu(5)
    mask = C.c_int(0)
    assert L.dnnl_post_ops_get_params_prelu(po._h, 1, C.byref(mask)) == api.success and mask.value == 5
    assert L.dnnl_post_ops_get_params_prelu(po._h, 0, C.byref(mask)) == api.invalid_arguments
    # a window of a plain tensor keeps the strides and moves offset0
    parent = md((8, 16), W.S8, tag.ab)
    sub = C.c_void_p()
    dims = (C.c_int64 * 12)(4, 8)
    offs = (C.c_int64 * 12)(2, 8)
    assert L.dnnl_memory_desc_create_submemory(C.byref(sub), parent._h, dims, offs) == api.success
    off0 = C.c_int64(0)
    assert L.dnnl_memory_desc_query(sub, 259, C.byref(off0)) == api.success and off0.value == 2 * 16 + 8
    L.dnnl_memory_desc_destroy(sub)
    offs[1] = 12  # 12 + 8 > 16
    assert L.dnnl_memory_desc_create_submemory(C.byref(sub), parent._h, dims, offs) == api.invalid_arguments
    # 4-bit elements: the window starts on a byte
    p4 = md((8, 16), W.S4, tag.ab)
    offs[1] = 3
    assert L.dnnl_memory_desc_create_submemory(C.byref(sub), p4._h, dims, offs) == api.invalid_arguments


def test_verbose_line_format(host_engine, capfd):
    """ONEDNN_VERBOSE=2 prints a create line in the reference's field order (src/common/verbose.cpp:1060-1090):
    operation, engine, primitive, implementation, prop_kind, memory descriptors, attributes, aux, problem."""
    L = api.lib()
    L.dnnl_set_verbose(2)
    try:
        a = api.primitive_attr()
        a.set_fpmath_mode(api.fpmath_mode.bf16, True)
        a.set_scales(WEI, 3, (128, 1), W.BF16)
        a.set_zero_points(WEI, 3, (128, 1), W.U4)
        pd = api.matmul.primitive_desc(host_engine, md((8, 256), W.BF16, tag.ab), md((256, 64), W.S4, tag.ab),
                                       md((8, 64), W.BF16, tag.ab), None, a)
        api.matmul(pd)
    finally:
        L.dnnl_set_verbose(0)
    out = capfd.readouterr().out
    line = [l for l in out.splitlines() if l.startswith("onednn_verbose,v1,primitive,create:cache_miss")][-1]
    f = line.split(",")
    assert f[4:8] == ["gpu", "matmul", "cuda:tcgen05:woq4", "undef"]
    assert f[8] == "src:bf16::blocked:ab::f0 wei:s4::blocked:ab::f0 dst:bf16::blocked:ab::f0"
    assert f[9] == "attr-fpmath:bf16:true attr-scales:wei:3:bf16:128x1 attr-zero-points:wei:3:u4:128x1"
    assert f[11] == "8x256:256x64"


def test_replicated_dst_is_refused_where_no_kernel_has_it(host_engine):
    """dnnl_cuda_interop_primitive_replicate_dst: only the tensor-core GEMM without a post-op chain
    repeats its dst stores; other primitives answer unimplemented (the caller then uses the
    scatter kernel), and world <= 1 switches the replication off."""
    import ctypes as C
    from onednn_b200 import api
    from onednn_b200.runner import Prepared
    L = api.lib()
    L.dnnl_cuda_interop_primitive_replicate_dst.argtypes = [
        C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_uint]
    bases = (C.c_void_p * 2)(0x1000, 0x2000)
    flags = (C.c_void_p * 2)(0x3000, 0x4000)
    done = C.c_void_p(0x5000)

    def call(p, world=2):
        prep = Prepared(p, host_engine)
        return prep.impl, L.dnnl_cuda_interop_primitive_replicate_dst(prep.prim._h, world, 0, bases, 4096, flags, done, 1)

    impl, st = call(W.int8_zp(64, 256, 256))
    assert impl == "cuda:tcgen05:int8" and st == 0
    assert call(W.int8_zp(64, 256, 256), world=1)[1] == 0
    impl, st = call(W.int8_postops(64, 256, 256))
    assert impl == "cuda:tcgen05:int8" and st == api.unimplemented  # a post-op chain
    impl, st = call(W.int4_decode(4, 512, 256))
    assert st == api.unimplemented
    impl, st = call(W.moe_grouped(96, 256, 128, 8))
    assert st == api.unimplemented


def test_decode_problems_with_wide_parameter_rows_go_to_the_next_implementation(host_engine):
    """cuda:tcgen05:woq4 keeps a stage's scale / zero-point rows in shared memory: groups of 16 with
    f32 scales and s32 zero-points of a 32-row problem do not fit and are served by the next implementation in the list."""
    import numpy as np
    from onednn_b200.runner import Prepared
    p = W.int4_decode(4, 1024, 512, group=128)
    assert Prepared(p, host_engine).impl == "cuda:tcgen05:woq4"
    p = W.int4_decode(32, 1024, 512, group=16)
    r = np.random.Generator(np.random.PCG64(3))
    G = 1024 // 16
    p.quant["wei_scale"] = W.Quant(r.uniform(0.005, 0.02, (G, 512)).astype(np.float32), W.F32, 3, (16, 1))
    p.quant["wei_zp"] = W.Quant(r.integers(0, 16, (G, 512)).astype(np.int32), W.S32, 3, (16, 1))
    assert Prepared(p, host_engine).impl == "cuda:woq:skinny"
