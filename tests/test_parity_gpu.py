"""GPU parity: every workload type through the C API against the CPU oracle
on the same seeded inputs (sizes the oracle finishes in seconds)."""
import numpy as np
import pytest

from onednn_b200 import workloads as W
from onednn_b200.runner import run_problem
from oracle import oracle as O
from util import assert_parity, summation_slack, summation_slack_grouped


def slack_for(p, impl):
    """Summation slack only for floating-point sums taken in another order
    than the reference's (every implementation but the cuda:ref kernels)."""
    if impl.startswith("cuda:ref") or p.src.dt in (W.S8, W.U8):
        return None
    return summation_slack_grouped(p) if p.offsets is not None else summation_slack(p)

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
    assert_parity(got, want, p.dst_dt, "%s via %s" % (name, impl), slack_for(p, impl))


def _ba(p):
    """Same problem with the weights stored K-contiguous (format tag `ba`)."""
    w = p.wei.data.reshape(p.K, p.N)
    p.wei = W.QTensor(np.ascontiguousarray(w.T), p.wei.dt, (p.K, p.N), (1, p.K))
    return p


def _wei_zp(p, per_n):
    r = np.random.Generator(np.random.PCG64(3))
    z = r.integers(-5, 6, (1, p.N) if per_n else (1,)).astype(np.int32)
    p.quant["wei_zp"] = W.Quant(z, W.S32, 2 if per_n else 0)
    return p


TC_CASES = {
    "cfg1_s32": lambda: W.int8_zp(256, 1024, 1024),
    "cfg1_f32": lambda: W.int8_zp(256, 1024, 1024, per_n_scales=True),
    "int8_tails": lambda: W.int8_zp(200, 272, 176),
    "int8_one_tile": lambda: W.int8_zp(5, 16, 16),
    "int8_wide": lambda: W.int8_zp(384, 512, 9984),
    "int8_ba": lambda: _ba(W.int8_zp(130, 256, 320)),
    "int8_wzp": lambda: _wei_zp(W.int8_zp(96, 256, 160), False),
    "int8_wzp_per_n": lambda: _wei_zp(W.int8_zp(96, 256, 160, per_n_scales=True), True),
    "int8_postops": lambda: W.int8_postops(256, 512, 512),
    "int8_postops_tails": lambda: W.int8_postops(77, 144, 208),
    "fp8": lambda: W.fp8_prefill(256, 512, 512),
    "fp8_tails": lambda: W.fp8_prefill(300, 528, 272),
    "fp8_wide": lambda: W.fp8_prefill(256, 256, 10240),
    "fp8_ba": lambda: _ba(W.fp8_prefill(128, 384, 256)),
    "fp8_e5m2": lambda: W.fp8_prefill(64, 256, 128, src_dt=W.F8_E5M2, wei_dt=W.F8_E5M2),
    "fp8_mixed": lambda: W.fp8_prefill(64, 256, 128, src_dt=W.F8_E4M3, wei_dt=W.F8_E5M2),
}


@pytest.mark.parametrize("name", sorted(TC_CASES))
def test_tcgen05_gemm_matches_oracle(gpu, name):
    eng, strm = gpu
    p = TC_CASES[name]()
    want = O.run_port(p)
    got, impl = run_problem(p, eng, strm, impl="tcgen05")
    assert impl.startswith("cuda:tcgen05")
    assert_parity(got, want, p.dst_dt, name, slack_for(p, impl))


def _per_n_scale(p):
    r = np.random.Generator(np.random.PCG64(8))
    p.quant["wei_scale"] = W.Quant(W.f32_to_bf16(r.uniform(0.005, 0.02, (1, p.N)).astype(np.float32)), W.BF16, 2)
    p.quant.pop("wei_zp", None)
    return p


def _wide_params(p):
    """f32 scales and s32 zero-points per (K-group, column): several parameter rows per stage."""
    r = np.random.Generator(np.random.PCG64(9))
    g = p.quant["wei_scale"].groups
    G = p.K // g[0]
    p.quant["wei_scale"] = W.Quant(r.uniform(0.005, 0.02, (G, p.N)).astype(np.float32), W.F32, 3, g)
    p.quant["wei_zp"] = W.Quant(r.integers(0, 16, (G, p.N)).astype(np.int32), W.S32, 3, g)
    return p


def _with_bias_relu(p):
    r = np.random.Generator(np.random.PCG64(9))
    p.bias = W.QTensor(W.f32_to_bf16(r.standard_normal((1, p.N), dtype=np.float32)), W.BF16, (1, p.N))
    p.post_ops.append(W.PostOp(W.PO_ELTWISE, W.ELTWISE["relu"], 0.0, 0.0, 1.0))
    return p


WOQ_CASES = {
    "m1": lambda: W.int4_decode(1, 2048, 1024),
    "m8": lambda: W.int4_decode(8, 2048, 1024),
    "m3_tail_cols": lambda: W.int4_decode(3, 1024, 288),
    "m17_two_passes": lambda: W.int4_decode(17, 512, 512),
    "m32": lambda: W.int4_decode(32, 1024, 256),
    "long_k_splits": lambda: W.int4_decode(4, 8192, 512),
    "group32": lambda: W.int4_decode(5, 512, 256, group=32),
    "u4_u8zp": lambda: W.int4_decode(2, 1024, 256, wei_dt=W.U4, zp_dt=W.U8),
    "s4_s4zp": lambda: W.int4_decode(2, 1024, 256, zp_dt=W.S4),
    "no_zp": lambda: W.int4_decode(6, 1024, 256, with_zp=False),
    "per_n_scale": lambda: _per_n_scale(W.int4_decode(4, 1024, 256)),
    "f16_src": lambda: W.int4_decode(4, 1024, 256, src_dt=W.F16, dst_dt=W.F16),
    "bias_relu": lambda: _with_bias_relu(W.int4_decode(7, 1024, 512)),
    "f32_dst": lambda: W.int4_decode(2, 512, 256, dst_dt=W.F32),
    "group16_f32_scales_s32_zp": lambda: _wide_params(W.int4_decode(4, 1024, 512, group=16)),
    "group64_m32": lambda: W.int4_decode(32, 1024, 512, group=64),
    "group256_m12": lambda: W.int4_decode(12, 2048, 256, group=256),
}


WOQ_CASES.update({
    "m16": lambda: W.int4_decode(16, 1024, 512),
    "m32_wide": lambda: W.int4_decode(32, 2048, 1536),
    "m9_many_tiles": lambda: W.int4_decode(9, 4096, 2080),
    "k_tail_stage": lambda: W.int4_decode(5, 1104, 512, group=48),
    "u4_no_zp_f32": lambda: W.int4_decode(3, 768, 256, wei_dt=W.U4, with_zp=False, dst_dt=W.F32),
})


@pytest.mark.parametrize("kernel", ["cuda:tcgen05:woq4", "cuda:woq:skinny"])
@pytest.mark.parametrize("name", sorted(WOQ_CASES))
def test_woq_decode_matches_oracle(gpu, name, kernel):
    """Both int4 decompression kernels (tensor-memory operand; mma.sync) on every case."""
    eng, strm = gpu
    p = WOQ_CASES[name]()
    want = O.run_port(p)
    got, impl = run_problem(p, eng, strm, impl=kernel)
    assert impl == kernel
    assert_parity(got, want, p.dst_dt, name, slack_for(p, impl))
    # the arrival counters are left at zero: a second execution gives the same bits
    got2, _ = run_problem(p, eng, strm, impl=kernel)
    assert np.array_equal(got, got2)


GROUPED_TC_CASES = {
    "small": lambda: W.moe_grouped(96, 256, 128, 8),
    "empty_groups": lambda: W.moe_grouped(40, 128, 64, 6, sizes=[0, 17, 0, 3, 20, 0]),
    "all_in_one": lambda: W.moe_grouped(70, 192, 256, 4, sizes=[0, 0, 70, 0]),
    "several_row_blocks": lambda: W.moe_grouped(700, 128, 256, 3, sizes=[513, 1, 186]),
    "tails_n_k": lambda: W.moe_grouped(50, 200, 176, 3, sizes=[16, 33, 1]),
    "zipf": lambda: W.moe_grouped(1024, 512, 384, 16),
}


@pytest.mark.parametrize("name", sorted(GROUPED_TC_CASES))
def test_tcgen05_grouped_matches_oracle(gpu, name):
    eng, strm = gpu
    p = GROUPED_TC_CASES[name]()
    want = O.run_port(p)
    got, impl = run_problem(p, eng, strm, impl="tcgen05:grouped")
    assert impl == "cuda:tcgen05:grouped"
    assert_parity(got, want, p.dst_dt, name, summation_slack_grouped(p))


def _woq8(M, K, N, per_n=True, dst_dt=W.BF16, seed=31):
    """bf16 src x s8 weights, one weight scale per column (or per tensor), nothing else."""
    r = np.random.Generator(np.random.PCG64(seed))
    sc = r.uniform(0.001, 0.01, (1, N) if per_n else (1,)).astype(np.float32)
    q = {"wei_scale": W.Quant(sc, W.F32, 2 if per_n else 0)}
    return W.Problem("woq8", M, N, K, W.QTensor(W.f32_to_bf16(r.standard_normal((M, K), dtype=np.float32)), W.BF16, (M, K)),
                     W.QTensor(r.integers(-127, 128, (K, N), dtype=np.int8), W.S8, (K, N)), dst_dt, quant=q,
                     apply_to_int=True, fpmath=1)


def _woq8_bias_chain():
    """... with a bf16 bias per column, relu and a multiplication by an f32 column vector (one value per row)."""
    p = _with_bias_relu(_woq8(150, 256, 256))
    r = np.random.Generator(np.random.PCG64(12))
    p.post_ops.append(W.PostOp(W.PO_BINARY, W.BINARY["mul"],
                               src1=W.QTensor(r.uniform(0.5, 1.5, (p.M, 1)).astype(np.float32), W.F32, (p.M, 1))))
    return p


def _moe_bias_gelu():
    """Grouped problem with one f32 bias row per expert and gelu_erf."""
    p = W.moe_grouped(120, 128, 128, 5, sizes=[40, 0, 33, 46, 1])
    r = np.random.Generator(np.random.PCG64(13))
    p.bias = W.QTensor(r.standard_normal((5, p.N)).astype(np.float32), W.F32, (5, p.N))
    p.post_ops.append(W.PostOp(W.PO_ELTWISE, W.ELTWISE["gelu_erf"], 0.0, 0.0, 1.0))
    return p


def _moe_zero_points(zp_dt=W.S8):
    """Grouped problem with one weight zero-point per (expert, column), several row blocks in one expert."""
    p = W.moe_grouped(400, 192, 176, 4, sizes=[150, 0, 249, 1])
    r = np.random.Generator(np.random.PCG64(14))
    lo, hi = (0, 9) if zp_dt == W.U8 else (-8, 9)
    z = r.integers(lo, hi, (p.groups, 1, p.N)).astype({W.S8: np.int8, W.U8: np.uint8, W.S32: np.int32}[zp_dt])
    p.quant["wei_zp"] = W.Quant(z, zp_dt, 0b101)
    return p


def _woq8_zp(per_n, zp_dt=W.S8):
    """Dense s8 decompression with a weight zero-point per column (or one for the tensor)."""
    p = _woq8(200, 320, 208, per_n=per_n)
    r = np.random.Generator(np.random.PCG64(15))
    z = r.integers(-8, 9, (1, p.N) if per_n else (1,)).astype({W.S8: np.int8, W.S32: np.int32}[zp_dt])
    p.quant["wei_zp"] = W.Quant(z, zp_dt, 2 if per_n else 0)
    return p


GROUPED_TC_CHAIN_CASES = {
    "bias_gelu": _moe_bias_gelu,
    "zero_points_s8": _moe_zero_points,
    "zero_points_u8": lambda: _moe_zero_points(W.U8),
    "zero_points_s32": lambda: _moe_zero_points(W.S32),
}


@pytest.mark.parametrize("name", sorted(GROUPED_TC_CHAIN_CASES))
def test_tcgen05_grouped_bias_and_eltwise(gpu, name):
    """Attributes the grouped kernel folds into its epilogue: bias, eltwise, weight zero-points
    (sum_k s (w - z) = sum_k s w - z sum_k s, the row sums from a pre-kernel)."""
    eng, strm = gpu
    p = GROUPED_TC_CHAIN_CASES[name]()
    want = O.run_port(p)
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:grouped"
    assert_parity(got, want, p.dst_dt, p.name, summation_slack_grouped(p))


WOQ8_CASES = {
    "bias_relu_mul": _woq8_bias_chain,
    "zero_point_per_column": lambda: _woq8_zp(True),
    "zero_point_common_s32": lambda: _woq8_zp(False, W.S32),
    "prefill": lambda: _woq8(300, 512, 384),
    "tails": lambda: _woq8(77, 200, 176),
    "one_row": lambda: _woq8(1, 256, 128),
    "common_scale_f32": lambda: _woq8(130, 128, 256, per_n=False, dst_dt=W.F32),
}


@pytest.mark.parametrize("name", sorted(WOQ8_CASES))
def test_tcgen05_dense_woq8_matches_oracle(gpu, name):
    """Dense weight decompression with s8 weights runs the grouped kernel with one group."""
    eng, strm = gpu
    p = WOQ8_CASES[name]()
    want = O.run_port(p)
    got, impl = run_problem(p, eng, strm)
    assert impl == "cuda:tcgen05:woq8"
    assert_parity(got, want, p.dst_dt, name, summation_slack(p))


SCRATCHPAD_CASES = {
    "int8_zero_points": lambda: _wei_zp(W.int8_zp(200, 272, 176), True),  # column and row sums
    "int4_split_k": lambda: W.int4_decode(3, 4096, 512),  # partial sums and arrival counters
    "moe_plan": lambda: W.moe_grouped(96, 256, 128, 8),  # per-expert tile ranges
    "fp8_none": lambda: W.fp8_prefill(64, 256, 128),  # asks for no scratchpad
}


@pytest.mark.parametrize("name", sorted(SCRATCHPAD_CASES))
def test_user_scratchpad_gives_the_same_bits(gpu, name):
    """scratchpad_mode::user (the buffer comes from the caller through DNNL_ARG_SCRATCHPAD,
    with arbitrary contents) against the default library-owned scratchpad, twice in a row."""
    from onednn_b200.runner import Prepared
    eng, strm = gpu
    p = SCRATCHPAD_CASES[name]()
    want, impl = run_problem(p, eng, strm)
    r = Prepared(p, eng, user_scratchpad=True).upload()
    assert r.impl == impl
    for _ in range(2):
        r.execute(strm)
        strm.wait()
        assert np.array_equal(r.download(), want), name


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


RUNTIME_M_CASES = {
    "int8_zp_f32": lambda M: W.int8_zp(M, 1024, 1024, per_n_scales=True),
    "fp8": lambda M: W.fp8_prefill(M, 512, 384),
    "int4_decode": lambda M: W.int4_decode(M, 1024, 512),
}


@pytest.mark.parametrize("name", sorted(RUNTIME_M_CASES))
def test_runtime_m_matches_oracle(gpu, name):
    """M = DNNL_RUNTIME_DIM_VAL at creation (src/common/matmul.cpp:630-744): the same primitive object
    serves several M, each execution choosing the implementation for the M of its memory objects."""
    from onednn_b200.runner import Prepared
    eng, strm = gpu
    for M in (1, 24, 100):
        p = RUNTIME_M_CASES[name](M)
        if p.M > 32 and name == "int4_decode":
            continue
        r = Prepared(p, eng, runtime_m=True).upload()
        r.execute(strm)
        strm.wait()
        got = r.download()
        fixed, impl = run_problem(p, eng, strm)
        assert np.array_equal(got, fixed), "%s M=%d: runtime-M result differs from the fixed-M primitive (%s)" % (name, M, impl)
        assert_parity(got, O.run_port(p), p.dst_dt, "%s M=%d" % (name, M), slack_for(p, impl))


@pytest.mark.gpu
def test_one_primitive_serves_several_shapes(gpu):
    """M, K and N all DNNL_RUNTIME_DIM_VAL (and the strides that depend on them): ONE primitive
    object executes problems of different shapes, settling shapes, implementation and the
    zero-point scratch from the memory objects of each call."""
    from onednn_b200.runner import Prepared
    eng, strm = gpu
    first = None
    for M, K, N in ((24, 256, 128), (100, 512, 384), (7, 80, 48), (24, 256, 128)):
        p = W.int8_zp(M, K, N, per_n_scales=True)
        r = Prepared(p, eng, runtime_m=(3, 3)).upload()
        first = first or r
        assert first.pd.src_desc().get_dims() == (api_rt(), api_rt())
        first.prim.execute(strm, r.args)
        strm.wait()
        assert_parity(r.download(), O.run_port(p), p.dst_dt, "run-time M, K, N = %d, %d, %d" % (M, K, N))
    # memory objects that contradict what the descriptor states are refused
    from onednn_b200 import api
    p = W.int8_zp(16, 64, 32)
    fixed_k = Prepared(p, eng, runtime_m=(1, 2)).upload()  # M and N open, K = 64 stated
    other = Prepared(W.int8_zp(16, 128, 32), eng).upload()
    with pytest.raises(api.error) as ei:
        fixed_k.prim.execute(strm, other.args)
    assert ei.value.status == api.invalid_arguments


def api_rt():
    from onednn_b200 import api
    return api.RUNTIME_DIM_VAL


def test_two_engines_in_one_process(gpu):
    """An engine per device in one process (the ordinary oneDNN usage): the opt-in to large shared
    memory belongs to the (kernel, device) pair, so every kernel family must launch on the second
    device too.  Plain kernels only, no peer memory.  Needs two visible GPUs."""
    from onednn_b200 import api
    if api.engine.get_count(api.engine.kind.gpu) < 2:
        pytest.skip("one GPU visible")
    eng0, strm0 = gpu
    eng1 = api.engine(api.engine.kind.gpu, 1)
    strm1 = api.stream(eng1)
    for make in (lambda: W.int8_zp(64, 256, 256), lambda: W.int4_decode(4, 512, 256), lambda: W.moe_grouped(96, 256, 128, 8),
                 lambda: W.fp8_prefill(96, 512, 384)):
        p = make()
        want = O.run_port(p)
        for eng, strm in ((eng0, strm0), (eng1, strm1), (eng0, strm0)):
            got, impl = run_problem(p, eng, strm)
            assert_parity(got, want, p.dst_dt, "%s via %s" % (p.name, impl), slack_for(p, impl))


@pytest.mark.gpu
@pytest.mark.parametrize("make", [lambda: W.int8_zp(256, 1024, 1024), lambda: W.fp8_prefill(300, 512, 640),
                                  lambda: W.int8_zp(300, 512, 2048, per_n_scales=True)], ids=["int8_zp", "fp8", "int8_zp_f32"])
def test_replicated_dst_fills_every_buffer(gpu, make):
    """The fused exchange of the tensor-core GEMM, checked on ONE GPU: the two 'ranks' run one
    after the other on the same stream (their kernels only store and raise flags, neither waits
    for the other), each writing its column slice into both full buffers; the flag wait that
    follows finds both flags set.  Both buffers must then hold the oracle's full result."""
    import ctypes as C
    import torch
    from onednn_b200 import api, sharding
    from onednn_b200.runner import Prepared
    eng, strm = gpu
    full = make()
    want = O.run_port(full)
    es = W.nbytes(full.dst_dt, 1)
    world = 2
    dev = torch.device("cuda:0")
    bufs = [torch.zeros(full.M * full.N * es, dtype=torch.uint8, device=dev) for _ in range(world)]
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(world)]
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    bases = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    flagp = (C.c_void_p * world)(*[f.data_ptr() for f in flags])
    L = api.lib()
    L.dnnl_cuda_interop_primitive_replicate_dst.argtypes = [
        C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_uint]
    L.dnnl_cuda_interop_peer_wait.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_uint]
    keep = []
    for epoch in (1, 2):  # twice: the CTA counter must be back at zero
        for b in bufs:
            b.zero_()
        for rank in range(world):
            p = sharding.shard(full, rank, world)
            lo, _ = sharding.column_range(full.N, rank, world)
            prep = Prepared(p, eng, dst_ld=full.N)
            assert prep.impl in ("cuda:tcgen05:int8", "cuda:tcgen05:fp8")
            ptrs = {}
            def put(name, arr):
                t = torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1).copy()).to(dev)
                keep.append(t)
                ptrs[name] = t.data_ptr()
            put("src", p.src.data)
            put("wei", p.wei.data)
            if p.bias is not None:
                put("bias", p.bias.data)
            for name, q in p.quant.items():
                put(name, q.data)
            for i, e in enumerate(p.post_ops):
                if e.kind == W.PO_BINARY:
                    put("po%d" % i, e.src1.data)
            ptrs["dst"] = bufs[rank].data_ptr() + lo * es
            prep.bind_device(ptrs)
            torch.cuda.synchronize()  # torch's copies and fills run on its own stream
            st = L.dnnl_cuda_interop_primitive_replicate_dst(prep.prim._h, world, rank, bases, C.c_size_t(bufs[0].numel()), flagp,
                                                             done.data_ptr(), epoch)
            assert st == 0
            prep.execute(strm)
            keep.append(prep)
        for rank in range(world):
            assert L.dnnl_cuda_interop_peer_wait(strm._h, world, flags[rank].data_ptr(), epoch) == 0
        strm.wait()
        for b in bufs:
            got = b.cpu().numpy().view(W.NP_STORAGE[full.dst_dt]).reshape(full.M, full.N)
            assert_parity(got, want, full.dst_dt, "%s replicated, epoch %d" % (full.name, epoch), slack_for(full, "cuda:tcgen05"))
        assert int(done.item()) == 0


@pytest.mark.gpu
def test_peer_scatter_and_wait_on_one_gpu(gpu):
    """The exchange kernels with both 'ranks' on one GPU, one after the other on the same stream
    (the scatter only stores and raises flags; the wait finds them raised): column blocks of a
    dense result and row segments of a grouped one must land in both full buffers."""
    import ctypes as C
    import torch
    from onednn_b200 import api
    eng, strm = gpu
    dev = torch.device("cuda:0")
    L = api.lib()
    L.dnnl_cuda_interop_peer_scatter.argtypes = [
        C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int,
        C.c_void_p, C.c_void_p, C.c_uint, C.c_void_p]
    L.dnnl_cuda_interop_peer_wait.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_uint]
    world, M, N, es = 2, 70, 96, 2
    g = torch.Generator(device="cpu").manual_seed(5)
    full = torch.randint(0, 2 ** 15, (M, N), dtype=torch.int16, generator=g)
    bufs = [torch.zeros(M, N, dtype=torch.int16, device=dev) for _ in range(world)]
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(world)]
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    bases = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    flagp = (C.c_void_p * world)(*[f.data_ptr() for f in flags])
    keep = []
    # dense: rank r owns columns [48 r, 48 r + 48)
    for rank in range(world):
        local = full[:, 48 * rank:48 * rank + 48].contiguous().to(dev)
        keep.append(local)
        seg = (C.c_int64 * 3)(0, 0, M)
        torch.cuda.synchronize()
        assert L.dnnl_cuda_interop_peer_scatter(strm._h, world, rank, local.data_ptr(), 48 * es, 48 * es, bases, N * es,
                                                48 * rank * es, 1, seg, flagp, 1, done.data_ptr()) == 0
    for rank in range(world):
        assert L.dnnl_cuda_interop_peer_wait(strm._h, world, flags[rank].data_ptr(), 1) == 0
    strm.wait()
    for b in bufs:
        assert torch.equal(b.cpu(), full)
    # grouped: rank 0 owns rows [0, 10) and [40, 70), rank 1 rows [10, 40), as two / one segments
    for b in bufs:
        b.zero_()
    owned = {0: [(0, 10), (40, 70)], 1: [(10, 40)]}
    for rank in range(world):
        local = torch.cat([full[a:b] for a, b in owned[rank]]).contiguous().to(dev)
        keep.append(local)
        trip, at = [], 0
        for a, b in owned[rank]:
            trip += [at, a, b - a]
            at += b - a
        seg = (C.c_int64 * len(trip))(*trip)
        torch.cuda.synchronize()
        assert L.dnnl_cuda_interop_peer_scatter(strm._h, world, rank, local.data_ptr(), N * es, N * es, bases, N * es, 0,
                                                len(owned[rank]), seg, flagp, 2, done.data_ptr()) == 0
    for rank in range(world):
        assert L.dnnl_cuda_interop_peer_wait(strm._h, world, flags[rank].data_ptr(), 2) == 0
    strm.wait()
    for b in bufs:
        assert torch.equal(b.cpu(), full)
    assert int(done.item()) == 0
    # a flag that nothing raises: the wait gives up after its limit and the stream reports it
    assert L.dnnl_cuda_interop_peer_wait(strm._h, world, flags[0].data_ptr(), 3) == 0
    with pytest.raises(api.error):
        strm.wait()
