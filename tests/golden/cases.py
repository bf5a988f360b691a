"""The small seeded problems whose reference outputs are committed as golden
fixtures (golden.npz).  Shared by make_golden.py and the tests."""
from onednn_b200 import workloads as W


def _sum_case():
    import numpy as np
    p = W.int8_postops(24, 128, 48, seed=77)
    p.post_ops.insert(0, W.PostOp(W.PO_SUM, scale=0.5, zero_point=0))
    r = np.random.Generator(np.random.PCG64(5))
    p.dst_init = r.integers(-100, 100, (24, 48)).astype(np.int8)
    return p


def _eltwise_chain():
    p = W.int8_zp(16, 64, 40, per_n_scales=True, seed=9)
    for name, a, b in [("relu", 0.1, 0.0), ("linear", 1.5, -0.25), ("tanh", 0, 0), ("swish", 1.0, 0),
                       ("clip_v2", -0.5, 0.5), ("gelu_erf", 0, 0), ("logistic", 0, 0), ("abs", 0, 0)]:
        p.post_ops.append(W.PostOp(W.PO_ELTWISE, W.ELTWISE[name], a, b, 1.0))
    return p


def _pr_case():
    """int8 with grouped weight zero-points and precomputed src reductions."""
    import numpy as np
    r = np.random.Generator(np.random.PCG64(11))
    M, K, N, g = 8, 128, 32, 32
    src = r.integers(-20, 20, (M, K)).astype(np.int8)
    wei = r.integers(-20, 20, (K, N)).astype(np.int8)
    wz = r.integers(-3, 4, (K // g, N)).astype(np.int8)
    pr = src.astype(np.int32).reshape(M, K // g, g).sum(-1).astype(np.int32)
    q = {"wei_zp": W.Quant(wz, W.S8, 3, (g, 1)), "src_pr": W.Quant(pr, W.S32, 3, (1, g))}
    return W.Problem("int8_pr", M, N, K, W.QTensor(src, W.S8, (M, K)), W.QTensor(wei, W.S8, (K, N)), W.F32, quant=q)


CASES = {
    "int8_zp_s32": lambda: W.int8_zp(48, 256, 96),
    "int8_zp_f32": lambda: W.int8_zp(48, 256, 96, per_n_scales=True),
    "fp8_bf16": lambda: W.fp8_prefill(24, 192, 80),
    "fp8_e5m2": lambda: W.fp8_prefill(8, 64, 48, src_dt=W.F8_E5M2, wei_dt=W.F8_E5M2),
    "int4_m1": lambda: W.int4_decode(1, 512, 128),
    "int4_m8": lambda: W.int4_decode(8, 256, 64),
    "u4_u8zp": lambda: W.int4_decode(3, 256, 64, wei_dt=W.U4, zp_dt=W.U8),
    "s8w_nozp": lambda: W.int4_decode(5, 256, 48, wei_dt=W.S8, with_zp=False),
    "f16_src_int4": lambda: W.int4_decode(2, 256, 64, src_dt=W.F16, dst_dt=W.F16),
    "int8_postops": lambda: W.int8_postops(40, 256, 72),
    "int8_sum": _sum_case,
    "eltwise_chain": _eltwise_chain,
    "int8_pr": _pr_case,
    "moe": lambda: W.moe_grouped(72, 128, 48, 6),
    "moe_empty": lambda: W.moe_grouped(30, 64, 32, 5, sizes=[0, 11, 0, 19, 0]),
}
