"""Small problems that walk the attribute combinations the reference's own
matmul test inputs use (tests/benchdnn/inputs/matmul/test_matmul_int8:10-56,
harness_matmul_grouped_2dby3d), restated as seeded problems.  Shared by a CPU
test (C restatement against the live reference, where it is built) and a GPU
test (every implementation that accepts the problem against the C
restatement)."""
import numpy as np

from onednn_b200 import workloads as W


def _r(seed):
    return np.random.Generator(np.random.PCG64(seed))


def _s8(r, shape, lo=-30, hi=31):
    return r.integers(lo, hi, shape).astype(np.int8)


def _s32(v):
    return np.array([v], np.int32)


def zero_points_all_common():
    """s8:s8:s8, src zp 1 + wei zp -1 + dst zp 2 (all per tensor)."""
    r = _r(101)
    M, K, N = 20, 96, 48
    q = {"src_zp": W.Quant(_s32(1), W.S32, 0), "wei_zp": W.Quant(_s32(-1), W.S32, 0),
         "dst_zp": W.Quant(_s32(2), W.S32, 0), "dst_scale": W.Quant(np.array([37.5], np.float32), W.F32, 0)}
    return W.Problem("zp_common", M, N, K, W.QTensor(_s8(r, (M, K)), W.S8, (M, K)),
                     W.QTensor(_s8(r, (K, N)), W.S8, (K, N)), W.S8, quant=q)


def zero_points_src_per_k():
    """u8:s8:f32, src zp per K (mask 1<<1) + wei zp 1 + dst zp 2."""
    r = _r(102)
    M, K, N = 12, 64, 40
    q = {"src_zp": W.Quant(r.integers(0, 9, (1, K)).astype(np.int32), W.S32, 2),
         "wei_zp": W.Quant(_s32(1), W.S32, 0), "dst_zp": W.Quant(_s32(2), W.S32, 0)}
    return W.Problem("zp_src_per_k", M, N, K, W.QTensor(r.integers(0, 256, (M, K)).astype(np.uint8), W.U8, (M, K)),
                     W.QTensor(_s8(r, (K, N)), W.S8, (K, N)), W.F32, quant=q)


def scales_and_post_op_chain():
    """s8:s8:f32, scales src 1.25 + wei per column + dst 0.5; post-ops sum, mul by an s32 row
    vector per column, linear 2 x - 1."""
    r = _r(103)
    M, K, N = 18, 80, 56
    q = {"src_scale": W.Quant(np.array([1.25], np.float32), W.F32, 0),
         "wei_scale": W.Quant(r.uniform(0.01, 0.1, (1, N)).astype(np.float32), W.F32, 2),
         "dst_scale": W.Quant(np.array([0.5], np.float32), W.F32, 0)}
    po = [W.PostOp(W.PO_SUM, scale=1.0, zero_point=0),
          W.PostOp(W.PO_BINARY, W.BINARY["mul"], src1=W.QTensor(r.integers(-3, 4, (1, N)).astype(np.int32), W.S32, (1, N))),
          W.PostOp(W.PO_ELTWISE, W.ELTWISE["linear"], 2.0, -1.0, 1.0)]
    p = W.Problem("scales_chain", M, N, K, W.QTensor(_s8(r, (M, K)), W.S8, (M, K)),
                  W.QTensor(_s8(r, (K, N)), W.S8, (K, N)), W.F32, quant=q, post_ops=po)
    p.dst_init = r.standard_normal((M, N)).astype(np.float32)
    return p


def binary_add_full():
    """u8:s8:s32 with a dense f32 operand added."""
    r = _r(104)
    M, K, N = 10, 48, 32
    po = [W.PostOp(W.PO_BINARY, W.BINARY["add"],
                   src1=W.QTensor(np.round(r.standard_normal((M, N)) * 50).astype(np.float32), W.F32, (M, N)))]
    return W.Problem("binary_add", M, N, K, W.QTensor(r.integers(0, 256, (M, K)).astype(np.uint8), W.U8, (M, K)),
                     W.QTensor(_s8(r, (K, N)), W.S8, (K, N)), W.S32, post_ops=po)


def decompress_f32_common():
    """f32:s8:f32 weights decompression: wei scale 1.25 (f32) and wei zp -1 (s8), per tensor."""
    r = _r(105)
    M, K, N = 6, 64, 32
    q = {"wei_scale": W.Quant(np.array([1.25], np.float32), W.F32, 0),
         "wei_zp": W.Quant(np.array([-1], np.int8), W.S8, 0)}
    return W.Problem("woq_f32_common", M, N, K, W.QTensor(r.standard_normal((M, K)).astype(np.float32), W.F32, (M, K)),
                     W.QTensor(_s8(r, (K, N), -127, 128), W.S8, (K, N)), W.F32, quant=q, apply_to_int=True, fpmath=1)


def decompress_bf16_per_oc():
    """bf16:s8:bf16: wei scales per column (bf16), wei zps per column (u8)."""
    r = _r(106)
    M, K, N = 9, 96, 48
    q = {"wei_scale": W.Quant(W.f32_to_bf16(r.uniform(0.01, 0.05, (1, N)).astype(np.float32)), W.BF16, 2),
         "wei_zp": W.Quant(r.integers(0, 6, (1, N)).astype(np.uint8), W.U8, 2)}
    return W.Problem("woq_bf16_per_oc", M, N, K,
                     W.QTensor(W.f32_to_bf16(r.standard_normal((M, K)).astype(np.float32)), W.BF16, (M, K)),
                     W.QTensor(_s8(r, (K, N), -127, 128), W.S8, (K, N)), W.BF16, quant=q, apply_to_int=True, fpmath=1)


def decompress_bf16_per_element():
    """bf16:s8:bf16 with 1x1 groups: one scale and one zero-point per weight."""
    r = _r(107)
    M, K, N = 5, 32, 16
    q = {"wei_scale": W.Quant(W.f32_to_bf16(r.uniform(0.01, 0.05, (K, N)).astype(np.float32)), W.BF16, 3, (1, 1)),
         "wei_zp": W.Quant(r.integers(0, 6, (K, N)).astype(np.uint8), W.U8, 3, (1, 1))}
    return W.Problem("woq_bf16_per_elem", M, N, K,
                     W.QTensor(W.f32_to_bf16(r.standard_normal((M, K)).astype(np.float32)), W.BF16, (M, K)),
                     W.QTensor(_s8(r, (K, N), -127, 128), W.S8, (K, N)), W.BF16, quant=q, apply_to_int=True, fpmath=1)


def transposed_tags():
    """u8:s8:s32 with src and weights stored transposed (tags ba)."""
    r = _r(108)
    M, K, N = 24, 64, 48
    src = r.integers(0, 256, (M, K)).astype(np.uint8)
    wei = _s8(r, (K, N))
    return W.Problem("tags_ba", M, N, K, W.QTensor(np.ascontiguousarray(src.T), W.U8, (M, K), (1, M)),
                     W.QTensor(np.ascontiguousarray(wei.T), W.S8, (K, N), (1, K)), W.S32)


def grouped_f32_plain():
    """Grouped f32 x f32 with an empty group."""
    r = _r(109)
    sizes = np.array([5, 0, 9, 2])
    M, K, N, G = int(sizes.sum()), 32, 24, 4
    return W.Problem("grouped_f32", M, N, K, W.QTensor(r.standard_normal((M, K)).astype(np.float32), W.F32, (M, K)),
                     W.QTensor(r.standard_normal((G, K, N)).astype(np.float32), W.F32, (G, K, N)), W.F32,
                     offsets=np.cumsum(sizes).astype(np.int32))


def grouped_woq_zero_points_relu():
    """Grouped f16 x s8 decompression: scales and s8 zero-points per (expert, column), relu."""
    r = _r(110)
    sizes = np.array([7, 3, 0, 6])
    M, K, N, G = int(sizes.sum()), 64, 32, 4
    q = {"wei_scale": W.Quant(r.uniform(0.01, 0.05, (G, 1, N)).astype(np.float32), W.F32, 0b101),
         "wei_zp": W.Quant(r.integers(-3, 4, (G, 1, N)).astype(np.int8), W.S8, 0b101)}
    po = [W.PostOp(W.PO_ELTWISE, W.ELTWISE["relu"], 0.0, 0.0, 1.0)]
    return W.Problem("grouped_woq_zp", M, N, K,
                     W.QTensor(r.standard_normal((M, K)).astype(np.float16).view(np.uint16), W.F16, (M, K)),
                     W.QTensor(_s8(r, (G, K, N), -127, 128), W.S8, (G, K, N)), W.F16, quant=q, post_ops=po,
                     apply_to_int=True, fpmath=2, offsets=np.cumsum(sizes).astype(np.int32))


def prelu_per_column_after_sum():
    """s8:s8:f32 with scales, a sum and a prelu whose f32 weights vary per column (mask 1 << 1)."""
    r = _r(111)
    M, K, N = 14, 64, 48
    q = {"src_scale": W.Quant(np.array([0.25], np.float32), W.F32, 0),
         "wei_scale": W.Quant(np.array([0.5], np.float32), W.F32, 0),
         "dst_scale": W.Quant(np.array([4.0], np.float32), W.F32, 0)}
    po = [W.PostOp(W.PO_SUM, scale=1.0, zero_point=0),
          W.PostOp(W.PO_PRELU, src1=W.QTensor(r.uniform(-1.0, 1.0, (1, N)).astype(np.float32), W.F32, (1, N)))]
    p = W.Problem("prelu_per_oc", M, N, K, W.QTensor(_s8(r, (M, K)), W.S8, (M, K)),
                  W.QTensor(_s8(r, (K, N)), W.S8, (K, N)), W.F32, quant=q, post_ops=po)
    p.dst_init = r.standard_normal((M, N)).astype(np.float32)
    return p


CASES = {f.__name__: f for f in (
    zero_points_all_common, zero_points_src_per_k, scales_and_post_op_chain, binary_add_full, decompress_f32_common,
    decompress_bf16_per_oc, decompress_bf16_per_element, transposed_tags, grouped_f32_plain,
    grouped_woq_zero_points_relu, prelu_per_column_after_sum)}
