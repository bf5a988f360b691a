"""Reorder problems of the quantized-matmul flow: quantizing weights and
activations before the matmul, decompressing 4-bit weights, changing between
row-major and column-major storage.  Small seeded tensors; the same list is
pinned against the reference library on the CPU (tests/golden/reorder.npz)
and run through the CUDA library on the GPU."""
import numpy as np

from onednn_b200 import workloads as W


def _r(seed):
    return np.random.Generator(np.random.PCG64(seed))


def _f32(r, dims, scale=1.0):
    return W.QTensor((r.standard_normal(dims) * scale).astype(np.float32), W.F32, dims)


def quantize_weights_per_column():
    """f32 [K,N] -> s8 with one f32 dst scale per column."""
    r = _r(201)
    K, N = 48, 40
    q = {"dst_scale": W.Quant(r.uniform(0.005, 0.03, (1, N)).astype(np.float32), W.F32, 2)}
    return W.Reorder("quantize_weights_per_column", _f32(r, (K, N)), W.S8, quant=q)


def quantize_activations_u8():
    """f32 [M,K] -> u8 with a common src scale, common dst scale and a dst zero-point."""
    r = _r(202)
    q = {"src_scale": W.Quant(np.array([0.5], np.float32), W.F32, 0),
         "dst_scale": W.Quant(np.array([0.02], np.float32), W.F32, 0),
         "dst_zp": W.Quant(np.array([128], np.int32), W.S32, 0)}
    return W.Reorder("quantize_activations_u8", _f32(r, (33, 70), 3.0), W.U8, quant=q)


def quantize_activations_per_row():
    """bf16 [M,K] -> s8 with one dst scale per row (per-token quantization)."""
    r = _r(215)
    M, K = 21, 64
    x = W.QTensor(W.f32_to_bf16(r.standard_normal((M, K)).astype(np.float32) * 2), W.BF16, (M, K))
    q = {"dst_scale": W.Quant(r.uniform(0.01, 0.05, (M, 1)).astype(np.float32), W.F32, 1)}
    return W.Reorder("quantize_activations_per_row", x, W.S8, quant=q)


def _f8_edge_values(r, dims, top):
    """Normal data plus the values where an 8-bit float conversion decides: the largest finite
    value, the round-down / overflow boundary above it, tiny and subnormal magnitudes, zeros."""
    x = (r.standard_normal(dims) * top / 6).astype(np.float32)
    edge = np.array([top, top * 1.03, top * 1.04, -top * 1.2, 3 * top, 2.0 ** -10, 2.0 ** -10 * 1.01, 2.0 ** -9,
                     1.5 * 2.0 ** -9, 2.0 ** -7 * 1.0625, -2.0 ** -17, 2.0 ** -16, 1e-30, 0.0, -0.0, 0.4375, 0.46875,
                     17.0, 18.0, 19.0, 0.099, -0.0991], np.float32)
    x.reshape(-1)[:edge.size] = edge
    return x


def quantize_f32_to_e4m3():
    """f32 -> f8_e4m3 with a common dst scale (the fp8 GEMM's weight / activation quantization)."""
    r = _r(216)
    dims = (24, 64)
    q = {"dst_scale": W.Quant(np.array([0.5], np.float32), W.F32, 0)}
    return W.Reorder("quantize_f32_to_e4m3", W.QTensor(_f8_edge_values(r, dims, 224.0), W.F32, dims), W.F8_E4M3, quant=q)


def quantize_f32_to_e5m2():
    r = _r(217)
    dims = (16, 48)
    x = _f8_edge_values(r, dims, 57344.0)
    x.reshape(-1)[40:44] = [np.inf, -np.inf, 61184.0, 61500.0]
    return W.Reorder("quantize_f32_to_e5m2", W.QTensor(x, W.F32, dims), W.F8_E5M2)


def quantize_bf16_to_e4m3_per_column():
    r = _r(218)
    K, N = 40, 32
    x = W.QTensor(W.f32_to_bf16(r.standard_normal((K, N)).astype(np.float32)), W.BF16, (K, N))
    q = {"dst_scale": W.Quant(r.uniform(0.005, 0.02, (1, N)).astype(np.float32), W.F32, 2)}
    return W.Reorder("quantize_bf16_to_e4m3_per_column", x, W.F8_E4M3, quant=q)


def transpose_f32_to_e5m2():
    r = _r(219)
    return W.Reorder("transpose_f32_to_e5m2", _f32(r, (18, 30), 100.0), W.F8_E5M2, dst_strides=(1, 18))


def dequantize_experts_transposed():
    """s8 [G,K,N] row-major -> f32 with K and N swapped in memory, one src scale per column and
    a common src zero-point."""
    r = _r(220)
    G, K, N = 3, 40, 34
    q = {"src_scale": W.Quant(r.uniform(0.01, 0.1, (1, 1, N)).astype(np.float32), W.F32, 4),
         "src_zp": W.Quant(np.array([-2], np.int32), W.S32, 0)}
    src = W.QTensor(r.integers(-128, 128, (G, K, N)).astype(np.int8), W.S8, (G, K, N))
    return W.Reorder("dequantize_experts_transposed", src, W.F32, dst_strides=(K * N, 1, K), quant=q)


def quantize_transposed_per_row():
    """f32 [K,N] column-major -> s8 row-major with one dst scale per row of the matrix."""
    r = _r(221)
    K, N = 70, 33
    x = W.QTensor((r.standard_normal((K, N)) * 0.1).astype(np.float32), W.F32, (K, N), strides=(1, K))
    q = {"dst_scale": W.Quant(r.uniform(0.001, 0.003, (K, 1)).astype(np.float32), W.F32, 1)}
    return W.Reorder("quantize_transposed_per_row", x, W.S8, quant=q)


def transpose_f32_to_bf16():
    """f32 row-major -> bf16 column-major."""
    r = _r(203)
    return W.Reorder("transpose_f32_to_bf16", _f32(r, (37, 52)), W.BF16, dst_strides=(1, 37))


def dequantize_s8_per_column():
    """s8 [K,N] -> f32 with one src scale per column and a common src zero-point."""
    r = _r(204)
    K, N = 64, 24
    q = {"src_scale": W.Quant(r.uniform(0.01, 0.1, (1, N)).astype(np.float32), W.F32, 2),
         "src_zp": W.Quant(np.array([3], np.int32), W.S32, 0)}
    src = W.QTensor(r.integers(-128, 128, (K, N)).astype(np.int8), W.S8, (K, N))
    return W.Reorder("dequantize_s8_per_column", src, W.F32, quant=q)


def compress_f32_to_s4():
    """f32 -> s4: saturating round, two elements per byte."""
    r = _r(205)
    return W.Reorder("compress_f32_to_s4", _f32(r, (32, 48), 5.0), W.S4)


def compress_f32_to_u4():
    r = _r(206)
    x = W.QTensor((r.standard_normal((16, 64)) * 6 + 7).astype(np.float32), W.F32, (16, 64))
    return W.Reorder("compress_f32_to_u4", x, W.U4)


def decompress_s4_grouped():
    """s4 [K,N] -> bf16 with bf16 scales and u4 zero-points per (32 k, column)."""
    r = _r(207)
    K, N, g = 128, 32, 32
    q = {"src_scale": W.Quant(W.f32_to_bf16(r.uniform(0.01, 0.1, (K // g, N)).astype(np.float32)), W.BF16, 3, (g, 1)),
         "src_zp": W.Quant(W.pack_int4(r.integers(0, 16, (K // g, N))), W.U4, 3, (g, 1))}
    src = W.QTensor(W.pack_int4(r.integers(-8, 8, (K, N))), W.S4, (K, N))
    return W.Reorder("decompress_s4_grouped", src, W.BF16, quant=q)


def decompress_u4_plain():
    """u4 -> f32, no attributes."""
    r = _r(208)
    src = W.QTensor(W.pack_int4(r.integers(0, 16, (24, 40))), W.U4, (24, 40))
    return W.Reorder("decompress_u4_plain", src, W.F32)


def quantize_experts_per_column():
    """f32 [G,K,N] -> s8 with one dst scale per column (mask 4)."""
    r = _r(209)
    G, K, N = 3, 16, 24
    q = {"dst_scale": W.Quant(r.uniform(0.005, 0.03, (1, 1, N)).astype(np.float32), W.F32, 4)}
    return W.Reorder("quantize_experts_per_column", _f32(r, (G, K, N)), W.S8, quant=q)


def accumulate_with_sum():
    """f32 -> f32 with a common src scale and a sum post-op (dst += ...)."""
    r = _r(210)
    dims = (20, 36)
    q = {"src_scale": W.Quant(np.array([0.25], np.float32), W.F32, 0)}
    init = r.standard_normal(dims).astype(np.float32)
    return W.Reorder("accumulate_with_sum", _f32(r, dims), W.F32, quant=q, beta=0.5, dst_init=init)


def saturate_s32_to_s8():
    r = _r(211)
    src = W.QTensor(r.integers(-400, 400, (18, 30)).astype(np.int32), W.S32, (18, 30))
    return W.Reorder("saturate_s32_to_s8", src, W.S8)


def shift_u8_to_s8():
    """u8 -> s8 through a src zero-point of 128 (the s8s8 / u8s8 switch)."""
    r = _r(212)
    src = W.QTensor(r.integers(0, 256, (25, 16)).astype(np.uint8), W.U8, (25, 16))
    q = {"src_zp": W.Quant(np.array([128], np.int32), W.S32, 0)}
    return W.Reorder("shift_u8_to_s8", src, W.S8, quant=q)


def widen_e4m3_to_f32():
    r = _r(213)
    x = W.QTensor(W.f32_to_e4m3(r.standard_normal((16, 48)).astype(np.float32) * 4), W.F8_E4M3, (16, 48))
    return W.Reorder("widen_e4m3_to_f32", x, W.F32)


def narrow_bf16_to_f16_transposed():
    r = _r(214)
    x = W.QTensor(W.f32_to_bf16(r.standard_normal((30, 44)).astype(np.float32)), W.BF16, (30, 44), strides=(1, 30))
    return W.Reorder("narrow_bf16_to_f16_transposed", x, W.F16)


CASES = {f.__name__: f for f in (
    quantize_weights_per_column, quantize_activations_u8, transpose_f32_to_bf16, dequantize_s8_per_column,
    compress_f32_to_s4, compress_f32_to_u4, decompress_s4_grouped, decompress_u4_plain,
    quantize_experts_per_column, accumulate_with_sum, saturate_s32_to_s8, shift_u8_to_s8, widen_e4m3_to_f32,
    narrow_bf16_to_f16_transposed, quantize_activations_per_row, quantize_f32_to_e4m3, quantize_f32_to_e5m2,
    quantize_bf16_to_e4m3_per_column, transpose_f32_to_e5m2, dequantize_experts_transposed,
    quantize_transposed_per_row)}
