"""Seeded synthetic inputs for the quantized-matmul workloads.

A :class:`Problem` is a plain description of one ``dnnl::matmul`` call: the
tensors as raw numpy buffers (sub-byte and 16/8-bit float types are kept as
their storage bytes), the quantization attributes, the post-op chain.  The
same object feeds the library through its C API (``onednn_b200.api``), the CPU
oracle used by the tests, and the benchmark.

Data-type codes are the values of ``dnnl_data_type_t``
(include/oneapi/dnnl/dnnl_common_types.h:75-115 in oneDNN).
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

F16, BF16, F32, S32, S8, U8 = 1, 2, 3, 4, 5, 6
F8_E5M2, F8_E4M3, S4, U4 = 9, 10, 11, 12

DT_NAME = {F16: "f16", BF16: "bf16", F32: "f32", S32: "s32", S8: "s8", U8: "u8",
           F8_E5M2: "f8_e5m2", F8_E4M3: "f8_e4m3", S4: "s4", U4: "u4"}
NP_STORAGE = {F16: np.uint16, BF16: np.uint16, F32: np.float32, S32: np.int32,
              S8: np.int8, U8: np.uint8, F8_E5M2: np.uint8, F8_E4M3: np.uint8,
              S4: np.uint8, U4: np.uint8}

# dnnl_alg_kind_t values (include/oneapi/dnnl/dnnl_types.h:2117-2228)
ELTWISE = {"relu": 0x20, "tanh": 0x21, "elu": 0x22, "square": 0x23, "abs": 0x24,
           "sqrt": 0x25, "linear": 0x26, "soft_relu": 0x27, "hardsigmoid": 0x28,
           "logistic": 0x29, "exp": 0x2a, "gelu_tanh": 0x2b, "swish": 0x2c,
           "log": 0x2d, "clip": 0x2e, "clip_v2": 0x2f, "pow": 0x30,
           "gelu_erf": 0x31, "round": 0x32, "mish": 0x33, "hardswish": 0x34}
BINARY = {"add": 0x1fff0, "mul": 0x1fff1, "max": 0x1fff2, "min": 0x1fff3,
          "div": 0x1fff4, "sub": 0x1fff5}

PO_SUM, PO_ELTWISE, PO_BINARY, PO_PRELU = 1, 2, 3, 4  # PO_PRELU: src1 = f32 weights over the masked dst dims


def nbytes(dt: int, nelems: int) -> int:
    if dt in (S4, U4):
        return (nelems + 1) // 2
    return nelems * np.dtype(NP_STORAGE[dt]).itemsize


# ---------------------------------------------------------------- conversions
def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 storage (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> OCP e4m3 storage bytes, saturating."""
    import ml_dtypes
    x = np.clip(np.asarray(x, dtype=np.float32), -448.0, 448.0)
    return x.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    import ml_dtypes
    return b.view(ml_dtypes.float8_e4m3fn).astype(np.float32)


def f32_to_e5m2(x: np.ndarray) -> np.ndarray:
    import ml_dtypes
    x = np.clip(np.asarray(x, dtype=np.float32), -57344.0, 57344.0)
    return x.astype(ml_dtypes.float8_e5m2).view(np.uint8)


def pack_int4(v: np.ndarray) -> np.ndarray:
    """Packs integers (-8..7 or 0..15), last dim even, two per byte: the
    element with the even index sits in the low nibble (oneDNN
    src/common/nibble.hpp:28-65)."""
    v = np.asarray(v).astype(np.int16) & 0xF
    lo, hi = v[..., 0::2], v[..., 1::2]
    return (lo | (hi << 4)).astype(np.uint8)


def unpack_int4(b: np.ndarray, signed: bool) -> np.ndarray:
    lo = (b & 0xF).astype(np.int16)
    hi = (b >> 4).astype(np.int16)
    out = np.stack([lo, hi], axis=-1).reshape(*b.shape[:-1], b.shape[-1] * 2)
    if signed:
        out = np.where(out >= 8, out - 16, out)
    return out


def to_storage(x: np.ndarray, dt: int) -> np.ndarray:
    """Converts real/integer values to the storage bytes of data type dt."""
    if dt == F32:
        return np.ascontiguousarray(x, dtype=np.float32)
    if dt == BF16:
        return f32_to_bf16(x)
    if dt == F16:
        return np.ascontiguousarray(x, dtype=np.float16).view(np.uint16)
    if dt == F8_E4M3:
        return f32_to_e4m3(x)
    if dt == F8_E5M2:
        return f32_to_e5m2(x)
    if dt in (S4, U4):
        return pack_int4(x)
    return np.ascontiguousarray(x).astype(NP_STORAGE[dt])


def to_f32(data: np.ndarray, dt: int) -> np.ndarray:
    """Decodes storage bytes to float32 values (for error reporting)."""
    if dt == F32:
        return data
    if dt == BF16:
        return bf16_to_f32(data)
    if dt == F16:
        return data.view(np.float16).astype(np.float32)
    if dt == F8_E4M3:
        return e4m3_to_f32(data)
    if dt == F8_E5M2:  # the upper byte of a half
        return (data.astype(np.uint16) << 8).view(np.float16).astype(np.float32)
    if dt in (S4, U4):
        return unpack_int4(data, dt == S4).astype(np.float32)
    return data.astype(np.float32)


# ------------------------------------------------------------------- records
@dataclass
class QTensor:
    data: np.ndarray  # storage bytes, see NP_STORAGE
    dt: int
    dims: Tuple[int, ...]
    strides: Optional[Tuple[int, ...]] = None  # elements; None = row-major

    def __post_init__(self):
        if self.strides is None:
            s, acc = [], 1
            for d in reversed(self.dims):
                s.append(acc)
                acc *= d
            self.strides = tuple(reversed(s))


@dataclass
class Quant:
    data: np.ndarray
    dt: int
    mask: int  # bit i = dim i of the tensor the parameter belongs to
    groups: Tuple[int, int] = (1, 1)  # group sizes along the last two dims


@dataclass
class Reorder:
    """One ``dnnl::reorder`` call between two plain (strided) layouts of the
    same logical tensor: ``src`` carries data, dims and strides; the result has
    data type ``dst_dt`` and strides ``dst_strides`` (None = row-major)."""
    name: str
    src: QTensor
    dst_dt: int
    dst_strides: Optional[Tuple[int, ...]] = None
    quant: Dict[str, Quant] = field(default_factory=dict)  # src_scale, dst_scale, src_zp, dst_zp
    beta: float = 0.0  # scale of a sum post-op (0 = none)
    dst_init: Optional[np.ndarray] = None  # dst storage before the call (sum)

    def __post_init__(self):
        if self.dst_strides is None:
            self.dst_strides = QTensor(self.src.data, self.src.dt, self.src.dims).strides

    def dst_nelems(self) -> int:
        """Elements the dst buffer spans (largest offset + 1)."""
        return 1 + sum((d - 1) * s for d, s in zip(self.src.dims, self.dst_strides))


@dataclass
class PostOp:
    kind: int
    alg: int = 0
    alpha: float = 0.0
    beta: float = 0.0
    scale: float = 1.0
    zero_point: int = 0
    src1: Optional[QTensor] = None


@dataclass
class Problem:
    name: str
    M: int
    N: int
    K: int
    src: QTensor
    wei: QTensor
    dst_dt: int
    bias: Optional[QTensor] = None
    # keys: src_scale wei_scale dst_scale src_zp wei_zp dst_zp src_pr
    quant: Dict[str, Quant] = field(default_factory=dict)
    post_ops: List[PostOp] = field(default_factory=list)
    apply_to_int: bool = False
    fpmath: int = 0  # dnnl_fpmath_mode_t: 0 strict, 1 bf16, 2 f16, 3 any, 4 tf32
    # grouped (MoE) problems: cumulative END row of each group
    offsets: Optional[np.ndarray] = None
    dst_init: Optional[np.ndarray] = None  # dst contents before the call (sum)

    @property
    def groups(self) -> int:
        return 0 if self.offsets is None else int(self.offsets.shape[0])

    def ops(self) -> int:
        return 2 * self.M * self.N * self.K

    def algorithmic_bytes(self) -> int:
        """Inputs and outputs touched once, no workspace."""
        b = self.src.data.nbytes + self.wei.data.nbytes
        b += nbytes(self.dst_dt, self.M * self.N)
        if self.bias is not None:
            b += self.bias.data.nbytes
        for q in self.quant.values():
            b += q.data.nbytes
        for po in self.post_ops:
            if po.src1 is not None:
                b += po.src1.data.nbytes
        if self.offsets is not None:
            b += 2 * self.offsets.nbytes
        return b

    def take_rows(self, rows: np.ndarray) -> "Problem":
        """The sub-problem made of the given src rows (dense problems only):
        every dst element depends on one src row, so its result equals the
        same rows of the full problem."""
        assert self.offsets is None
        rows = np.asarray(rows, dtype=np.int64)
        assert self.src.dt not in (S4, U4)
        src2d = self.src.data.reshape(self.M, self.K)
        q = {}
        for k, v in self.quant.items():
            if k.startswith("src") and (v.mask & 1):
                d = v.data.reshape(self.M, -1)[rows]
                q[k] = Quant(np.ascontiguousarray(d), v.dt, v.mask, v.groups)
            else:
                q[k] = v
        pos = []
        for po in self.post_ops:
            if po.src1 is not None and po.src1.dims[0] == self.M and self.M > 1:
                d = po.src1.data.reshape(self.M, -1)[rows]
                t = QTensor(np.ascontiguousarray(d), po.src1.dt, (len(rows), po.src1.dims[1]))
                pos.append(PostOp(po.kind, po.alg, po.alpha, po.beta, po.scale, po.zero_point, t))
            else:
                pos.append(po)
        bias = self.bias
        if bias is not None and bias.dims[0] == self.M and self.M > 1:
            bias = QTensor(np.ascontiguousarray(bias.data.reshape(self.M, -1)[rows]), bias.dt,
                           (len(rows), bias.dims[1]))
        return Problem(self.name + "/rows", len(rows), self.N, self.K,
                       QTensor(np.ascontiguousarray(src2d[rows]), self.src.dt, (len(rows), self.K)),
                       self.wei, self.dst_dt, bias, q, pos, self.apply_to_int)


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


# ------------------------------------------------------------------ workloads
def int8_zp(M=256, K=1024, N=1024, dst_dt=S32, per_n_scales=False, seed=20261) -> Problem:
    """u8 src with per-tensor zero-point 128, s8 weights; dst s32 bit-exact,
    or f32 with per-N weight scales."""
    r = _rng(seed)
    src = r.integers(0, 256, (M, K), dtype=np.int64).astype(np.uint8)
    wei = r.integers(-127, 128, (K, N), dtype=np.int64).astype(np.int8)
    q = {"src_zp": Quant(np.array([128], np.int32), S32, 0)}
    if per_n_scales:
        q["wei_scale"] = Quant(r.uniform(0.001, 0.01, (1, N)).astype(np.float32), F32, 2)
        dst_dt = F32
    return Problem("int8_zp", M, N, K, QTensor(src, U8, (M, K)), QTensor(wei, S8, (K, N)),
                   dst_dt, quant=q)


def fp8_prefill(M=4096, K=4096, N=14336, seed=20262, src_dt=F8_E4M3, wei_dt=F8_E4M3) -> Problem:
    """e4m3 x e4m3 -> bf16 with per-tensor f32 scales and a bf16 bias."""
    r = _rng(seed)
    fac = 448.0 / 6.0
    src = to_storage(r.standard_normal((M, K), dtype=np.float32) * fac, src_dt)
    wei = to_storage(r.standard_normal((K, N), dtype=np.float32) * fac, wei_dt)
    bias = f32_to_bf16(r.standard_normal((1, N), dtype=np.float32))
    q = {"src_scale": Quant(np.array([1.0 / fac], np.float32), F32, 0),
         "wei_scale": Quant(np.array([1.0 / fac], np.float32), F32, 0)}
    return Problem("fp8_prefill", M, N, K, QTensor(src, src_dt, (M, K)),
                   QTensor(wei, wei_dt, (K, N)), BF16, QTensor(bias, BF16, (1, N)), q)


def int4_decode(M=1, K=8192, N=28672, group=128, seed=20263, wei_dt=S4, zp_dt=U4,
                src_dt=BF16, with_zp=True, dst_dt=BF16) -> Problem:
    """bf16 src x s4 weights with bf16 scales and u4 zero-points per
    (K/group, N); fpmath bf16 with apply_to_int (weights decompression)."""
    r = _rng(seed)
    src = to_storage(r.standard_normal((M, K), dtype=np.float32), src_dt)
    if wei_dt == S4:
        w = r.integers(-8, 8, (K, N), dtype=np.int64)
    elif wei_dt == U4:
        w = r.integers(0, 16, (K, N), dtype=np.int64)
    elif wei_dt == S8:
        w = r.integers(-127, 128, (K, N), dtype=np.int64)
    else:
        w = r.integers(0, 256, (K, N), dtype=np.int64)
    wei = to_storage(w, wei_dt)
    G = K // group
    q = {"wei_scale": Quant(f32_to_bf16(r.uniform(0.005, 0.02, (G, N)).astype(np.float32)),
                            BF16, 3, (group, 1))}
    if with_zp:
        z = r.integers(0, 16, (G, N), dtype=np.int64)
        q["wei_zp"] = Quant(to_storage(z, zp_dt), zp_dt, 3, (group, 1))
    return Problem("int4_decode", M, N, K, QTensor(src, src_dt, (M, K)),
                   QTensor(wei, wei_dt, (K, N)), dst_dt, quant=q, apply_to_int=True,
                   fpmath=2 if src_dt == F16 else 1)


def int8_postops(M=2048, K=4096, N=11008, seed=20264, dst_scale=None) -> Problem:
    """s8 x s8 with per-row src scales and per-N weight scales, + f32 bias,
    gelu_tanh, + f32 residual, requantized to s8 (dst scale, zero-point 0)."""
    r = _rng(seed)
    src = r.integers(-64, 64, (M, K), dtype=np.int64).astype(np.int8)
    wei = r.integers(-127, 128, (K, N), dtype=np.int64).astype(np.int8)
    ss = r.uniform(0.001, 0.01, (M, 1)).astype(np.float32)
    ws = r.uniform(0.001, 0.01, (1, N)).astype(np.float32)
    bias = r.standard_normal((1, N), dtype=np.float32)
    resid = r.standard_normal((M, N), dtype=np.float32)
    if dst_scale is None:
        # typical |y| after the chain is a few units for these ranges; spread
        # it over most of the s8 range
        dst_scale = 0.06 * np.sqrt(K / 4096.0)
    q = {"src_scale": Quant(ss, F32, 1), "wei_scale": Quant(ws, F32, 2),
         "dst_scale": Quant(np.array([dst_scale], np.float32), F32, 0),
         "dst_zp": Quant(np.array([0], np.int32), S32, 0)}
    po = [PostOp(PO_ELTWISE, ELTWISE["gelu_tanh"], 0.0, 0.0, 1.0),
          PostOp(PO_BINARY, BINARY["add"], src1=QTensor(resid, F32, (M, N)))]
    return Problem("int8_postops", M, N, K, QTensor(src, S8, (M, K)), QTensor(wei, S8, (K, N)),
                   S8, QTensor(bias, F32, (1, N)), q, po)


def zipf_group_sizes(total: int, groups: int, a: float = 1.1, seed: int = 20265) -> np.ndarray:
    """`total` draws from Zipf(a) truncated to ranks 1..groups, counted per rank."""
    r = _rng(seed)
    p = 1.0 / np.arange(1, groups + 1, dtype=np.float64) ** a
    p /= p.sum()
    return np.bincount(r.choice(groups, size=total, p=p), minlength=groups).astype(np.int64)


def moe_grouped(total_M=8192, K=4096, N=14336, experts=64, seed=20265, sizes=None) -> Problem:
    """Grouped (MoE) matmul: bf16 src rows concatenated in expert order, s8
    weights [E,K,N] with per-(expert,N) f32 scales, bf16 dst."""
    r = _rng(seed)
    if sizes is None:
        sizes = zipf_group_sizes(total_M, experts, seed=seed)
    sizes = np.asarray(sizes, dtype=np.int64)
    assert sizes.sum() == total_M and len(sizes) == experts
    offsets = np.cumsum(sizes).astype(np.int32)
    src = f32_to_bf16(r.standard_normal((total_M, K), dtype=np.float32))
    wei = r.integers(-127, 128, (experts, K, N), dtype=np.int8)
    ws = r.uniform(0.001, 0.01, (experts, 1, N)).astype(np.float32)
    q = {"wei_scale": Quant(ws, F32, 0b101)}
    return Problem("moe_grouped", total_M, N, K, QTensor(src, BF16, (total_M, K)),
                   QTensor(wei, S8, (experts, K, N)), BF16, quant=q, apply_to_int=True, fpmath=1,
                   offsets=offsets)
