// Device-side scalar semantics shared by all kernels: typed loads/stores,
// eltwise/binary formulas and the ordered post-op chain.  The arithmetic
// follows oneDNN's reference helpers so results agree with its CPU matmul:
//   loads/stores   src/cpu/ref_io_helper.hpp:34-150, src/cpu/simple_q10n.hpp:41-81
//   bf16 rounding  src/common/bfloat16.cpp:22-47
//   eltwise        src/common/math_utils.hpp:140-420
//   chain order    src/cpu/primitive_attr_postops.cpp:312-394
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <math.h>

#include "kernel_args.h"

namespace qmm {

__device__ __forceinline__ float bf16_bits_to_f32(unsigned short b) {
    return __uint_as_float(((unsigned)b) << 16);
}

// RNE; f32 subnormal inputs flush to signed zero; NaN is quieted.
__device__ __forceinline__ unsigned short f32_to_bf16_bits(float f) {
    unsigned u = __float_as_uint(f);
    unsigned e = u & 0x7f800000u;
    if (e == 0) return (unsigned short)((u >> 16) & 0x8000u);
    if (e == 0x7f800000u) {
        if (u & 0x007fffffu) return (unsigned short)((u >> 16) | 0x40u);
        return (unsigned short)(u >> 16);
    }
    unsigned lsb = (u >> 16) & 1u;
    return (unsigned short)((u + 0x7fffu + lsb) >> 16);
}

__device__ __forceinline__ float e4m3_to_f32(unsigned char b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
    return __half2float(__half(h));
}
__device__ __forceinline__ float e5m2_to_f32(unsigned char b) {
    __half_raw h;
    h.x = (unsigned short)b << 8;
    return __half2float(__half(h));
}

// element i of a nibble-packed buffer: byte i/2, low nibble when i is even
__device__ __forceinline__ int load_nibble(const void *p, int64_t i, bool sgn) {
    unsigned byte = ((const unsigned char *)p)[i >> 1];
    int v = (i & 1) ? (byte >> 4) : (byte & 0xF);
    if (sgn && (v & 8)) v -= 16;
    return v;
}

__device__ __forceinline__ int load_int(int dt, const void *p, int64_t i) {
    switch (dt) {
        case DT_S32: return ((const int *)p)[i];
        case DT_S8: return ((const signed char *)p)[i];
        case DT_U8: return ((const unsigned char *)p)[i];
        case DT_S4: return load_nibble(p, i, true);
        case DT_U4: return load_nibble(p, i, false);
        default: return 0;
    }
}

__device__ __forceinline__ float load_float(int dt, const void *p, int64_t i) {
    switch (dt) {
        case DT_F32: return ((const float *)p)[i];
        case DT_BF16: return bf16_bits_to_f32(((const unsigned short *)p)[i]);
        case DT_F16: return __half2float(((const __half *)p)[i]);
        case DT_F8_E4M3: return e4m3_to_f32(((const unsigned char *)p)[i]);
        case DT_F8_E5M2: return e5m2_to_f32(((const unsigned char *)p)[i]);
        case DT_S32: return (float)((const int *)p)[i];
        case DT_S8: return (float)((const signed char *)p)[i];
        case DT_U8: return (float)((const unsigned char *)p)[i];
        case DT_S4: return (float)load_nibble(p, i, true);
        case DT_U4: return (float)load_nibble(p, i, false);
        default: return 0.f;
    }
}

// f32 -> f8 as the reference converts (src/common/float8.cpp:216-274, 47-117): through f16, then
// round to nearest even.  e4m3: above 464 (and NaN / inf) the result is NaN S.1111.111, at or
// below 2^-10 a signed zero.  e5m2: the upper byte of the rounded half, NaN with the quiet bit.
__device__ __forceinline__ unsigned char f32_to_e4m3_bits(float f) {
    const unsigned h = __half_as_ushort(__float2half_rn(f));
    const unsigned s = (h & 0x8000u) >> 8, a = h & 0x7fffu;
    if (a > 0x5f40u) return (unsigned char)(s | 0x7fu);
    if (a <= 0x1400u) return (unsigned char)s;
    const unsigned e16 = a >> 10, m = a & 0x3ffu;
    unsigned v, rem, half;
    if (e16 >= 9) { // normal target: three of the ten mantissa bits stay
        v = ((e16 - 8) << 3) | (m >> 7);
        rem = m & 0x7fu;
        half = 0x40u;
    } else { // subnormal target in units of 2^-9
        const unsigned sig = 1024u + m, sh = 16u - e16;
        v = sig >> sh;
        rem = sig & ((1u << sh) - 1u);
        half = 1u << (sh - 1u);
    }
    if (rem > half || (rem == half && (v & 1u))) ++v;
    return (unsigned char)(s | v);
}
__device__ __forceinline__ unsigned char f32_to_e5m2_bits(float f) {
    const unsigned h = __half_as_ushort(__float2half_rn(f));
    const bool special = (h & 0x7c00u) == 0x7c00u;
    if (special && (h & 0x03ffu)) return (unsigned char)((h >> 8) | 0x02u);
    if (special) return (unsigned char)(h >> 8);
    return (unsigned char)(((h + 0x007fu + ((h & 0x0100u) >> 8)) & 0xffffu) >> 8);
}

// saturate + round-half-even for integer targets; RNE for bf16/f16/f8
__device__ __forceinline__ void store_float(int dt, float v, void *p, int64_t i) {
    switch (dt) {
        case DT_F32: ((float *)p)[i] = v; break;
        case DT_BF16: ((unsigned short *)p)[i] = f32_to_bf16_bits(v); break;
        case DT_F16: ((__half *)p)[i] = __float2half_rn(v); break;
        case DT_F8_E4M3: ((unsigned char *)p)[i] = f32_to_e4m3_bits(v); break;
        case DT_F8_E5M2: ((unsigned char *)p)[i] = f32_to_e5m2_bits(v); break;
        case DT_S32: {
            v = fmaxf(v, -2147483648.f);
            v = fminf(v, 2147483520.f);
            ((int *)p)[i] = (v != v) ? (int)0x80000000 : __float2int_rn(v);
        } break;
        case DT_S8: {
            v = fminf(fmaxf(v, -128.f), 127.f);
            ((signed char *)p)[i] = (signed char)__float2int_rn(v);
        } break;
        case DT_U8: {
            v = fminf(fmaxf(v, 0.f), 255.f);
            ((unsigned char *)p)[i] = (unsigned char)__float2int_rn(v);
        } break;
        default: break;
    }
}

__device__ __forceinline__ float logistic_f(float s) {
    float in = -s;
    return in < 88.72283172607421875f ? __fdiv_rn(1.f, 1.f + expf(in)) : 0.f;
}
__device__ __forceinline__ float soft_relu_f(float s, float alpha) {
    float in = s * alpha;
    float v = in < 88.72283172607421875f ? log1pf(expf(in)) : in;
    return __fdiv_rn(v, alpha);
}
__device__ __forceinline__ float hardsigmoid_f(float s, float a, float b) {
    float v = __fadd_rn(__fmul_rn(a, s), b);
    return v <= 0.f ? 0.f : v >= 1.f ? 1.f : v;
}

// gelu_tanh as the reference evaluates it: the tanh argument in f32 (no
// fused multiply-adds), the final 0.5*s*(1+v) in double, then narrowed.
__device__ __forceinline__ float gelu_tanh_f(float s) {
    const float c0 = 0.79788458347320556640625f, c1 = 0.044715f;
    float t = __fmul_rn(__fmul_rn(c0, s),
            __fadd_rn(1.f, __fmul_rn(__fmul_rn(c1, s), s)));
    float v = tanhf(t);
    return (float)(0.5 * (double)s * (1. + (double)v));
}

// gelu_tanh for results that are requantized to 8-bit integers: the same tanh argument, tanh(t) =
// 1 - 2 / (exp(2t) + 1) through the hardware's exp2 and reciprocal approximations, and the final
// 0.5 s (1 + tanh t) = s - s / (exp(2t) + 1) in f32.  Absolute error below 4e-7 max(1, |s|), i.e.
// a few millionths of an s8 step for values inside the s8 range: the rounded integer differs from
// the reference's (by one) only where the reference value lies that close to a rounding boundary.
__device__ __forceinline__ float gelu_tanh_coarse(float s) {
    // 2 t log2(e) = s (k1 + k3 s^2): k1 = 2 log2(e) sqrt(2 / pi), k3 = 0.044715 k1
    const float k1 = 2.30220826355710f, k3 = 0.10294324250496f;
    const float t2 = s * fmaf(k3, s * s, k1);
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t2)); // exp(2t)
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.f));
    return fmaf(-s, r, s);
}

// d / scale with a reciprocal computed once (rcp = round(1 / scale)): product, exact remainder,
// correction -- the correctly rounded quotient whenever no intermediate over- or underflows
// (Markstein); an infinite or NaN product is returned as it is.
__device__ __forceinline__ float div_by_scale(float d, float scale, float rcp) {
    const float q = d * rcp;
    const float rem = fmaf(-q, scale, d);
    const float q2 = fmaf(rem, rcp, q);
    return fabsf(q) < __int_as_float(0x7f800000) ? q2 : q;
}

__device__ __forceinline__ float eltwise_fwd(int alg, float s, float a, float b) {
    switch (alg) {
        case 0x20: return s > 0 ? s : __fmul_rn(s, a); // relu
        case 0x21: return tanhf(s);
        case 0x22: return s > 0 ? s : __fmul_rn(a, expm1f(s)); // elu
        case 0x23: return __fmul_rn(s, s);
        case 0x24: return s > 0 ? s : -s;
        case 0x25: return sqrtf(s);
        case 0x26: return __fadd_rn(__fmul_rn(a, s), b); // linear
        case 0x27: return soft_relu_f(s, a);
        case 0x28: return hardsigmoid_f(s, a, b);
        case 0x29: return logistic_f(s);
        case 0x2a: return expf(s);
        case 0x2b: return gelu_tanh_f(s);
        case 0x2c: return __fmul_rn(s, logistic_f(__fmul_rn(a, s))); // swish
        case 0x2d: return logf(s);
        case 0x2e: s = s > a ? s : a; return s > b ? b : s; // clip
        case 0x2f: s = s > a ? s : a; return s < b ? s : b; // clip_v2
        case 0x30: return __fmul_rn(a, powf(s, b));
        case 0x31: // gelu_erf
            return __fmul_rn(__fmul_rn(0.5f, s),
                    __fadd_rn(1.f, erff(__fmul_rn(s, 0.707106769084930419921875f))));
        case 0x32: return rintf(s);
        case 0x33: return __fmul_rn(s, tanhf(soft_relu_f(s, 1.f))); // mish
        case 0x34: return __fmul_rn(s, hardsigmoid_f(s, a, b)); // hardswish
        default: return s;
    }
}

__device__ __forceinline__ float binary_op(int alg, float x, float y) {
    switch (alg) {
        case 0x1fff0: return __fadd_rn(x, y);
        case 0x1fff1: return __fmul_rn(x, y);
        case 0x1fff2: return x > y ? x : y;
        case 0x1fff3: return x < y ? x : y;
        case 0x1fff4: return __fdiv_rn(x, y);
        case 0x1fff5: return __fsub_rn(x, y);
        case 0x1fff6: return x >= y;
        case 0x1fff7: return x > y;
        case 0x1fff8: return x <= y;
        case 0x1fff9: return x < y;
        case 0x1fffa: return x == y;
        case 0x1fffb: return x != y;
        case ALG_PRELU: return x >= 0 ? x : __fmul_rn(y, x);
        default: return x;
    }
}

// Ordered post-op chain on one f32 value at dst position (m, n); `gid` is the
// expert index for grouped problems (per-group binary operands).
__device__ __forceinline__ float apply_post_ops(const MatmulArgs &a, float res,
        float dst_old, int64_t m, int64_t n, int gid) {
    for (int i = 0; i < a.n_po; ++i) {
        const PostOpArg &e = a.po[i];
        if (e.kind == PO_ELTWISE) {
            res = __fmul_rn(eltwise_fwd(e.alg, res, e.alpha, e.beta), e.scale);
        } else if (e.kind == PO_BINARY) {
            const int64_t em = e.per_group ? gid : m;
            float y = load_float(e.src1_dt, e.src1, em * e.sm + n * e.sn);
            res = binary_op(e.alg, res, y);
        } else if (e.kind == PO_SUM) {
            res = __fadd_rn(res,
                    __fmul_rn(e.scale, __fsub_rn(dst_old, (float)e.zero_point)));
        }
    }
    return res;
}

__device__ __forceinline__ bool has_sum(const MatmulArgs &a) {
    for (int i = 0; i < a.n_po; ++i)
        if (a.po[i].kind == PO_SUM) return true;
    return false;
}

// The same ordered chain applied to R values of one dst column n at rows
// m0 .. m0+R-1 held in registers.  Every post-op is one phase of straight-line
// code over the R values: its kind / algorithm / operand type is decided once
// per phase instead of once per element, and the R dependency chains
// interleave.  Rows at or beyond M (the tail of the last tile) read row M-1 of
// binary operands and old dst; their results are never stored.
// COARSE: the result is requantized to an 8-bit integer, which lets gelu_tanh use its cheap form.
// FULL: all R rows exist (m0 + R <= M), so no row index has to be clamped.
template <int R, bool COARSE = false, bool FULL = false>
__device__ __forceinline__ void apply_post_ops_rows(const MatmulArgs &a, float (&d)[R], int64_t m0, int64_t n) {
    for (int i = 0; i < a.n_po; ++i) {
        const PostOpArg &e = a.po[i];
        if (e.kind == PO_ELTWISE) {
            const float al = e.alpha, be = e.beta, sc = e.scale;
            switch (e.alg) {
#define QMM_ELT_PHASE(ALG, EXPR) \
    case ALG: \
        _Pragma("unroll") for (int j = 0; j < R; ++j) { const float s = d[j]; d[j] = __fmul_rn((EXPR), sc); } \
        break;
                QMM_ELT_PHASE(0x20, s > 0 ? s : __fmul_rn(s, al)) // relu
                QMM_ELT_PHASE(0x21, tanhf(s))
                QMM_ELT_PHASE(0x26, __fadd_rn(__fmul_rn(al, s), be)) // linear
                QMM_ELT_PHASE(0x29, logistic_f(s))
                QMM_ELT_PHASE(0x2b, COARSE ? gelu_tanh_coarse(s) : gelu_tanh_f(s))
                QMM_ELT_PHASE(0x2c, __fmul_rn(s, logistic_f(__fmul_rn(al, s)))) // swish
                QMM_ELT_PHASE(0x2e, ((s > al ? s : al) > be ? be : (s > al ? s : al))) // clip
                QMM_ELT_PHASE(0x31,
                        __fmul_rn(__fmul_rn(0.5f, s),
                                __fadd_rn(1.f, erff(__fmul_rn(s, 0.707106769084930419921875f))))) // gelu_erf
#undef QMM_ELT_PHASE
                default:
#pragma unroll
                    for (int j = 0; j < R; ++j) d[j] = __fmul_rn(eltwise_fwd(e.alg, d[j], al, be), sc);
            }
        } else if (e.kind == PO_BINARY) {
            float y[R];
            const char *base = (const char *)e.src1;
            const int64_t last = a.M - 1;
            const int64_t o0 = m0 * e.sm + n * e.sn; // element offset of row m0; row j lies j * sm further
            if (e.src1_dt == DT_F32) {
                const float *row = (const float *)base + o0;
#pragma unroll
                for (int j = 0; j < R; ++j) y[j] = FULL ? row[j * e.sm] : ((const float *)base)[min(m0 + j, last) * e.sm + n * e.sn];
            } else if (e.src1_dt == DT_BF16) {
                const unsigned short *row = (const unsigned short *)base + o0;
#pragma unroll
                for (int j = 0; j < R; ++j)
                    y[j] = bf16_bits_to_f32(FULL ? row[j * e.sm] : ((const unsigned short *)base)[min(m0 + j, last) * e.sm + n * e.sn]);
            } else {
#pragma unroll
                for (int j = 0; j < R; ++j)
                    y[j] = load_float(e.src1_dt, base, FULL ? o0 + j * e.sm : min(m0 + j, last) * e.sm + n * e.sn);
            }
            switch (e.alg) {
                case 0x1fff0:
#pragma unroll
                    for (int j = 0; j < R; ++j) d[j] = __fadd_rn(d[j], y[j]);
                    break;
                case 0x1fff1:
#pragma unroll
                    for (int j = 0; j < R; ++j) d[j] = __fmul_rn(d[j], y[j]);
                    break;
                default:
#pragma unroll
                    for (int j = 0; j < R; ++j) d[j] = binary_op(e.alg, d[j], y[j]);
            }
        } else if (e.kind == PO_SUM) {
            const int64_t last = a.M - 1;
#pragma unroll
            for (int j = 0; j < R; ++j) {
                const float old = load_float(a.sum_dt, a.dst, (FULL ? m0 + j : min(m0 + j, last)) * a.dst_sm + n * a.dst_sn);
                d[j] = __fadd_rn(d[j], __fmul_rn(e.scale, __fsub_rn(old, (float)e.zero_point)));
            }
        }
    }
}

// Everything after the K reduction for a dense problem: bias was already
// added by the caller.  Post-ops, dst scale (a division, as in the
// reference), dst zero-point, saturating store.
__device__ __forceinline__ void finish_store(const MatmulArgs &a, float d,
        int64_t m, int64_t n, bool int8_path) {
    const int64_t off = m * a.dst_sm + n * a.dst_sn;
    if (a.non_default_attr) {
        float old = 0.f;
        if (a.n_po && has_sum(a)) old = load_float(a.sum_dt, a.dst, off);
        d = apply_post_ops(a, d, old, m, n, 0);
        if (a.dst_scale.ptr)
            d = __fdiv_rn(d, load_float(a.dst_scale.dt, a.dst_scale.ptr, 0));
        else if (a.dst_scale.on_host)
            d = __fdiv_rn(d, a.dst_scale.host_value);
        if (int8_path && a.dst_zp.ptr)
            d = __fadd_rn(d,
                    (float)((const int *)a.dst_zp.ptr)[a.dst_zp.mask > 0 ? n : 0]);
    }
    store_float(a.dst_dt, d, a.dst, off);
}

// offset of the quantization parameter that applies to element (i0, i1)
__device__ __forceinline__ int64_t qoff(const QParam &q, int64_t i0, int64_t i1) {
    int64_t r = (q.mask & 1) ? i0 / q.g0 : 0;
    int64_t c = (q.mask & 2) ? i1 / q.g1 : 0;
    return r * q.ld + c;
}

} // namespace qmm
