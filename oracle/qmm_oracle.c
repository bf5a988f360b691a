/*
 * CPU oracle for the quantized matmul path -- TEST INFRASTRUCTURE ONLY.
 * See qmm_oracle.h.  Compile with gcc -O2 -fopenmp -ffp-contract=off: the
 * reference is built without FMA contraction, and the loops below keep its
 * summation order, so results are bit-identical to it (checked against
 * outputs of the reference library in tests/golden/).
 */
#include "qmm_oracle.h"

#include <math.h>
#include <string.h>

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ---- low-precision scalar types ---------------------------------------- */

/* src/common/bfloat16.cpp:22-47: RNE, f32 subnormals flush to signed zero,
 * NaN quieted. */
static uint16_t f32_to_bf16(float f) {
    uint32_t r = f2u(f);
    switch (fpclassify(f)) {
        case FP_SUBNORMAL:
        case FP_ZERO: return (uint16_t)(r >> 16) & 0x8000;
        case FP_INFINITE: return (uint16_t)(r >> 16);
        case FP_NAN: return (uint16_t)(r >> 16) | (1 << 6);
        default: {
            uint32_t lsb = (r >> 16) & 1u;
            return (uint16_t)((r + 0x7FFFu + lsb) >> 16);
        }
    }
}
static float bf16_to_f32(uint16_t b) { return u2f((uint32_t)b << 16); }

/* src/common/float16.hpp:50-92 */
static uint16_t f32_to_f16(float f) {
    uint32_t i = f2u(f);
    uint32_t s = i >> 31, e = (i >> 23) & 0xFF, m = i & 0x7FFFFF;
    uint32_t mm = m >> 13, r = m & 0x1FFF, ee = 0;
    int32_t eee = (int32_t)e - 127 + 15;
    if (e == 0) {
        ee = 0; mm = 0;
    } else if (e == 0xFF) {
        ee = 0x1F;
        if (m != 0) mm |= 0x200;
    } else if (eee > 0 && eee < 0x1F) {
        ee = (uint32_t)eee;
        if (r > (0x1000 - (mm & 1))) {
            mm++;
            if (mm == 0x400) { mm = 0; ee++; }
        }
    } else if (eee >= 0x1F) {
        ee = 0x1F; mm = 0;
    } else {
        float ff = fabsf(f) + 0.5f;
        ee = 0;
        mm = f2u(ff) & 0x7FF;
    }
    return (uint16_t)((s << 15) | (ee << 10) | mm);
}
/* src/common/float16.hpp:94-120 */
static float f16_to_f32(uint16_t h) {
    uint32_t ss = h >> 15, ee = (h >> 10) & 0x1F, mm = h & 0x3FF;
    uint32_t m = mm << 13, e;
    if (ee == 0) {
        if (mm == 0) e = 0;
        else return (ss ? -1.f : 1.f) * scalbnf((float)mm, -24);
    } else if (ee == 0x1F) {
        e = 0xFF;
        if (m != 0) m |= 0x400000;
    } else
        e = ee - 15 + 127;
    return u2f((ss << 31) | (e << 23) | m);
}
/* src/common/float8.cpp:346-375 (e4m3 -> f16 -> f32); OCP e4m3: bias 7,
 * S.1111.111 is NaN, no infinities */
static float e4m3_to_f32(uint8_t b) {
    uint16_t s8 = (b & 0x80) >> 7, e8 = (b & 0x78) >> 3, m8 = b & 7;
    uint16_t e16 = e8 + 8, m16 = m8;
    if (e8 == 0 && m8 != 0) {
        uint16_t count = 2;
        count = m8 > 1 ? 1 : count;
        count = m8 > 3 ? 0 : count;
        e16 -= count;
        m16 = (m16 << (count + 1)) & 7;
    } else if (e8 == 0 && m8 == 0) {
        e16 = 0;
    } else if (e8 == 0xF && m8 == 7) {
        e16 = 0x1F; m16 = 4;
    }
    return f16_to_f32((uint16_t)((s8 << 15) | (e16 << 10) | (m16 << 7)));
}
/* e5m2 is the upper byte of an IEEE half (src/common/float8.cpp:47-110) */
static float e5m2_to_f32(uint8_t b) { return f16_to_f32((uint16_t)b << 8); }

/* f16 -> e4m3, src/common/float8.cpp:216-267: round to nearest even; above
 * 464 (and NaN / inf) the result is NaN S.1111.111, at or below 2^-10 a signed
 * zero.  The reference rounds by adding and subtracting a shifter constant;
 * the integer form below gives the same nearest-even result. */
static uint8_t f16_to_e4m3(uint16_t h) {
    uint8_t s = (uint8_t)((h & 0x8000) >> 8);
    uint32_t a = h & 0x7fff;
    if (a > 0x5f40) return s | 0x7f;
    if (a <= 0x1400) return s;
    uint32_t e16 = a >> 10, m = a & 0x3ff, v, rem, half;
    if (e16 >= 9) { /* normal target: e8 = e16 - 8, three of ten mantissa bits stay */
        v = ((e16 - 8) << 3) | (m >> 7);
        rem = m & 0x7f;
        half = 0x40;
    } else { /* subnormal target, unit 2^-9: (1024 + m) * 2^(e16 - 16) units */
        uint32_t sig = 1024 + m, sh = 16 - e16;
        v = sig >> sh;
        rem = sig & ((1u << sh) - 1);
        half = 1u << (sh - 1);
    }
    if (rem > half || (rem == half && (v & 1))) v++;
    return (uint8_t)(s | v);
}
/* f16 -> e5m2, src/common/float8.cpp:47-73: NaN keeps its sign and gets the
 * quiet bit, infinity passes, everything else rounds to nearest even on the
 * raw bits (an overflow carries into infinity) */
static uint8_t f16_to_e5m2(uint16_t h) {
    int special = (h & 0x7c00) == 0x7c00;
    if (special && (h & 0x03ff)) return (uint8_t)((h >> 8) | 0x02);
    if (special) return (uint8_t)(h >> 8);
    return (uint8_t)((uint16_t)(h + 0x007f + ((h & 0x0100) >> 8)) >> 8);
}

/* ---- typed loads / stores (src/cpu/ref_io_helper.hpp:34-150) ------------ */

/* src/common/nibble.hpp:28-65, int4.hpp:28-68: element i lives in byte i/2,
 * low nibble when i is even; s4 is 4-bit two's complement */
static inline int load_nibble(const void *p, int64_t i, int is_signed) {
    uint8_t byte = ((const uint8_t *)p)[i / 2];
    int v = (i % 2) ? (byte >> 4) : (byte & 0xF);
    if (is_signed && (v & 8)) v -= 16;
    return v;
}

int qmm_load_int(int32_t dt, const void *p, int64_t i) {
    switch (dt) {
        case QMM_S32: return ((const int32_t *)p)[i];
        case QMM_S8: return ((const int8_t *)p)[i];
        case QMM_U8: return ((const uint8_t *)p)[i];
        case QMM_S4: return load_nibble(p, i, 1);
        case QMM_U4: return load_nibble(p, i, 0);
        default: return 0x7fffffff;
    }
}

float qmm_load_float(int32_t dt, const void *p, int64_t i) {
    switch (dt) {
        case QMM_F32: return ((const float *)p)[i];
        case QMM_BF16: return bf16_to_f32(((const uint16_t *)p)[i]);
        case QMM_F16: return f16_to_f32(((const uint16_t *)p)[i]);
        case QMM_F8_E4M3: return e4m3_to_f32(((const uint8_t *)p)[i]);
        case QMM_F8_E5M2: return e5m2_to_f32(((const uint8_t *)p)[i]);
        case QMM_S32: return (float)((const int32_t *)p)[i];
        case QMM_S8: return (float)((const int8_t *)p)[i];
        case QMM_U8: return (float)((const uint8_t *)p)[i];
        case QMM_S4: return (float)load_nibble(p, i, 1);
        case QMM_U4: return (float)load_nibble(p, i, 0);
        default: return NAN;
    }
}

/* saturate_and_round, src/cpu/simple_q10n.hpp:41-81: integer targets clamp to
 * [lowest, max] (the s32 upper bound is the largest float below 2^31,
 * src/common/type_helpers.hpp:222-232) and round with nearbyintf under the
 * default rounding mode (src/common/math_utils.hpp:125-132). */
void qmm_store_float(int32_t dt, float v, void *p, int64_t i) {
    switch (dt) {
        case QMM_F32: ((float *)p)[i] = v; break;
        case QMM_BF16: ((uint16_t *)p)[i] = f32_to_bf16(v); break;
        case QMM_F16: ((uint16_t *)p)[i] = f32_to_f16(v); break;
        /* float -> f8 goes through f16 (float8.cpp:269-274, 112-117) */
        case QMM_F8_E4M3: ((uint8_t *)p)[i] = f16_to_e4m3(f32_to_f16(v)); break;
        case QMM_F8_E5M2: ((uint8_t *)p)[i] = f16_to_e5m2(f32_to_f16(v)); break;
        case QMM_S32: {
            if (v < -2147483648.f) v = -2147483648.f;
            if (v > 2147483520.f) v = 2147483520.f;
            ((int32_t *)p)[i] = (int32_t)nearbyintf(v);
        } break;
        case QMM_S8: {
            if (v < -128.f) v = -128.f;
            if (v > 127.f) v = 127.f;
            ((int8_t *)p)[i] = (int8_t)(int)nearbyintf(v);
        } break;
        case QMM_U8: {
            if (v < 0.f) v = 0.f;
            if (v > 255.f) v = 255.f;
            ((uint8_t *)p)[i] = (uint8_t)(int)nearbyintf(v);
        } break;
        default: break;
    }
}

/* ---- eltwise / binary scalars ------------------------------------------ */

/* src/common/math_utils.hpp:140-420 */
static float logistic(float s) {
    float in = -s;
    return in < 88.72283172607421875f ? 1.f / (1.f + expf(in)) : 0.f;
}
static float soft_relu(float s, float alpha) {
    float in = s * alpha;
    float v = in < 88.72283172607421875f ? log1pf(expf(in)) : in;
    return v / alpha;
}
static float hardsigmoid(float s, float a, float b) {
    float v = a * s + b;
    return v <= 0.f ? 0.f : v >= 1.f ? 1.f : v;
}

float qmm_eltwise(int32_t alg, float s, float a, float b) {
    switch (alg) {
        case QMM_ELT_RELU: return s > 0 ? s : s * a;
        case QMM_ELT_TANH: return tanhf(s);
        case QMM_ELT_ELU: return s > 0 ? s : a * expm1f(s);
        case QMM_ELT_SQUARE: return s * s;
        case QMM_ELT_ABS: return s > 0 ? s : -s;
        case QMM_ELT_SQRT: return sqrtf(s);
        case QMM_ELT_LINEAR: return a * s + b;
        case QMM_ELT_SOFT_RELU: return soft_relu(s, a);
        case QMM_ELT_HARDSIGMOID: return hardsigmoid(s, a, b);
        case QMM_ELT_LOGISTIC: return logistic(s);
        case QMM_ELT_EXP: return expf(s);
        case QMM_ELT_GELU_TANH: {
            /* math_utils.hpp:313-319: tanh argument in f32, the final
             * product in double, then narrowed */
            const float c0 = 0.79788458347320556640625f, c1 = 0.044715f;
            float v = tanhf(c0 * s * (1 + c1 * s * s));
            return (float)(0.5 * s * (1. + v));
        }
        case QMM_ELT_SWISH: return s * logistic(a * s);
        case QMM_ELT_LOG: return logf(s);
        case QMM_ELT_CLIP: s = s > a ? s : a; return s > b ? b : s;
        case QMM_ELT_CLIP_V2: s = s > a ? s : a; return s < b ? s : b;
        case QMM_ELT_POW: return a * powf(s, b);
        case QMM_ELT_GELU_ERF:
            return 0.5f * s * (1.f + erff(s * 0.707106769084930419921875f));
        case QMM_ELT_ROUND: return nearbyintf(s);
        case QMM_ELT_MISH: return s * tanhf(soft_relu(s, 1.f));
        case QMM_ELT_HARDSWISH: return s * hardsigmoid(s, a, b);
        default: return NAN;
    }
}

/* src/cpu/primitive_attr_postops.cpp:30-47 */
static float binary_op(int32_t alg, float x, float y) {
    switch (alg) {
        case QMM_BIN_ADD: return x + y;
        case QMM_BIN_MUL: return x * y;
        case QMM_BIN_MAX: return x > y ? x : y;
        case QMM_BIN_MIN: return x < y ? x : y;
        case QMM_BIN_DIV: return x / y;
        case QMM_BIN_SUB: return x - y;
        case 0x1fff6: return x >= y;
        case 0x1fff7: return x > y;
        case 0x1fff8: return x <= y;
        case 0x1fff9: return x < y;
        case 0x1fffa: return x == y;
        case 0x1fffb: return x != y;
        default: return NAN;
    }
}

/* ordered chain, src/cpu/primitive_attr_postops.cpp:312-394 */
static float run_post_ops(const qmm_problem_t *p, float res, float dst_old,
        int64_t m, int64_t n) {
    for (int i = 0; i < p->n_po; ++i) {
        const qmm_postop_t *e = &p->po[i];
        if (e->kind == QMM_PO_SUM) {
            res += e->scale * (dst_old - (float)e->zero_point);
        } else if (e->kind == QMM_PO_ELTWISE) {
            res = qmm_eltwise(e->alg, res, e->alpha, e->beta) * e->scale;
        } else if (e->kind == QMM_PO_BINARY) {
            float y = qmm_load_float(
                    e->src1_dt, e->src1, m * e->src1_sm + n * e->src1_sn);
            res = binary_op(e->alg, res, y);
        } else if (e->kind == QMM_PO_PRELU) {
            /* primitive_attr_postops.cpp:363-389: non-negative values pass;
             * the others are multiplied by the f32 weight of their position
             * (src1 holds the weights over the masked dst dims) */
            if (!(res >= 0))
                res = ((const float *)e->src1)[m * e->src1_sm + n * e->src1_sn]
                        * res;
        }
    }
    return res;
}

/* matmul_helper_t::get_quant_off, src/cpu/matmul/matmul_utils.hpp:154-173,
 * specialised to 2D: masked index, last two dims divided by their groups,
 * row-major offset in the parameter buffer */
static inline int64_t quant_off(const qmm_quant_t *q, int64_t i0, int64_t i1) {
    int64_t a = (q->mask & 1) ? i0 / q->g0 : 0;
    int64_t b = (q->mask & 2) ? i1 / q->g1 : 0;
    return a * q->ld + b;
}

static inline int64_t ngroups_k(const qmm_quant_t *q, int64_t K, int kdim) {
    int64_t g = kdim == 0 ? q->g0 : q->g1;
    return (q->ptr && g > 1) ? K / g : 1;
}
static inline int64_t max64(int64_t a, int64_t b) { return a > b ? a : b; }

static void finish_and_store(const qmm_problem_t *p, float d, int64_t m,
        int64_t n) {
    const int64_t dst_off = m * p->dst_sm + n * p->dst_sn;
    if (p->non_default_attr) {
        float dst_old = 0.f;
        for (int i = 0; i < p->n_po; ++i)
            if (p->po[i].kind == QMM_PO_SUM)
                dst_old = qmm_load_float(p->sum_dt, p->dst, dst_off);
        d = run_post_ops(p, d, dst_old, m, n);
        if (p->dst_scale.ptr)
            d /= qmm_load_float(p->dst_scale.dt, p->dst_scale.ptr, 0);
        if (p->dst_zp.ptr) {
            int64_t zi = (p->dst_zp.mask > 0) ? n : 0;
            d += (float)qmm_load_int(QMM_S32, p->dst_zp.ptr, zi);
        }
    }
    qmm_store_float(p->dst_dt, d, p->dst, dst_off);
}

/* ---- ref_matmul_int8_t::execute_ref (ref_matmul_int8.cpp:40-309) -------- */
int qmm_oracle_int8(const qmm_problem_t *p) {
    const int64_t K = p->K;
    if (p->M == 0 || p->N == 0 || K == 0) return 0;
    const int with_src_zp = p->src_zp.ptr != 0;
    const int with_wei_zp = p->wei_zp.ptr != 0;
    const int with_pr = p->src_pr.ptr != 0;
    int64_t ng = max64(ngroups_k(&p->src_zp, K, 1), ngroups_k(&p->wei_zp, K, 0));
    ng = max64(ng, max64(ngroups_k(&p->src_scale, K, 1),
                           ngroups_k(&p->wei_scale, K, 0)));
    ng = max64(ng, ngroups_k(&p->src_pr, K, 1));
    const int64_t gk = K / ng;
    const int64_t nrows = p->rows ? p->n_rows : p->M;

#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t r = 0; r < nrows; ++r)
        for (int64_t n = 0; n < p->N; ++n) {
            const int64_t m = p->rows ? p->rows[r] : r;
            float d = 0;
            for (int64_t g = 0; g < ng; ++g) {
                int acc = 0;
                for (int64_t kk = 0; kk < gk; ++kk) {
                    const int64_t k = kk + g * gk;
                    int s = qmm_load_int(
                            p->src_dt, p->src, m * p->src_sm + k * p->src_sk);
                    int w = qmm_load_int(
                            p->wei_dt, p->wei, k * p->wei_sk + n * p->wei_sn);
                    if (with_src_zp)
                        s -= qmm_load_int(p->src_zp.dt, p->src_zp.ptr,
                                quant_off(&p->src_zp, m, k));
                    if (with_wei_zp && !with_pr)
                        w -= qmm_load_int(p->wei_zp.dt, p->wei_zp.ptr,
                                quant_off(&p->wei_zp, k, n));
                    acc += s * w;
                }
                if (with_pr) {
                    const int64_t k0 = g * gk;
                    int pr = qmm_load_int(p->src_pr.dt, p->src_pr.ptr,
                            quant_off(&p->src_pr, m, k0));
                    int wz = qmm_load_int(p->wei_zp.dt, p->wei_zp.ptr,
                            quant_off(&p->wei_zp, k0, n));
                    acc -= pr * wz;
                    if (with_src_zp) {
                        int sz = qmm_load_int(p->src_zp.dt, p->src_zp.ptr,
                                quant_off(&p->src_zp, m, k0));
                        acc += (int)(gk * wz * sz);
                    }
                }
                float acc_f = (float)acc;
                const int64_t k0 = g * gk;
                if (p->src_scale.ptr)
                    acc_f *= qmm_load_float(p->src_scale.dt, p->src_scale.ptr,
                            quant_off(&p->src_scale, m, k0));
                if (p->wei_scale.ptr)
                    acc_f *= qmm_load_float(p->wei_scale.dt, p->wei_scale.ptr,
                            quant_off(&p->wei_scale, k0, n));
                d += acc_f;
            }
            if (p->bias)
                d += qmm_load_float(
                        p->bias_dt, p->bias, m * p->bias_sm + n * p->bias_sn);
            finish_and_store(p, d, m, n);
        }
    return 0;
}

/* ---- ref_matmul_t::execute_ref (ref_matmul.cpp:55-428) ------------------
 * Static quantization only (no dropout, no dynamic dst scales). */
int qmm_oracle_fp(const qmm_problem_t *p) {
    const int64_t K = p->K;
    if (p->M == 0 || p->N == 0 || K == 0) return 0;
    const int wdt = p->wei_dt;
    const int decomp = p->apply_to_int
            && (wdt == QMM_S8 || wdt == QMM_U8 || wdt == QMM_S4 || wdt == QMM_U4);
    /* ref_matmul.cpp:137,147,169: the number of K groups is
     * max(K / src_group_k, K / wei_group_k) where a parameter without groups
     * (or an absent one) reports group 1 (primitive_attr_quant.hpp:91-93).
     * Hence unless BOTH scales are grouped along K every k is a group of its
     * own: each product is scaled and added to the result one by one. */
    const int64_t gs = (p->src_scale.ptr && p->src_scale.g1 > 1) ? p->src_scale.g1 : 1;
    const int64_t gw = (p->wei_scale.ptr && p->wei_scale.g0 > 1) ? p->wei_scale.g0 : 1;
    const int64_t ng = max64(K / gs, K / gw);
    const int64_t gk = K / ng;
    const int64_t nrows = p->rows ? p->n_rows : p->M;

#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t r = 0; r < nrows; ++r)
        for (int64_t n = 0; n < p->N; ++n) {
            const int64_t m = p->rows ? p->rows[r] : r;
            float res = 0.f;
            for (int64_t g = 0; g < ng; ++g) {
                float acc = 0.f;
                for (int64_t kk = 0; kk < gk; ++kk) {
                    const int64_t k = kk + g * gk;
                    const float s = qmm_load_float(
                            p->src_dt, p->src, m * p->src_sm + k * p->src_sk);
                    float w = qmm_load_float(
                            wdt, p->wei, k * p->wei_sk + n * p->wei_sn);
                    if (decomp) {
                        if (p->wei_zp.ptr)
                            w -= qmm_load_float(p->wei_zp.dt, p->wei_zp.ptr,
                                    quant_off(&p->wei_zp, k, n));
                        if (p->wei_scale.ptr)
                            w *= qmm_load_float(p->wei_scale.dt,
                                    p->wei_scale.ptr,
                                    quant_off(&p->wei_scale, k, n));
                    }
                    acc += s * w;
                }
                const int64_t k0 = g * gk;
                if (p->src_scale.ptr)
                    acc *= qmm_load_float(p->src_scale.dt, p->src_scale.ptr,
                            quant_off(&p->src_scale, m, k0));
                if (p->wei_scale.ptr && !decomp)
                    acc *= qmm_load_float(p->wei_scale.dt, p->wei_scale.ptr,
                            quant_off(&p->wei_scale, k0, n));
                res += acc;
            }
            if (p->bias)
                res += qmm_load_float(
                        p->bias_dt, p->bias, m * p->bias_sm + n * p->bias_sn);
            /* ref_matmul.cpp:298-321: post-ops only for non-default attr;
             * dst scale by division; no dst zero-point on this path */
            const int64_t dst_off = m * p->dst_sm + n * p->dst_sn;
            if (p->non_default_attr) {
                float dst_old = 0.f;
                for (int i = 0; i < p->n_po; ++i)
                    if (p->po[i].kind == QMM_PO_SUM)
                        dst_old = qmm_load_float(p->sum_dt, p->dst, dst_off);
                res = run_post_ops(p, res, dst_old, m, n);
            }
            if (p->dst_scale.ptr)
                res /= qmm_load_float(p->dst_scale.dt, p->dst_scale.ptr, 0);
            qmm_store_float(p->dst_dt, res, p->dst, dst_off);
        }
    return 0;
}

/* ---- ref_grouped_t::execute, 2D x 3D (ref_grouped_gemm.cpp:39-447) ------ */
int qmm_oracle_grouped(const qmm_problem_t *p) {
    const int64_t G = p->group_count, K = p->K, N = p->N;
    /* runtime offsets validation, ref_grouped_gemm.cpp:164-213 */
    for (int64_t g = 0; g < G; ++g) {
        int64_t b = g == 0 ? 0 : p->offsets[g - 1], e = p->offsets[g];
        if (b < 0 || e > p->M || e < b) return 2;
    }
    const int sdt = p->src_dt, wdt = p->wei_dt;
    const int wint = wdt == QMM_S8 || wdt == QMM_U8 || wdt == QMM_S4
            || wdt == QMM_U4;
    const int use_int = (sdt == QMM_S8 || sdt == QMM_U8) && wint;
    const int use_woq = (sdt == QMM_F32 || sdt == QMM_BF16 || sdt == QMM_F16)
            && wint && p->apply_to_int;
    const int64_t ss_ng = ngroups_k(&p->src_scale, K, 1);
    const int64_t ws_ng = ngroups_k(&p->wei_scale, K, 0);
    const int64_t sz_ng = ngroups_k(&p->src_zp, K, 1);
    const int64_t wz_ng = ngroups_k(&p->wei_zp, K, 0);
    const int64_t ng = max64(max64(ss_ng, ws_ng), max64(sz_ng, wz_ng));
    const int64_t gk = K / ng;

#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t gid = 0; gid < G; ++gid) {
        const int64_t row0 = gid == 0 ? 0 : p->offsets[gid - 1];
        const int64_t Mg = p->offsets[gid] - row0;
        const int64_t wbase = gid * p->wei_sg;
        for (int64_t mm = 0; mm < Mg; ++mm) {
            const int64_t m = row0 + mm;
            if (p->rows) { /* optional row subset */
                int hit = 0;
                for (int64_t r = 0; r < p->n_rows; ++r)
                    if (p->rows[r] == m) { hit = 1; break; }
                if (!hit) continue;
            }
            for (int64_t n = 0; n < N; ++n) {
                float result = 0.f;
                for (int64_t ig = 0; ig < ng; ++ig) {
                    int szp = 0, wzp = 0;
                    float wsc = 1.f;
                    if (use_int || use_woq) {
                        if (p->src_zp.ptr)
                            szp = qmm_load_int(p->src_zp.dt, p->src_zp.ptr,
                                    m * sz_ng + ig * sz_ng / ng);
                        if (p->wei_scale.ptr)
                            wsc = qmm_load_float(p->wei_scale.dt,
                                    p->wei_scale.ptr,
                                    gid * ws_ng * N + (ig * ws_ng / ng) * N + n);
                        if (p->wei_zp.ptr)
                            wzp = qmm_load_int(p->wei_zp.dt, p->wei_zp.ptr,
                                    gid * wz_ng * N + (ig * wz_ng / ng) * N + n);
                    }
                    float acc = 0.f;
                    if (use_int) {
                        int ai = 0;
                        for (int64_t kk = 0; kk < gk; ++kk) {
                            const int64_t k = kk + ig * gk;
                            int s = qmm_load_int(sdt, p->src,
                                    m * p->src_sm + k * p->src_sk);
                            int w = qmm_load_int(wdt, p->wei,
                                    wbase + k * p->wei_sk + n * p->wei_sn);
                            ai += (s - szp) * (w - wzp);
                        }
                        acc = (float)ai;
                    } else if (use_woq) {
                        for (int64_t kk = 0; kk < gk; ++kk) {
                            const int64_t k = kk + ig * gk;
                            float s = qmm_load_float(sdt, p->src,
                                    m * p->src_sm + k * p->src_sk);
                            int w = qmm_load_int(wdt, p->wei,
                                    wbase + k * p->wei_sk + n * p->wei_sn);
                            acc += s * (float)(w - wzp);
                        }
                    } else {
                        for (int64_t kk = 0; kk < gk; ++kk) {
                            const int64_t k = kk + ig * gk;
                            float s = qmm_load_float(sdt, p->src,
                                    m * p->src_sm + k * p->src_sk);
                            float w = qmm_load_float(wdt, p->wei,
                                    wbase + k * p->wei_sk + n * p->wei_sn);
                            acc += s * w;
                        }
                    }
                    if (p->src_scale.ptr)
                        acc *= qmm_load_float(p->src_scale.dt,
                                p->src_scale.ptr, m * ss_ng + ig * ss_ng / ng);
                    if (use_int || use_woq) {
                        result += acc * wsc;
                    } else {
                        if (p->wei_scale.ptr)
                            acc *= qmm_load_float(p->wei_scale.dt,
                                    p->wei_scale.ptr,
                                    gid * ws_ng * N + (ig * ws_ng / ng) * N + n);
                        result += acc;
                    }
                }
                if (p->bias)
                    result += qmm_load_float(
                            p->bias_dt, p->bias, gid * p->bias_sg + n);
                /* ref_grouped_gemm.cpp:399-440: eltwise and dense binary
                 * post-ops; a [G,1] binary operand is indexed by group */
                for (int i = 0; i < p->n_po; ++i) {
                    const qmm_postop_t *e = &p->po[i];
                    if (e->kind == QMM_PO_ELTWISE)
                        result = qmm_eltwise(e->alg, result, e->alpha, e->beta)
                                * e->scale;
                    else if (e->kind == QMM_PO_BINARY) {
                        /* zero_point != 0 flags a per-group [G,1] operand */
                        int64_t em = e->zero_point ? gid : m;
                        float y = qmm_load_float(e->src1_dt, e->src1,
                                em * e->src1_sm + n * e->src1_sn);
                        result = binary_op(e->alg, result, y);
                    }
                }
                qmm_store_float(
                        p->dst_dt, result, p->dst, m * p->dst_sm + n * p->dst_sn);
            }
        }
    }
    return 0;
}

/* ---- reorder -------------------------------------------------------------- */

/* get_quant_off, simple_reorder.hpp:184-201: the parameter tensor has the
 * data tensor's dims where the mask bit is set and 1 elsewhere, the last two
 * divided by the groups, dense row-major; a grouped index is idx / group. */
static int64_t rquant_off(const qmm_rquant_t *q, const qmm_reorder_t *r,
        const int64_t *idx) {
    int64_t off = 0;
    for (int d = 0; d < r->ndims; ++d) {
        int64_t g = 1;
        if (r->ndims >= 2 && d == r->ndims - 1) g = q->g1;
        if (r->ndims >= 2 && d == r->ndims - 2) g = q->g0;
        int64_t extent = (q->mask >> d) & 1 ? r->dims[d] / g : 1;
        int64_t i = (q->mask >> d) & 1 ? idx[d] / g : 0;
        off = off * extent + i;
    }
    return off;
}

static int is_int_dt(int32_t dt) {
    return dt == QMM_S32 || dt == QMM_S8 || dt == QMM_U8 || dt == QMM_S4
            || dt == QMM_U4;
}

static void store_nibble(void *p, int64_t i, float v, int is_signed) {
    /* saturate_and_round to the 4-bit range, nibble.hpp packing: even element
     * in the low half of byte i/2 */
    float lo = is_signed ? -8.f : 0.f, hi = is_signed ? 7.f : 15.f;
    if (v < lo) v = lo;
    if (v > hi) v = hi;
    int q = (int)nearbyintf(v) & 0xF;
    uint8_t *b = (uint8_t *)p + i / 2;
    *b = (i % 2) ? (uint8_t)((*b & 0x0F) | (q << 4)) : (uint8_t)((*b & 0xF0) | q);
}

int qmm_oracle_reorder(const qmm_reorder_t *r) {
    const int src4 = r->src_dt == QMM_S4 || r->src_dt == QMM_U4;
    const int dst4 = r->dst_dt == QMM_S4 || r->dst_dt == QMM_U4;
    if (r->ndims < 1 || r->ndims > QMM_MAX_DIMS) return 2;
    /* the reference's implementation lists: 4-bit targets only from f32 and
     * without arithmetic, 4-bit sources only to floating-point types and
     * without dst scales, dst zero-points or a sum */
    if (dst4
            && (r->src_dt != QMM_F32 || r->src_scale.ptr || r->dst_scale.ptr
                    || r->src_zp.ptr || r->dst_zp.ptr || r->beta != 0.f))
        return 3;
    if (src4
            && ((r->dst_dt != QMM_F32 && r->dst_dt != QMM_BF16
                        && r->dst_dt != QMM_F16)
                    || r->dst_scale.ptr || r->dst_zp.ptr || r->beta != 0.f))
        return 3;
    int64_t nelems = 1;
    for (int d = 0; d < r->ndims; ++d) nelems *= r->dims[d];
    const int32_t dst_zp
            = r->dst_zp.ptr ? ((const int32_t *)r->dst_zp.ptr)[0] : 0;
    for (int64_t l = 0; l < nelems; ++l) {
        int64_t idx[QMM_MAX_DIMS], rem = l, i_off = 0, o_off = 0;
        for (int d = r->ndims - 1; d >= 0; --d) {
            idx[d] = rem % r->dims[d];
            rem /= r->dims[d];
            i_off += idx[d] * r->src_strides[d];
            o_off += idx[d] * r->dst_strides[d];
        }
        if (dst4) {
            store_nibble(r->dst, o_off, ((const float *)r->src)[i_off],
                    r->dst_dt == QMM_S4);
            continue;
        }
        float src_scale = 1.f, dst_scale = 1.f;
        if (r->src_scale.ptr)
            src_scale = qmm_load_float(r->src_scale.dt, r->src_scale.ptr,
                    rquant_off(&r->src_scale, r, idx));
        if (r->dst_scale.ptr)
            dst_scale = ((const float *)r->dst_scale.ptr)[rquant_off(
                    &r->dst_scale, r, idx)];
        int zp = 0;
        if (r->src_zp.ptr)
            zp = (int)qmm_load_float(
                    r->src_zp.dt, r->src_zp.ptr, rquant_off(&r->src_zp, r, idx));
        /* input[i_off] - src_zp_val: integer arithmetic for integer sources,
         * float otherwise (the 4-bit path converts to the float type first) */
        float diff;
        if (is_int_dt(r->src_dt) && !src4)
            diff = (float)(qmm_load_int(r->src_dt, r->src, i_off) - zp);
        else
            diff = qmm_load_float(r->src_dt, r->src, i_off) - (float)zp;
        float d = src_scale * diff;
        if (!src4) {
            if (r->beta != 0.f)
                d += r->beta * qmm_load_float(r->dst_dt, r->dst, o_off);
            /* The scalar implementation adds the zero-point always (so a -0
             * result becomes +0); the library dispatches it only for reorders
             * with a sum.  Its JIT implementations, which serve the others,
             * add a zero-point only when the attribute is set and keep -0. */
            d = d / dst_scale;
            if (r->dst_zp.ptr || r->beta != 0.f) d += (float)dst_zp;
        }
        qmm_store_float(r->dst_dt, d, r->dst, o_off);
    }
    return 0;
}
