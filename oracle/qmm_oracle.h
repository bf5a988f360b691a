/*
 * CPU oracle for the quantized matmul path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic of oneDNN's scalar reference
 * matmuls (src/cpu/matmul/ref_matmul_int8.cpp, ref_matmul.cpp,
 * ref_grouped_gemm.cpp) and of the helpers they call.  Only tests, the smoke
 * check and the CPU-baseline leg of the benchmark may load this code; the
 * library proper never does.
 *
 * Every tensor is described by a base pointer, a data type code (the numeric
 * values of dnnl_data_type_t, include/oneapi/dnnl/dnnl_common_types.h:75-115)
 * and element strides, so the same entry points cover plain `ab`, transposed
 * `ba` and sub-byte layouts.
 */
#ifndef QMM_ORACLE_H
#define QMM_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    QMM_F16 = 1, QMM_BF16 = 2, QMM_F32 = 3, QMM_S32 = 4, QMM_S8 = 5,
    QMM_U8 = 6, QMM_F8_E5M2 = 9, QMM_F8_E4M3 = 10, QMM_S4 = 11, QMM_U4 = 12
};

enum { QMM_PO_SUM = 1, QMM_PO_ELTWISE = 2, QMM_PO_BINARY = 3, QMM_PO_PRELU = 4 };

/* eltwise / binary algorithm codes = dnnl_alg_kind_t values
 * (include/oneapi/dnnl/dnnl_types.h) */
enum {
    QMM_ELT_RELU = 0x20, QMM_ELT_TANH = 0x21, QMM_ELT_ELU = 0x22,
    QMM_ELT_SQUARE = 0x23, QMM_ELT_ABS = 0x24, QMM_ELT_SQRT = 0x25,
    QMM_ELT_LINEAR = 0x26, QMM_ELT_SOFT_RELU = 0x27, QMM_ELT_HARDSIGMOID = 0x28,
    QMM_ELT_LOGISTIC = 0x29, QMM_ELT_EXP = 0x2a, QMM_ELT_GELU_TANH = 0x2b,
    QMM_ELT_SWISH = 0x2c, QMM_ELT_LOG = 0x2d, QMM_ELT_CLIP = 0x2e,
    QMM_ELT_CLIP_V2 = 0x2f, QMM_ELT_POW = 0x30, QMM_ELT_GELU_ERF = 0x31,
    QMM_ELT_ROUND = 0x32, QMM_ELT_MISH = 0x33, QMM_ELT_HARDSWISH = 0x34,
    QMM_BIN_ADD = 0x1fff0, QMM_BIN_MUL = 0x1fff1, QMM_BIN_MAX = 0x1fff2,
    QMM_BIN_MIN = 0x1fff3, QMM_BIN_DIV = 0x1fff4, QMM_BIN_SUB = 0x1fff5
};

/* One quantization parameter (scale / zero-point / precomputed reduction).
 * The buffer is dense row-major over the masked dims of its tensor with the
 * last two dims divided by the groups (primitive_attr_quant.hpp:116-140). */
typedef struct {
    const void *ptr; /* NULL = parameter absent (default attr) */
    int32_t dt;
    int32_t mask; /* bit0 = dim 0 of the 2D tensor, bit1 = dim 1 */
    int64_t g0, g1; /* group sizes along dim 0 and dim 1 (>= 1) */
    int64_t ld; /* row pitch of the parameter buffer in elements */
} qmm_quant_t;

typedef struct {
    int32_t kind; /* QMM_PO_* */
    int32_t alg; /* eltwise or binary algorithm */
    float alpha, beta, scale; /* eltwise params; sum: scale */
    int32_t zero_point; /* sum only */
    int32_t src1_dt; /* binary only */
    const void *src1;
    int64_t src1_sm, src1_sn; /* element strides, 0 on a broadcast dim */
} qmm_postop_t;

typedef struct {
    int64_t M, N, K;
    const void *src;
    int32_t src_dt;
    int64_t src_sm, src_sk;
    const void *wei;
    int32_t wei_dt;
    int64_t wei_sk, wei_sn;
    const void *bias; /* NULL = none */
    int32_t bias_dt;
    int64_t bias_sm, bias_sn; /* 0 on a broadcast dim */
    void *dst;
    int32_t dst_dt;
    int64_t dst_sm, dst_sn;
    qmm_quant_t src_scale, wei_scale, dst_scale;
    qmm_quant_t src_zp, wei_zp, dst_zp;
    qmm_quant_t src_pr; /* precomputed reductions, int8 path only */
    int32_t apply_to_int; /* fpmath apply_to_int: weights decompression */
    int32_t non_default_attr; /* attr != default: run post-ops/dst quant */
    int32_t sum_dt; /* data type the sum post-op reads dst in */
    int32_t n_po;
    qmm_postop_t po[32];
    /* optional row subset: compute only these M rows (NULL = all) */
    const int64_t *rows;
    int64_t n_rows;
    /* grouped (2D x 3D) problems only */
    int64_t group_count;
    const int32_t *offsets; /* cumulative END row per group */
    int64_t wei_sg; /* weights stride between groups */
    int64_t bias_sg;
    /* dnnl_fpmath_mode_t value (0 strict, 1 bf16, 2 f16, 3 any, 4 tf32); only
     * the reference runner needs it, to build the same attribute */
    int32_t fpmath_mode;
} qmm_problem_t;

/* src in {s8,u8}: follows ref_matmul_int8.cpp:40-309. returns 0 on success */
int qmm_oracle_int8(const qmm_problem_t *p);
/* floating-point src (+ weights decompression): ref_matmul.cpp:55-428 */
int qmm_oracle_fp(const qmm_problem_t *p);
/* grouped 2D x 3D: ref_grouped_gemm.cpp:39-447; returns 2 (invalid
 * arguments) when the offsets are not monotone or exceed M */
int qmm_oracle_grouped(const qmm_problem_t *p);

/* ---- reorder (quantizing / dequantizing copy between plain layouts) ------- */
#define QMM_MAX_DIMS 6
typedef struct {
    const void *ptr; /* NULL = attribute not set */
    int32_t dt;
    int32_t mask; /* bit d set: one value per index of dim d */
    int64_t g0, g1; /* group sizes along the last two dims (1 = none) */
} qmm_rquant_t;

typedef struct {
    int32_t ndims;
    int64_t dims[QMM_MAX_DIMS];
    const void *src;
    int32_t src_dt;
    int64_t src_strides[QMM_MAX_DIMS]; /* elements */
    void *dst;
    int32_t dst_dt;
    int64_t dst_strides[QMM_MAX_DIMS];
    qmm_rquant_t src_scale, dst_scale, src_zp, dst_zp;
    float beta; /* scale of the sum post-op; 0 = no post-op */
} qmm_reorder_t;

/* simple_reorder.hpp reference implementations (:2168-2281 f32 -> 4-bit,
 * :2283-2425 4-bit -> float, :2527-2679 everything else).  Returns 3
 * (unimplemented) for combinations the reference has no implementation of. */
int qmm_oracle_reorder(const qmm_reorder_t *r);

/* scalar helpers exported for unit tests */
float qmm_load_float(int32_t dt, const void *ptr, int64_t idx);
int qmm_load_int(int32_t dt, const void *ptr, int64_t idx);
void qmm_store_float(int32_t dt, float v, void *ptr, int64_t idx);
float qmm_eltwise(int32_t alg, float s, float alpha, float beta);

#ifdef __cplusplus
}
#endif
#endif
