/*
 * C ABI of the B200-native quantized matmul library.
 *
 * The library is a drop-in for the `dnnl::matmul` path of oneDNN v3.14: it
 * exports the C entry points of oneDNN's own headers (include/oneapi/dnnl/
 * dnnl.h, dnnl_common.h) that this path uses, with identical names, argument
 * lists, enum values and status codes, so a program written against
 * dnnl.h / dnnl.hpp links against it unchanged.  `dnnl_gpu` selects the CUDA
 * engine (engine index = CUDA device ordinal); there is no CPU engine.
 *
 * This header restates those declarations for users that do not have the
 * oneDNN headers at hand (ctypes, cgo, JNI stubs ...).  When oneDNN's own
 * dnnl.h has been included first, only the additive CUDA interop section at
 * the end is declared.  Each block cites the oneDNN declaration it mirrors.
 */
#ifndef DNNL_B200_H
#define DNNL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef ONEAPI_DNNL_DNNL_H /* oneDNN's dnnl.h not included: declare the ABI */

/* ---- status / enums (dnnl_common_types.h:45-220, dnnl_types.h) ---------- */
typedef enum {
    dnnl_success = 0,
    dnnl_out_of_memory = 1,
    dnnl_invalid_arguments = 2,
    dnnl_unimplemented = 3,
    dnnl_last_impl_reached = 4,
    dnnl_runtime_error = 5,
    dnnl_not_required = 6,
} dnnl_status_t;

typedef enum {
    dnnl_data_type_undef = 0,
    dnnl_f16 = 1,
    dnnl_bf16 = 2,
    dnnl_f32 = 3,
    dnnl_s32 = 4,
    dnnl_s8 = 5,
    dnnl_u8 = 6,
    dnnl_f64 = 7,
    dnnl_boolean = 8,
    dnnl_f8_e5m2 = 9,
    dnnl_f8_e4m3 = 10,
    dnnl_s4 = 11,
    dnnl_u4 = 12,
    dnnl_e8m0 = 13,
    dnnl_f4_e2m1 = 14,
    dnnl_f4_e3m0 = 15,
    dnnl_s64 = 16,
    dnnl_data_type_max = 0x7fff,
} dnnl_data_type_t;

#define DNNL_MAX_NDIMS 12
typedef int64_t dnnl_dim_t;
typedef dnnl_dim_t dnnl_dims_t[DNNL_MAX_NDIMS];

typedef enum {
    dnnl_fpmath_mode_strict,
    dnnl_fpmath_mode_bf16,
    dnnl_fpmath_mode_f16,
    dnnl_fpmath_mode_any,
    dnnl_fpmath_mode_tf32,
} dnnl_fpmath_mode_t;

typedef enum {
    dnnl_accumulation_mode_strict,
    dnnl_accumulation_mode_relaxed,
    dnnl_accumulation_mode_any,
    dnnl_accumulation_mode_s32,
    dnnl_accumulation_mode_f32,
    dnnl_accumulation_mode_f16
} dnnl_accumulation_mode_t;

typedef enum { dnnl_any_engine, dnnl_cpu, dnnl_gpu } dnnl_engine_kind_t;

typedef enum {
    dnnl_stream_in_order = 0x1U,
    dnnl_stream_out_of_order = 0x2U,
    dnnl_stream_profiling = 0x4U, /* events around every primitive, read by dnnl_query_profiling_data */
    dnnl_stream_default_flags = dnnl_stream_in_order,
    dnnl_stream_flags_max = 0x7fff,
} dnnl_stream_flags_t;

/* dnnl_types.h:45-62 */
typedef enum {
    dnnl_format_kind_undef = 0,
    dnnl_format_kind_any,
    dnnl_blocked,
    dnnl_format_kind_opaque,
    dnnl_format_kind_sparse,
    dnnl_format_kind_host_scalar,
    dnnl_format_kind_max = 0x7fff,
} dnnl_format_kind_t;

/* dnnl_types.h:64-90; only the grouped encoding is implemented */
typedef enum {
    dnnl_sparse_encoding_undef = 0,
    dnnl_csr,
    dnnl_packed,
    dnnl_coo,
    dnnl_grouped,
} dnnl_sparse_encoding_t;

/* dnnl_types.h:177-208: the plain tags this path accepts */
typedef enum {
    dnnl_format_tag_undef = 0,
    dnnl_format_tag_any = 1,
    dnnl_a = 2,
    dnnl_ab = 3,
    dnnl_abc = 4,
    dnnl_abcd = 5,
    dnnl_ba = 14,
    dnnl_acb = 15,
    dnnl_bac = 16,
    dnnl_bca = 17,
    dnnl_cab = 18,
    dnnl_cba = 19,
} dnnl_format_tag_t;

/* dnnl_types.h:2055-2101 (values used by post-ops and queries) */
typedef enum {
    dnnl_undefined_primitive = 0,
    dnnl_reorder = 1,
    dnnl_sum = 4,
    dnnl_eltwise = 7,
    dnnl_binary = 13,
    dnnl_matmul = 14,
    dnnl_prelu = 18,
    dnnl_primitive_kind_max = 0x7fff,
} dnnl_primitive_kind_t;

/* dnnl_types.h:2105-2228 */
typedef enum {
    dnnl_alg_kind_undef = 0,
    dnnl_eltwise_relu = 0x20,
    dnnl_eltwise_tanh,
    dnnl_eltwise_elu,
    dnnl_eltwise_square,
    dnnl_eltwise_abs,
    dnnl_eltwise_sqrt,
    dnnl_eltwise_linear,
    dnnl_eltwise_soft_relu,
    dnnl_eltwise_hardsigmoid,
    dnnl_eltwise_logistic,
    dnnl_eltwise_exp,
    dnnl_eltwise_gelu_tanh,
    dnnl_eltwise_swish,
    dnnl_eltwise_log,
    dnnl_eltwise_clip,
    dnnl_eltwise_clip_v2,
    dnnl_eltwise_pow,
    dnnl_eltwise_gelu_erf,
    dnnl_eltwise_round,
    dnnl_eltwise_mish,
    dnnl_eltwise_hardswish,
    dnnl_binary_add = 0x1fff0,
    dnnl_binary_mul = 0x1fff1,
    dnnl_binary_max = 0x1fff2,
    dnnl_binary_min = 0x1fff3,
    dnnl_binary_div = 0x1fff4,
    dnnl_binary_sub = 0x1fff5,
    dnnl_binary_ge = 0x1fff6,
    dnnl_binary_gt = 0x1fff7,
    dnnl_binary_le = 0x1fff8,
    dnnl_binary_lt = 0x1fff9,
    dnnl_binary_eq = 0x1fffa,
    dnnl_binary_ne = 0x1fffb,
    dnnl_binary_select = 0x1fffc,
} dnnl_alg_kind_t;

/* dnnl_types.h:2452-2486 */
typedef enum { dnnl_scratchpad_mode_library, dnnl_scratchpad_mode_user } dnnl_scratchpad_mode_t;
typedef enum { dnnl_rounding_mode_environment, dnnl_rounding_mode_stochastic } dnnl_rounding_mode_t;
typedef enum {
    dnnl_quantization_mode_undef,
    dnnl_quantization_mode_static_sazp,
    dnnl_quantization_mode_dynamic_mx,
    dnnl_quantization_mode_dynamic_fp,
} dnnl_quantization_mode_t;

/* dnnl_types.h:2849-2922 (the queries this library answers) */
typedef enum {
    dnnl_query_undef = 0,
    dnnl_query_engine = 1,
    dnnl_query_primitive_kind = 2,
    dnnl_query_num_of_inputs_s32 = 3,
    dnnl_query_num_of_outputs_s32 = 4,
    dnnl_query_time_estimate_f64 = 5,
    dnnl_query_memory_consumption_s64 = 6,
    dnnl_query_scratchpad_engine = 7,
    dnnl_query_impl_info_str = 8,
    dnnl_query_prop_kind = 11,
    dnnl_query_strides = 14,
    dnnl_query_src_md = 129,
    dnnl_query_weights_md = 131,
    dnnl_query_dst_md = 133,
    dnnl_query_workspace_md = 135,
    dnnl_query_scratchpad_md = 136,
    dnnl_query_exec_arg_md = 255,
    dnnl_query_ndims_s32 = 256,
    dnnl_query_dims = 257,
    dnnl_query_data_type = 258,
    dnnl_query_submemory_offset_s64 = 259,
    dnnl_query_padded_dims = 260,
    dnnl_query_padded_offsets = 261,
    dnnl_query_format_kind = 262,
    dnnl_query_inner_nblks_s32 = 263,
    dnnl_query_inner_blks = 264,
    dnnl_query_inner_idxs = 265,
    dnnl_query_sparse_encoding = 266,
    dnnl_query_nnz_s64 = 267,
    dnnl_query_num_handles_s32 = 268,
    dnnl_query_max = 0x7fff,
} dnnl_query_t;

/* execution argument keys, dnnl_types.h:2542-2786 */
#define DNNL_ARG_SRC 1
#define DNNL_ARG_SRC_0 1
#define DNNL_ARG_SRC_1 2
#define DNNL_ARG_SRC_2 3
#define DNNL_ARG_DST 17
#define DNNL_ARG_FROM DNNL_ARG_SRC_0
#define DNNL_ARG_TO DNNL_ARG_DST
#define DNNL_ARG_WEIGHTS 33
#define DNNL_ARG_WEIGHTS_1 34
#define DNNL_ARG_WEIGHTS_2 35
#define DNNL_ARG_BIAS 41
#define DNNL_ARG_SCRATCHPAD 80
#define DNNL_ARG_HINT_MAX_GROUP_SIZE 384
#define DNNL_ARG_ATTR_PRECOMPUTED_REDUCTIONS 512
#define DNNL_ARG_MULTIPLE_SRC 1024
#define DNNL_ARG_ATTR_SCALES 4096
#define DNNL_ARG_ATTR_ZERO_POINTS 8192
#define DNNL_ARG_ATTR_POST_OP_DW 16384
#define DNNL_ARG_ATTR_MULTIPLE_POST_OP_BASE 32768
#define DNNL_ARG_ATTR_MULTIPLE_POST_OP(idx) (DNNL_ARG_ATTR_MULTIPLE_POST_OP_BASE * ((idx) + 1))

#define DNNL_MEMORY_NONE (NULL)
#define DNNL_MEMORY_ALLOCATE ((void *)(size_t)-1)
#define DNNL_RUNTIME_DIM_VAL INT64_MIN

/* ---- opaque handles (dnnl_common_types.h:189-229, dnnl_types.h) --------- */
struct dnnl_engine;
typedef struct dnnl_engine *dnnl_engine_t;
struct dnnl_stream;
typedef struct dnnl_stream *dnnl_stream_t;
typedef const struct dnnl_stream *const_dnnl_stream_t;
struct dnnl_memory_desc;
typedef struct dnnl_memory_desc *dnnl_memory_desc_t;
typedef const struct dnnl_memory_desc *const_dnnl_memory_desc_t;
struct dnnl_memory;
typedef struct dnnl_memory *dnnl_memory_t;
typedef const struct dnnl_memory *const_dnnl_memory_t;
struct dnnl_primitive_attr;
typedef struct dnnl_primitive_attr *dnnl_primitive_attr_t;
typedef const struct dnnl_primitive_attr *const_dnnl_primitive_attr_t;
struct dnnl_post_ops;
typedef struct dnnl_post_ops *dnnl_post_ops_t;
typedef const struct dnnl_post_ops *const_dnnl_post_ops_t;
struct dnnl_primitive_desc;
typedef struct dnnl_primitive_desc *dnnl_primitive_desc_t;
typedef const struct dnnl_primitive_desc *const_dnnl_primitive_desc_t;
struct dnnl_primitive;
typedef struct dnnl_primitive *dnnl_primitive_t;
typedef const struct dnnl_primitive *const_dnnl_primitive_t;

/* dnnl_types.h:2791-2794 */
typedef struct {
    int arg;
    dnnl_memory_t memory;
} dnnl_exec_arg_t;

/* dnnl_common_types.h:237-244 */
typedef struct {
    int major, minor, patch;
    const char *hash;
    unsigned cpu_runtime;
    unsigned gpu_runtime;
} dnnl_version_t;

#define DNNL_API

/* ---- engine / stream (dnnl_common.h:44-109) ----------------------------- */
size_t DNNL_API dnnl_engine_get_count(dnnl_engine_kind_t kind);
dnnl_status_t DNNL_API dnnl_engine_create(dnnl_engine_t *engine, dnnl_engine_kind_t kind, size_t index);
dnnl_status_t DNNL_API dnnl_engine_get_kind(dnnl_engine_t engine, dnnl_engine_kind_t *kind);
dnnl_status_t DNNL_API dnnl_engine_destroy(dnnl_engine_t engine);
dnnl_status_t DNNL_API dnnl_stream_create(dnnl_stream_t *stream, dnnl_engine_t engine, unsigned flags);
dnnl_status_t DNNL_API dnnl_stream_get_engine(const_dnnl_stream_t stream, dnnl_engine_t *engine);
dnnl_status_t DNNL_API dnnl_stream_wait(dnnl_stream_t stream);
dnnl_status_t DNNL_API dnnl_stream_destroy(dnnl_stream_t stream);

/* ---- service (dnnl_common.h:122-163, dnnl.h:3882-4048) ------------------ */
const dnnl_version_t DNNL_API *dnnl_version(void);
dnnl_status_t DNNL_API dnnl_set_verbose(int level);
dnnl_status_t DNNL_API dnnl_get_default_fpmath_mode(dnnl_fpmath_mode_t *mode);
dnnl_status_t DNNL_API dnnl_set_default_fpmath_mode(dnnl_fpmath_mode_t mode);
dnnl_status_t DNNL_API dnnl_get_primitive_cache_capacity(int *capacity);
dnnl_status_t DNNL_API dnnl_set_primitive_cache_capacity(int capacity);

/* ---- memory descriptors (dnnl.h:1018-1460) ------------------------------ */
dnnl_status_t DNNL_API dnnl_memory_desc_create_with_strides(dnnl_memory_desc_t *memory_desc, int ndims,
        const dnnl_dims_t dims, dnnl_data_type_t data_type, const dnnl_dims_t strides);
dnnl_status_t DNNL_API dnnl_memory_desc_create_with_tag(dnnl_memory_desc_t *memory_desc, int ndims,
        const dnnl_dims_t dims, dnnl_data_type_t data_type, dnnl_format_tag_t tag);
/* exported by the reference library for its own test driver, which declares them itself
 * (src/common/memory_desc.cpp:1140-1158, tests/benchdnn/dnnl_memory.cpp:49-54): a tag written as
 * letters, outermost dim first; the data type of an existing descriptor changed in place */
dnnl_status_t DNNL_API dnnl_memory_desc_create_with_string_tag(dnnl_memory_desc_t *memory_desc, int ndims,
        const dnnl_dims_t dims, dnnl_data_type_t data_type, const char *tag);
dnnl_status_t DNNL_API dnnl_memory_desc_set_data_type(dnnl_memory_desc_t memory_desc, dnnl_data_type_t data_type);
dnnl_status_t DNNL_API dnnl_memory_desc_create_with_grouped_encoding(dnnl_memory_desc_t *memory_desc,
        int ndims, const dnnl_dims_t dims, dnnl_data_type_t data_type, int variable_dim_idx,
        dnnl_dim_t group_count, dnnl_data_type_t offsets_dt);
dnnl_status_t DNNL_API dnnl_memory_desc_create_host_scalar(dnnl_memory_desc_t *memory_desc,
        dnnl_data_type_t data_type);
dnnl_status_t DNNL_API dnnl_memory_desc_clone(dnnl_memory_desc_t *memory_desc,
        const_dnnl_memory_desc_t existing_memory_desc);
dnnl_status_t DNNL_API dnnl_memory_desc_destroy(dnnl_memory_desc_t memory_desc);
/* dnnl.h:1219: a window of a plain strided tensor (same strides, offset0 moved) */
dnnl_status_t DNNL_API dnnl_memory_desc_create_submemory(dnnl_memory_desc_t *memory_desc,
        const_dnnl_memory_desc_t parent_memory_desc, const dnnl_dims_t dims, const dnnl_dims_t offsets);
dnnl_status_t DNNL_API dnnl_memory_desc_reshape(dnnl_memory_desc_t *out_memory_desc,
        const_dnnl_memory_desc_t in_memory_desc, int ndims, const dnnl_dims_t dims);
dnnl_status_t DNNL_API dnnl_memory_desc_permute_axes(dnnl_memory_desc_t *out_memory_desc,
        const_dnnl_memory_desc_t in_memory_desc, const int *permutation);
dnnl_status_t DNNL_API dnnl_memory_desc_query(const_dnnl_memory_desc_t memory_desc, dnnl_query_t what,
        void *result);
dnnl_status_t DNNL_API dnnl_memory_desc_query_v2(const_dnnl_memory_desc_t memory_desc, dnnl_query_t what,
        int index, void *result);
int DNNL_API dnnl_memory_desc_equal(const_dnnl_memory_desc_t lhs, const_dnnl_memory_desc_t rhs);
size_t DNNL_API dnnl_memory_desc_get_size(const_dnnl_memory_desc_t memory_desc);
size_t DNNL_API dnnl_memory_desc_get_size_v2(const_dnnl_memory_desc_t memory_desc, int index);
size_t DNNL_API dnnl_data_type_size(dnnl_data_type_t data_type);

/* ---- memory objects (dnnl.h:1482-1705) ----------------------------------
 * A handle is a CUDA device pointer on the engine's device, DNNL_MEMORY_NONE,
 * or DNNL_MEMORY_ALLOCATE (the library allocates and owns the buffer).
 * map/unmap stage the buffer through host memory. */
dnnl_status_t DNNL_API dnnl_memory_create(dnnl_memory_t *memory, const_dnnl_memory_desc_t memory_desc,
        dnnl_engine_t engine, void *handle);
dnnl_status_t DNNL_API dnnl_memory_create_v2(dnnl_memory_t *memory, const_dnnl_memory_desc_t memory_desc,
        dnnl_engine_t engine, int nhandles, void **handles);
dnnl_status_t DNNL_API dnnl_memory_create_host_scalar(dnnl_memory_t *memory,
        const_dnnl_memory_desc_t memory_desc, void *scalar_ptr);
dnnl_status_t DNNL_API dnnl_memory_get_host_scalar_value(const_dnnl_memory_t memory, void *value);
dnnl_status_t DNNL_API dnnl_memory_set_host_scalar_value(dnnl_memory_t memory, const void *value);
dnnl_status_t DNNL_API dnnl_memory_get_memory_desc(const_dnnl_memory_t memory,
        const_dnnl_memory_desc_t *memory_desc);
dnnl_status_t DNNL_API dnnl_memory_get_engine(const_dnnl_memory_t memory, dnnl_engine_t *engine);
dnnl_status_t DNNL_API dnnl_memory_map_data(const_dnnl_memory_t memory, void **mapped_ptr);
dnnl_status_t DNNL_API dnnl_memory_map_data_v2(const_dnnl_memory_t memory, void **mapped_ptr, int index);
dnnl_status_t DNNL_API dnnl_memory_unmap_data(const_dnnl_memory_t memory, void *mapped_ptr);
dnnl_status_t DNNL_API dnnl_memory_unmap_data_v2(const_dnnl_memory_t memory, void *mapped_ptr, int index);
dnnl_status_t DNNL_API dnnl_memory_get_data_handle(const_dnnl_memory_t memory, void **handle);
dnnl_status_t DNNL_API dnnl_memory_set_data_handle(dnnl_memory_t memory, void *handle);
dnnl_status_t DNNL_API dnnl_memory_get_data_handle_v2(const_dnnl_memory_t memory, void **handle, int index);
dnnl_status_t DNNL_API dnnl_memory_set_data_handle_v2(dnnl_memory_t memory, void *handle, int index);
dnnl_status_t DNNL_API dnnl_memory_destroy(dnnl_memory_t memory);

/* ---- attributes and post-ops (dnnl.h:258-1003) -------------------------- */
dnnl_status_t DNNL_API dnnl_primitive_attr_create(dnnl_primitive_attr_t *attr);
dnnl_status_t DNNL_API dnnl_primitive_attr_clone(dnnl_primitive_attr_t *attr,
        const_dnnl_primitive_attr_t existing_attr);
dnnl_status_t DNNL_API dnnl_primitive_attr_destroy(dnnl_primitive_attr_t attr);
dnnl_status_t DNNL_API dnnl_primitive_attr_get_fpmath_mode(const_dnnl_primitive_attr_t attr,
        dnnl_fpmath_mode_t *mode);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_fpmath_mode(dnnl_primitive_attr_t attr, dnnl_fpmath_mode_t mode);
dnnl_status_t DNNL_API dnnl_primitive_attr_get_fpmath_mode_v2(const_dnnl_primitive_attr_t attr,
        dnnl_fpmath_mode_t *mode, int *apply_to_int);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_fpmath_mode_v2(dnnl_primitive_attr_t attr,
        dnnl_fpmath_mode_t mode, int apply_to_int);
dnnl_status_t DNNL_API dnnl_primitive_attr_get_deterministic(const_dnnl_primitive_attr_t attr, int *value);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_deterministic(dnnl_primitive_attr_t attr, int value);
dnnl_status_t DNNL_API dnnl_primitive_attr_get_accumulation_mode(const_dnnl_primitive_attr_t attr,
        dnnl_accumulation_mode_t *mode);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_accumulation_mode(dnnl_primitive_attr_t attr,
        dnnl_accumulation_mode_t mode);
dnnl_status_t DNNL_API dnnl_primitive_attr_get_scratchpad_mode(const_dnnl_primitive_attr_t attr,
        dnnl_scratchpad_mode_t *mode);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_scratchpad_mode(dnnl_primitive_attr_t attr,
        dnnl_scratchpad_mode_t mode);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_scales_mask(dnnl_primitive_attr_t attr, int arg, int mask);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_scales(dnnl_primitive_attr_t attr, int arg, int mask,
        int group_ndims, const dnnl_dims_t group_dims, dnnl_data_type_t data_type);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_scales_v2(dnnl_primitive_attr_t attr, int arg, int mask,
        int ndims, const dnnl_dims_t group_dims, dnnl_data_type_t data_type, int is_on_host);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_scales_v3(dnnl_primitive_attr_t attr, int arg, int mask,
        int ndims, const dnnl_dims_t group_dims, dnnl_data_type_t data_type, int is_on_host,
        dnnl_quantization_mode_t qmode);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_zero_points_mask(dnnl_primitive_attr_t attr, int arg, int mask);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_zero_points(dnnl_primitive_attr_t attr, int arg, int mask,
        int group_ndims, const dnnl_dims_t group_dims, dnnl_data_type_t data_type);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_zero_points_v2(dnnl_primitive_attr_t attr, int arg, int mask,
        int ndims, const dnnl_dims_t group_dims, dnnl_data_type_t data_type, int is_on_host);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_precomputed_reductions(dnnl_primitive_attr_t attr, int arg,
        int mask, int group_ndims, const dnnl_dims_t group_dims, dnnl_data_type_t data_type);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_rounding(dnnl_primitive_attr_t attr, int arg,
        dnnl_rounding_mode_t mode);
dnnl_status_t DNNL_API dnnl_primitive_attr_get_rounding(dnnl_primitive_attr_t attr, int arg,
        dnnl_rounding_mode_t *mode);
dnnl_status_t DNNL_API dnnl_primitive_attr_get_post_ops(const_dnnl_primitive_attr_t attr,
        const_dnnl_post_ops_t *post_ops);
dnnl_status_t DNNL_API dnnl_primitive_attr_set_post_ops(dnnl_primitive_attr_t attr,
        const_dnnl_post_ops_t post_ops);
dnnl_status_t DNNL_API dnnl_post_ops_create(dnnl_post_ops_t *post_ops);
dnnl_status_t DNNL_API dnnl_post_ops_clone(dnnl_post_ops_t *post_ops, const_dnnl_post_ops_t existing_post_ops);
dnnl_status_t DNNL_API dnnl_post_ops_destroy(dnnl_post_ops_t post_ops);
int DNNL_API dnnl_post_ops_len(const_dnnl_post_ops_t post_ops);
dnnl_primitive_kind_t DNNL_API dnnl_post_ops_get_kind(const_dnnl_post_ops_t post_ops, int index);
dnnl_status_t DNNL_API dnnl_post_ops_append_sum(dnnl_post_ops_t post_ops, float scale, int32_t zero_point,
        dnnl_data_type_t data_type);
dnnl_status_t DNNL_API dnnl_post_ops_get_params_sum(const_dnnl_post_ops_t post_ops, int index, float *scale,
        int32_t *zero_point, dnnl_data_type_t *data_type);
dnnl_status_t DNNL_API dnnl_post_ops_append_eltwise(dnnl_post_ops_t post_ops, dnnl_alg_kind_t alg_kind,
        float alpha, float beta);
dnnl_status_t DNNL_API dnnl_post_ops_get_params_eltwise(const_dnnl_post_ops_t post_ops, int index,
        dnnl_alg_kind_t *alg_kind, float *alpha, float *beta);
dnnl_status_t DNNL_API dnnl_post_ops_append_binary(dnnl_post_ops_t post_ops, dnnl_alg_kind_t alg_kind,
        const_dnnl_memory_desc_t src1_desc);
dnnl_status_t DNNL_API dnnl_post_ops_get_params_binary(const_dnnl_post_ops_t post_ops, int index,
        dnnl_alg_kind_t *alg_kind, const_dnnl_memory_desc_t *src1_desc);
dnnl_status_t DNNL_API dnnl_post_ops_append_prelu(dnnl_post_ops_t post_ops, int mask);
/* dnnl.h:924-959: the third operand belongs to binary_select, which matmul does not apply
 * (unimplemented); for every other algorithm src2_desc must be NULL or empty */
dnnl_status_t DNNL_API dnnl_post_ops_append_binary_v2(dnnl_post_ops_t post_ops, dnnl_alg_kind_t alg_kind,
        const_dnnl_memory_desc_t src1_desc, const_dnnl_memory_desc_t src2_desc);
dnnl_status_t DNNL_API dnnl_post_ops_get_params_binary_v2(const_dnnl_post_ops_t post_ops, int index,
        dnnl_alg_kind_t *alg_kind, const_dnnl_memory_desc_t *src1_desc, const_dnnl_memory_desc_t *src2_desc);
/* dnnl.h:1003 */
dnnl_status_t DNNL_API dnnl_post_ops_get_params_prelu(const_dnnl_post_ops_t post_ops, int index, int *mask);

/* ---- primitive descriptor / primitive (dnnl.h:51-243, 3774) ------------- */
dnnl_status_t DNNL_API dnnl_matmul_primitive_desc_create(dnnl_primitive_desc_t *primitive_desc,
        dnnl_engine_t engine, const_dnnl_memory_desc_t src_desc, const_dnnl_memory_desc_t weights_desc,
        const_dnnl_memory_desc_t bias_desc, const_dnnl_memory_desc_t dst_desc,
        const_dnnl_primitive_attr_t attr);
/* dnnl.h:1727 (src/common/reorder.cpp:153-237): both engines must be the same
 * CUDA engine; plain strided layouts; src / dst scales, src zero-points, a
 * common dst zero-point and one sum post-op, as the reference's
 * simple_reorder reference implementations take them
 * (src/cpu/reorder/simple_reorder.hpp:2168-2679) */
dnnl_status_t DNNL_API dnnl_reorder_primitive_desc_create(dnnl_primitive_desc_t *reorder_primitive_desc,
        const_dnnl_memory_desc_t src_desc, dnnl_engine_t src_engine, const_dnnl_memory_desc_t dst_desc,
        dnnl_engine_t dst_engine, const_dnnl_primitive_attr_t attr);
dnnl_status_t DNNL_API dnnl_primitive_desc_next_impl(dnnl_primitive_desc_t primitive_desc);
dnnl_status_t DNNL_API dnnl_primitive_desc_clone(dnnl_primitive_desc_t *primitive_desc,
        const_dnnl_primitive_desc_t existing_primitive_desc);
dnnl_status_t DNNL_API dnnl_primitive_desc_get_attr(const_dnnl_primitive_desc_t primitive_desc,
        const_dnnl_primitive_attr_t *attr);
dnnl_status_t DNNL_API dnnl_primitive_desc_destroy(dnnl_primitive_desc_t primitive_desc);
dnnl_status_t DNNL_API dnnl_primitive_desc_query(const_dnnl_primitive_desc_t primitive_desc,
        dnnl_query_t what, int index, void *result);
const_dnnl_memory_desc_t DNNL_API dnnl_primitive_desc_query_md(const_dnnl_primitive_desc_t primitive_desc,
        dnnl_query_t what, int index);
int DNNL_API dnnl_primitive_desc_query_s32(const_dnnl_primitive_desc_t primitive_desc, dnnl_query_t what,
        int index);
dnnl_status_t DNNL_API dnnl_primitive_create(dnnl_primitive_t *primitive,
        const_dnnl_primitive_desc_t primitive_desc);
dnnl_status_t DNNL_API dnnl_primitive_create_from_cache_blob(dnnl_primitive_t *primitive,
        const_dnnl_primitive_desc_t primitive_desc, size_t size, const uint8_t *cache_blob);
dnnl_status_t DNNL_API dnnl_primitive_execute(const_dnnl_primitive_t primitive, dnnl_stream_t stream,
        int nargs, const dnnl_exec_arg_t *args);
dnnl_status_t DNNL_API dnnl_primitive_get_primitive_desc(const_dnnl_primitive_t primitive,
        const_dnnl_primitive_desc_t *primitive_desc);
dnnl_status_t DNNL_API dnnl_primitive_get_cache_blob(const_dnnl_primitive_t primitive, size_t *size,
        uint8_t *cache_blob);
dnnl_status_t DNNL_API dnnl_primitive_destroy(dnnl_primitive_t primitive);

/* ---- stream profiling (dnnl.h:4063-4085; streams created with
 * dnnl_stream_profiling).  One entry per primitive executed since the last
 * reset; data_kind 1 (dnnl_profiling_data_kind_time) gives nanoseconds of
 * device time between CUDA events recorded around the primitive's kernels.
 * Wait on the stream before querying. */
dnnl_status_t DNNL_API dnnl_reset_profiling(dnnl_stream_t stream);
dnnl_status_t DNNL_API dnnl_query_profiling_data(dnnl_stream_t stream, int data_kind, int *num_entries,
        uint64_t *data);

/* ---- value names (dnnl_debug.h:35-54).  The enumerations this header does
 * not declare are taken as int. */
#ifndef ONEAPI_DNNL_DNNL_DEBUG_H
const char DNNL_API *dnnl_status2str(dnnl_status_t v);
const char DNNL_API *dnnl_dt2str(dnnl_data_type_t v);
const char DNNL_API *dnnl_fpmath_mode2str(dnnl_fpmath_mode_t v);
const char DNNL_API *dnnl_accumulation_mode2str(dnnl_accumulation_mode_t v);
const char DNNL_API *dnnl_engine_kind2str(dnnl_engine_kind_t v);
const char DNNL_API *dnnl_sparse_encoding2str(dnnl_sparse_encoding_t v);
const char DNNL_API *dnnl_fmt_tag2str(dnnl_format_tag_t v);
const char DNNL_API *dnnl_fmt_kind2str(dnnl_format_kind_t v);
const char DNNL_API *dnnl_prop_kind2str(int v);
const char DNNL_API *dnnl_prim_kind2str(dnnl_primitive_kind_t v);
const char DNNL_API *dnnl_alg_kind2str(dnnl_alg_kind_t v);
const char DNNL_API *dnnl_rnn_flags2str(int v);
const char DNNL_API *dnnl_rnn_direction2str(int v);
const char DNNL_API *dnnl_scratchpad_mode2str(dnnl_scratchpad_mode_t v);
const char DNNL_API *dnnl_rounding_mode2str(dnnl_rounding_mode_t v);
const char DNNL_API *dnnl_quantization_mode2str(dnnl_quantization_mode_t v);
const char DNNL_API *dnnl_cpu_isa2str(int v);
const char DNNL_API *dnnl_cpu_isa_hints2str(int v);
const char DNNL_API *dnnl_runtime2str(unsigned v);
#endif

/* Every other function dnnl.h declares (the other primitives' descriptor
 * constructors, RNN / dropout attributes, sparse encodings other than
 * grouped, the BLAS-like gemm calls) is exported as a stub that returns
 * dnnl_unimplemented, so that unchanged programs link. */

#endif /* ONEAPI_DNNL_DNNL_H */

/* ---- CUDA interop: additive, modelled on oneDNN's OpenCL interop header
 * (include/oneapi/dnnl/dnnl_ocl.h:67-255) ---------------------------------- */

/* value reported in dnnl_version()->gpu_runtime by this library */
#define DNNL_RUNTIME_CUDA 2048u

/* Creates an engine for the CUDA device with the given ordinal; same as
 * dnnl_engine_create(&e, dnnl_gpu, device). */
dnnl_status_t dnnl_cuda_interop_engine_create(dnnl_engine_t *engine, int device);
dnnl_status_t dnnl_cuda_interop_engine_get_device(dnnl_engine_t engine, int *device);
/* Wraps an existing cudaStream_t (passed as void*); the library neither
 * synchronizes nor destroys it on dnnl_stream_destroy. */
dnnl_status_t dnnl_cuda_interop_stream_create(dnnl_stream_t *stream, dnnl_engine_t engine, void *cuda_stream);
dnnl_status_t dnnl_cuda_interop_stream_get_cuda_stream(dnnl_stream_t stream, void **cuda_stream);
/* Wraps a device pointer the caller owns. */
dnnl_status_t dnnl_cuda_interop_memory_create(dnnl_memory_t *memory, const_dnnl_memory_desc_t memory_desc,
        dnnl_engine_t engine, void *device_ptr);
/* Number of kernels this library has launched in the calling process; the
 * benchmark reports the difference over its timed region. */
uint64_t dnnl_cuda_interop_launch_count(void);
/* Human-readable text of the last CUDA error seen by the calling thread. */
const char *dnnl_cuda_interop_last_error(void);

/* dst[M,N] (s32) = (src[M,K] (u8) - src_zero_point) x weights[K,N] (s8), all
 * row-major device buffers, enqueued on `cuda_stream` (a cudaStream_t).
 *
 * This entry point has no counterpart in the reference.  It exists for
 * callers that must not trigger a device allocation: code running while a
 * CUDA graph is being assembled by someone else, real-time or embedded hosts
 * with a fixed memory plan, plugins whose host forbids cudaMalloc after
 * start-up.  The regular path (dnnl_primitive_create) allocates a scratch
 * buffer for the zero-point compensation sums; this one keeps that scratch in
 * a fixed array inside the library image instead, so it never calls
 * cudaMalloc / cudaFree or any allocating routine.
 *
 * Limits and rules:
 *  - N <= 131072 (the array holds one s32 per weight column, 512 KB per GPU,
 *    resident on every GPU that loads the library); larger N is rejected with
 *    dnnl_invalid_arguments.  K and N multiples of 16, src and weights
 *    16-byte aligned, else dnnl_unimplemented.
 *  - The first call on each device (with that device current) looks up the
 *    array's device address and opts the kernel in to its shared memory; make
 *    that first call outside any stream capture.
 *  - All calls share the one array: two calls that overlap on the GPU (other
 *    streams, other threads) race.  Serialize them on one stream.
 * The results equal those of the dnnl_matmul primitive with a per-tensor s32
 * src zero-point, bit for bit. */
dnnl_status_t dnnl_cuda_interop_matmul_u8s8s32_zp_static(void *cuda_stream, int64_t M, int64_t N, int64_t K,
        const uint8_t *src, const int8_t *weights, int32_t src_zero_point, int32_t *dst);

/* Companion of the call above (no counterpart in the reference either): the
 * kernels never trap; a wait inside them that runs out of time records
 * status 5 (runtime_error) in a word of the same static array and leaves dst
 * incomplete.  The word is sticky across calls.  This function waits for the
 * work already enqueued on `cuda_stream`, copies the word of the current
 * device to *status (0 = every call since the last query ran to completion)
 * and clears it.  It allocates nothing; it synchronises the stream, so do not
 * call it while the stream is being captured. */
dnnl_status_t dnnl_cuda_interop_matmul_u8s8s32_zp_static_status(void *cuda_stream, int *status);

/* ---- assembling a sharded result over NVLink (no counterpart in the reference, which is a
 * single-device library).  One process per GPU computes an N-slice (or the rows of its experts) of
 * dst; instead of a collective library, each rank stores its block into EVERY rank's full dst buffer
 * with plain peer stores and raises a flag there; the wait call blocks the stream (bounded) until
 * the blocks of all ranks have landed.
 *   peer_dst[p], peer_flags[p]: device addresses, valid on the calling GPU, of rank p's dst buffer
 *   and of its flag array (`world` 32-bit words, zero at start); peer-mapped memory such as CUDA IPC
 *   or symmetric-memory allocations, exchanged once at set-up.
 *   seg: nseg (<= 64) triples (first src row, first dst row, rows) of the local block.
 *   epoch: a number that grows with every exchange on these flags.  done: a zeroed 32-bit word of
 *   local device memory.  Byte sizes, pitches and offsets are multiples of 16.
 * A consumer must not overwrite a dst buffer that peers may still be filling for a later epoch:
 * alternate two buffers, or exchange an acknowledgement. */
dnnl_status_t dnnl_cuda_interop_peer_scatter(dnnl_stream_t stream, int world, int rank, const void *local,
        int64_t row_bytes, int64_t src_pitch, void *const *peer_dst, int64_t dst_pitch, int64_t dst_col_bytes,
        int nseg, const int64_t *seg, unsigned *const *peer_flags, unsigned epoch, unsigned *done);
/* Waits on the stream until flags[0..world) have all reached `epoch`; a wait that runs out (2 s)
 * records runtime_error for the next dnnl_stream_wait. */
dnnl_status_t dnnl_cuda_interop_peer_wait(dnnl_stream_t stream, int world, const unsigned *flags, unsigned epoch);
/* The fused form for the tcgen05 GEMM (`cuda:tcgen05:int8` / `fp8`): the next executions of the
 * primitive store every dst element into all `world` buffers at the offset the primitive's dst
 * memory has inside dst_bases[rank], and the kernel's last CTA publishes `epoch` in
 * peer_flags[r][rank] of every rank r: dnnl_cuda_interop_peer_wait is then the whole exchange.
 * Call again with the next epoch before each execution; world <= 1 or dst_bases == NULL switches it
 * off.  dnnl_unimplemented for other implementations (use dnnl_cuda_interop_peer_scatter). */
dnnl_status_t dnnl_cuda_interop_primitive_replicate_dst(dnnl_primitive_t primitive, int world, int rank,
        void *const *dst_bases, size_t buffer_bytes, unsigned *const *peer_flags, unsigned *done, unsigned epoch);

#ifdef __cplusplus
}
#endif
#endif
