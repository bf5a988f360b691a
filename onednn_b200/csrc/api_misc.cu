// C API, remaining surface: the value-to-name functions of dnnl_debug.h, the
// verbose info string of a primitive (format of oneDNN's
// src/common/verbose.cpp:527-575, 697-860, 1060-1090), stream profiling
// (dnnl.h:4063-4085, backed by CUDA events), sub-memory descriptors, the
// later post-op entry points, and every other dnnl_* name of dnnl.h as a stub
// that returns dnnl_unimplemented, so that programs written against the
// unchanged headers link against this library.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <sstream>

#include "launch.h"
#include "objects.hpp"

using namespace qmm;

namespace qmm {

const char *dt_name(int dt) {
    switch (dt) {
        case dnnl_data_type_undef: return "undef";
        case dnnl_f16: return "f16";
        case dnnl_bf16: return "bf16";
        case dnnl_f32: return "f32";
        case dnnl_s32: return "s32";
        case dnnl_s8: return "s8";
        case dnnl_u8: return "u8";
        case dnnl_f64: return "f64";
        case dnnl_boolean: return "boolean";
        case dnnl_f8_e5m2: return "f8_e5m2";
        case dnnl_f8_e4m3: return "f8_e4m3";
        case dnnl_s4: return "s4";
        case dnnl_u4: return "u4";
        case dnnl_e8m0: return "e8m0";
        case dnnl_f4_e2m1: return "f4_e2m1";
        case dnnl_f4_e3m0: return "f4_e3m0";
        case dnnl_s64: return "s64";
        default: return "unknown dt";
    }
}

namespace {

const char *alg_name(int a) {
    static const char *const eltwise[] = {"eltwise_relu", "eltwise_tanh", "eltwise_elu", "eltwise_square", "eltwise_abs",
            "eltwise_sqrt", "eltwise_linear", "eltwise_soft_relu", "eltwise_hardsigmoid", "eltwise_logistic",
            "eltwise_exp", "eltwise_gelu_tanh", "eltwise_swish", "eltwise_log", "eltwise_clip", "eltwise_clip_v2",
            "eltwise_pow", "eltwise_gelu_erf", "eltwise_round", "eltwise_mish", "eltwise_hardswish"};
    static const char *const binary[] = {"binary_add", "binary_mul", "binary_max", "binary_min", "binary_div",
            "binary_sub", "binary_ge", "binary_gt", "binary_le", "binary_lt", "binary_eq", "binary_ne", "binary_select"};
    if (a == 0) return "undef";
    if (a >= 0x20 && a < 0x20 + (int)(sizeof(eltwise) / sizeof(*eltwise))) return eltwise[a - 0x20];
    if (a >= 0x1fff0 && a < 0x1fff0 + (int)(sizeof(binary) / sizeof(*binary))) return binary[a - 0x1fff0];
    return "unknown alg_kind";
}

// "ab", "ba", "acb" ... for a plain strided layout: dims sorted by decreasing stride; empty when the
// strides are not a permutation of a dense layout's (the strides are printed instead)
std::string plain_tag(const dnnl_memory_desc &md, bool *dense) {
    int order[DNNL_MAX_NDIMS];
    for (int i = 0; i < md.ndims; ++i) order[i] = i;
    for (int i = 1; i < md.ndims; ++i) // insertion sort, stable: larger stride first
        for (int j = i; j > 0 && md.strides[order[j]] > md.strides[order[j - 1]]; --j) std::swap(order[j], order[j - 1]);
    std::string tag;
    dnnl_dim_t expect = 1;
    *dense = true;
    for (int i = md.ndims - 1; i >= 0; --i) {
        if (md.dims[order[i]] != 1 && md.strides[order[i]] != expect) *dense = false;
        expect *= md.dims[order[i]];
    }
    for (int i = 0; i < md.ndims; ++i) tag += (char)('a' + order[i]);
    return tag;
}

std::string dims_str(const dnnl_dim_t *d, int n) {
    std::string s;
    for (int i = 0; i < n; ++i) s += (i ? "x" : "") + std::to_string((long long)d[i]);
    return s;
}

std::string md_str(const char *name, const dnnl_memory_desc &md) {
    std::string s = std::string(name) + ":";
    if (md.ndims == 0) return s + "undef::undef:::";
    s += std::string(dt_name(md.data_type)) + ":" + (md.offset0 ? "0" : "") + ":";
    if (md.is_grouped())
        return s + "sparse:grouped:" + std::to_string(md.variable_dim_idx) + ":" + std::to_string((long long)md.group_count)
                + ":";
    if (md.format_kind == dnnl_format_kind_any) return s + "any:any:";
    if (md.format_kind != dnnl_blocked) return s + "undef:::";
    bool dense = true;
    const std::string tag = plain_tag(md, &dense);
    return s + "blocked:" + tag + ":" + (dense ? "" : dims_str(md.strides, md.ndims)) + ":f0";
}

const char *arg_name(int arg) {
    switch (arg) {
        case DNNL_ARG_SRC: return "src0";
        case DNNL_ARG_SRC_1: return "src1";
        case DNNL_ARG_WEIGHTS: return "wei";
        case DNNL_ARG_DST: return "dst";
        case DNNL_ARG_BIAS: return "bia";
        default: return "arg";
    }
}

std::string quant_str(const std::map<int, quant_entry_t> &m) {
    std::string s;
    for (const auto &kv : m) {
        const quant_entry_t &q = kv.second;
        if (!q.set) continue;
        if (!s.empty()) s += "+";
        s += std::string(arg_name(kv.first)) + ":" + std::to_string(q.mask) + ":" + dt_name(q.dt);
        if (q.group_ndims > 0) s += ":" + std::to_string((long long)q.groups[0]) + "x" + std::to_string((long long)q.groups[1]);
        if (q.on_host) s += ":host_scalar";
        if (q.qmode == dnnl_quantization_mode_dynamic_mx) s += ":dynamic_mx";
        if (q.qmode == dnnl_quantization_mode_dynamic_fp) s += ":dynamic_fp";
    }
    return s;
}

std::string attr_str(const dnnl_primitive_attr &attr) {
    std::string s;
    auto field = [&](const std::string &f) { s += (s.empty() ? "" : " ") + f; };
    if (attr.scratchpad_mode != dnnl_scratchpad_mode_library) field("attr-scratchpad:user");
    if (attr.fpmath != dnnl_fpmath_mode_strict || attr.apply_to_int)
        field(std::string("attr-fpmath:") + dnnl_fpmath_mode2str(attr.fpmath) + (attr.apply_to_int ? ":true" : ""));
    if (attr.acc_mode != dnnl_accumulation_mode_strict)
        field(std::string("attr-acc-mode:") + dnnl_accumulation_mode2str(attr.acc_mode));
    if (attr.deterministic) field("attr-deterministic:1");
    if (!attr.scales.empty()) field("attr-scales:" + quant_str(attr.scales));
    if (!attr.zero_points.empty()) field("attr-zero-points:" + quant_str(attr.zero_points));
    if (!attr.reductions.empty()) field("attr-precomputed-reductions:" + quant_str(attr.reductions));
    if (!attr.post_ops.entries.empty()) {
        std::string p;
        for (const auto &e : attr.post_ops.entries) {
            if (!p.empty()) p += "+";
            if (e.kind == dnnl_sum) {
                p += "sum";
                std::ostringstream o;
                if (e.scale != 1.f || e.zero_point != 0 || e.sum_dt != dnnl_data_type_undef) o << ":" << e.scale;
                if (e.zero_point != 0 || e.sum_dt != dnnl_data_type_undef) o << ":" << e.zero_point;
                if (e.sum_dt != dnnl_data_type_undef) o << ":" << dt_name(e.sum_dt);
                p += o.str();
            } else if (e.kind == dnnl_eltwise) {
                std::ostringstream o;
                o << alg_name(e.alg);
                if (e.alpha != 0.f || e.beta != 0.f || e.scale != 1.f) o << ":" << e.alpha;
                if (e.beta != 0.f || e.scale != 1.f) o << ":" << e.beta;
                if (e.scale != 1.f) o << ":" << e.scale;
                p += o.str();
            } else if (e.kind == dnnl_binary) {
                int mask = 0;
                for (int d = 0; d < e.src1.ndims; ++d) mask |= e.src1.dims[d] != 1 ? 1 << d : 0;
                bool dense = true;
                p += std::string(alg_name(e.alg)) + ":" + dt_name(e.src1.data_type) + ":" + std::to_string(mask) + ":"
                        + plain_tag(e.src1, &dense);
            } else if (e.kind == dnnl_prelu) {
                p += "prelu:" + std::to_string(e.prelu_mask);
            }
        }
        field("attr-post-ops:" + p);
    }
    return s;
}

} // namespace

// operation-independent part of a verbose line: engine, primitive, implementation, prop_kind,
// memory descriptors, attributes, auxiliary, problem description
std::string pd_info_string(const dnnl_primitive_desc &pd) {
    std::string s = "gpu,";
    if (pd.kind == dnnl_reorder) {
        s += "reorder," + pd.impl_name + ",undef," + md_str("src", pd.src) + " " + md_str("dst", pd.dst) + ","
                + attr_str(pd.attr) + ",," + dims_str(pd.src.dims, pd.src.ndims);
        return s;
    }
    s += "matmul," + pd.impl_name + ",undef," + md_str("src", pd.src) + " " + md_str("wei", pd.wei) + " ";
    if (pd.bias.ndims) {
        int mask = 0;
        for (int d = 0; d < pd.bias.ndims; ++d) mask |= pd.bias.dims[d] != 1 ? 1 << d : 0;
        s += md_str("bia", pd.bias) + "_mask" + std::to_string(mask) + " ";
    }
    s += md_str("dst", pd.dst) + "," + attr_str(pd.attr) + ",," + dims_str(pd.src.dims, pd.src.ndims) + ":"
            + dims_str(pd.wei.dims, pd.wei.ndims);
    return s;
}

void verbose_line(const char *operation, const dnnl_primitive_desc &pd, double ms) {
    printf("onednn_verbose,v1,primitive,%s,%s,%g\n", operation, pd_info_string(pd).c_str(), ms);
    fflush(stdout);
}

// ---- stream profiling -------------------------------------------------------
void profiling_begin(dnnl_stream_t s) {
    if (!(s->flags & dnnl_stream_profiling) || s->engine->device < 0) return;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return;
    cudaEventRecord(e0, s->stream);
    std::lock_guard<std::mutex> lock(s->prof_mu);
    s->prof.push_back({e0, e1});
    s->prof_open = true;
}
void profiling_end(dnnl_stream_t s) {
    std::lock_guard<std::mutex> lock(s->prof_mu);
    if (!s->prof_open || s->prof.empty()) return;
    cudaEventRecord(s->prof.back().second, s->stream);
    s->prof_open = false;
}
void profiling_clear(dnnl_stream_t s) {
    std::lock_guard<std::mutex> lock(s->prof_mu);
    for (auto &p : s->prof) {
        cudaEventDestroy(p.first);
        cudaEventDestroy(p.second);
    }
    s->prof.clear();
    s->prof_open = false;
}

} // namespace qmm

extern "C" {

/* ---- dnnl_debug.h:35-54 ---------------------------------------------------- */
const char *dnnl_status2str(dnnl_status_t v) {
    switch ((int)v) {
        case dnnl_success: return "success";
        case dnnl_out_of_memory: return "out_of_memory";
        case dnnl_invalid_arguments: return "invalid_arguments";
        case dnnl_unimplemented: return "unimplemented";
        case dnnl_last_impl_reached: return "last_impl_reached";
        case dnnl_runtime_error: return "runtime_error";
        case dnnl_not_required: return "not_required";
        default: return "unknown status";
    }
}
const char *dnnl_dt2str(dnnl_data_type_t v) { return dt_name((int)v); }
const char *dnnl_fpmath_mode2str(dnnl_fpmath_mode_t v) {
    switch ((int)v) {
        case dnnl_fpmath_mode_strict: return "strict";
        case dnnl_fpmath_mode_bf16: return "bf16";
        case dnnl_fpmath_mode_f16: return "f16";
        case dnnl_fpmath_mode_any: return "any";
        case dnnl_fpmath_mode_tf32: return "tf32";
        default: return "unknown fpmath_mode";
    }
}
const char *dnnl_accumulation_mode2str(dnnl_accumulation_mode_t v) {
    switch ((int)v) {
        case dnnl_accumulation_mode_strict: return "strict";
        case dnnl_accumulation_mode_relaxed: return "relaxed";
        case dnnl_accumulation_mode_any: return "any";
        case dnnl_accumulation_mode_s32: return "s32";
        case dnnl_accumulation_mode_f32: return "f32";
        case dnnl_accumulation_mode_f16: return "f16";
        default: return "unknown accumulation_mode";
    }
}
const char *dnnl_engine_kind2str(dnnl_engine_kind_t v) {
    switch ((int)v) {
        case dnnl_any_engine: return "any";
        case dnnl_cpu: return "cpu";
        case dnnl_gpu: return "gpu";
        default: return "unknown engine_kind";
    }
}
const char *dnnl_sparse_encoding2str(dnnl_sparse_encoding_t v) {
    switch ((int)v) {
        case dnnl_sparse_encoding_undef: return "undef";
        case dnnl_csr: return "csr";
        case dnnl_packed: return "packed";
        case dnnl_coo: return "coo";
        case dnnl_grouped: return "grouped";
        default: return "unknown sparse_encoding";
    }
}
// the plain tags this engine creates descriptors from; blocked tags do not exist here
const char *dnnl_fmt_tag2str(dnnl_format_tag_t v) {
    switch ((int)v) {
        case dnnl_format_tag_undef: return "undef";
        case dnnl_format_tag_any: return "any";
        case dnnl_a: return "a";
        case dnnl_ab: return "ab";
        case dnnl_abc: return "abc";
        case dnnl_abcd: return "abcd";
        case dnnl_ba: return "ba";
        case dnnl_acb: return "acb";
        case dnnl_bac: return "bac";
        case dnnl_bca: return "bca";
        case dnnl_cab: return "cab";
        case dnnl_cba: return "cba";
        default: return "unknown fmt_tag";
    }
}
const char *dnnl_fmt_kind2str(dnnl_format_kind_t v) {
    switch ((int)v) {
        case dnnl_format_kind_undef: return "undef";
        case dnnl_format_kind_any: return "any";
        case dnnl_blocked: return "blocked";
        case dnnl_format_kind_opaque: return "opaque";
        case dnnl_format_kind_sparse: return "sparse";
        case dnnl_format_kind_host_scalar: return "host_scalar";
        default: return "unknown fmt_kind";
    }
}
const char *dnnl_prop_kind2str(int v) {
    switch (v) {
        case 0: return "undef";
        case 64: return "forward_training";
        case 96: return "forward_inference";
        case 128: return "backward";
        case 160: return "backward_data";
        case 192: return "backward_weights";
        case 193: return "backward_bias";
        default: return "unknown prop_kind";
    }
}
const char *dnnl_prim_kind2str(dnnl_primitive_kind_t v) {
    static const char *const names[] = {"undef", "reorder", "shuffle", "concat", "sum", "convolution", "deconvolution",
            "eltwise", "lrn", "batch_normalization", "inner_product", "rnn", "gemm", "binary", "matmul", "resampling",
            "pooling", "reduction", "prelu", "softmax", "layer_normalization", "group_normalization"};
    const int i = (int)v;
    return i >= 0 && i < (int)(sizeof(names) / sizeof(*names)) ? names[i] : "unknown prim_kind";
}
const char *dnnl_alg_kind2str(dnnl_alg_kind_t v) { return alg_name((int)v); }
const char *dnnl_rnn_flags2str(int v) { return v == 0 ? "undef" : "unknown rnn_flags"; }
const char *dnnl_rnn_direction2str(int v) { return v == 0 ? "unidirectional_left2right" : "unknown rnn_direction"; }
const char *dnnl_scratchpad_mode2str(dnnl_scratchpad_mode_t v) {
    return v == dnnl_scratchpad_mode_library ? "library" : v == dnnl_scratchpad_mode_user ? "user" : "unknown scratchpad_mode";
}
const char *dnnl_rounding_mode2str(dnnl_rounding_mode_t v) {
    return v == dnnl_rounding_mode_environment ? "environment"
            : v == dnnl_rounding_mode_stochastic ? "stochastic" : "unknown rounding_mode";
}
const char *dnnl_quantization_mode2str(dnnl_quantization_mode_t v) {
    switch ((int)v) {
        case dnnl_quantization_mode_undef: return "undef";
        case dnnl_quantization_mode_static_sazp: return "static_sazp";
        case dnnl_quantization_mode_dynamic_mx: return "dynamic_mx";
        case dnnl_quantization_mode_dynamic_fp: return "dynamic_fp";
        default: return "unknown quantization_mode";
    }
}
const char *dnnl_cpu_isa2str(int v) { return v == 0 ? "isa_default" : "unknown cpu_isa"; }
const char *dnnl_cpu_isa_hints2str(int v) { return v == 0 ? "no_hints" : "unknown cpu_isa_hints"; }
const char *dnnl_runtime2str(unsigned v) {
    switch (v) {
        case 0u: return "none";
        case 1u: return "sequential";
        case 2u: return "OpenMP";
        case 4u: return "TBB";
        case 8u: return "threadpool";
        case 256u: return "OpenCL";
        case 512u: return "SYCL";
        case DNNL_RUNTIME_CUDA: return "CUDA";
        default: return "unknown";
    }
}

/* ---- profiling (dnnl.h:4063-4085) ------------------------------------------ */
// What the reference's test driver calls after reading the profiling data of a GPU stream
// (src/common/stream_profiler.cpp:55-63): the events recorded here need no such notice.
dnnl_status_t dnnl_impl_notify_profiling_complete(dnnl_stream_t stream) {
    if (!stream) return dnnl_invalid_arguments;
    return (stream->flags & dnnl_stream_profiling) ? dnnl_success : dnnl_invalid_arguments;
}
dnnl_status_t dnnl_reset_profiling(dnnl_stream_t stream) {
    if (!stream) return dnnl_invalid_arguments;
    if (!(stream->flags & dnnl_stream_profiling)) return dnnl_invalid_arguments;
    profiling_clear(stream);
    return dnnl_success;
}
// One entry per primitive executed on the stream since the last reset, in
// nanoseconds of device time (CUDA events around the primitive's kernels).
// The caller waits on the stream first, as the reference requires.
dnnl_status_t dnnl_query_profiling_data(dnnl_stream_t stream, int data_kind, int *num_entries, uint64_t *data) {
    if (!stream || !num_entries) return dnnl_invalid_arguments;
    if (!(stream->flags & dnnl_stream_profiling)) return dnnl_invalid_arguments;
    std::lock_guard<std::mutex> lock(stream->prof_mu);
    if (!data) {
        *num_entries = (int)stream->prof.size();
        return dnnl_success;
    }
    if (data_kind != 1 /* dnnl_profiling_data_kind_time */) return dnnl_invalid_arguments;
    if (*num_entries < (int)stream->prof.size()) return dnnl_invalid_arguments;
    for (size_t i = 0; i < stream->prof.size(); ++i) {
        float ms = 0.f;
        if (!cuda_ok(cudaEventElapsedTime(&ms, stream->prof[i].first, stream->prof[i].second), "cudaEventElapsedTime"))
            return dnnl_runtime_error; // not waited for
        data[i] = (uint64_t)((double)ms * 1e6 + 0.5);
    }
    *num_entries = (int)stream->prof.size();
    return dnnl_success;
}

/* ---- dnnl.h:924-959, 1003: later post-op entry points ---------------------- */
dnnl_status_t dnnl_post_ops_append_binary_v2(dnnl_post_ops_t post_ops, dnnl_alg_kind_t alg,
        const_dnnl_memory_desc_t src1, const_dnnl_memory_desc_t src2) {
    // the third operand exists for binary_select only, which the matmul path does not apply
    if ((int)alg == 0x1fffc) return src1 && src2 ? dnnl_unimplemented : dnnl_invalid_arguments;
    if (src2 && src2->ndims != 0) return dnnl_invalid_arguments;
    return dnnl_post_ops_append_binary(post_ops, alg, src1);
}
dnnl_status_t dnnl_post_ops_get_params_binary_v2(const_dnnl_post_ops_t post_ops, int index, dnnl_alg_kind_t *alg,
        const_dnnl_memory_desc_t *src1, const_dnnl_memory_desc_t *src2) {
    static const dnnl_memory_desc zero_md;
    const dnnl_status_t st = dnnl_post_ops_get_params_binary(post_ops, index, alg, src1);
    if (st == dnnl_success && src2) *src2 = &zero_md;
    return st;
}
dnnl_status_t dnnl_post_ops_get_params_prelu(const_dnnl_post_ops_t post_ops, int index, int *mask) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_invalid_arguments;
    const auto &e = post_ops->entries[index];
    if (e.kind != dnnl_prelu) return dnnl_invalid_arguments;
    if (mask) *mask = e.prelu_mask;
    return dnnl_success;
}

/* ---- dnnl.h:1219: a window into a plain strided tensor --------------------- */
dnnl_status_t dnnl_memory_desc_create_submemory(dnnl_memory_desc_t *memory_desc, const_dnnl_memory_desc_t parent,
        const dnnl_dims_t dims, const dnnl_dims_t offsets) {
    if (!memory_desc || !parent || !dims || !offsets) return dnnl_invalid_arguments;
    if (parent->format_kind != dnnl_blocked) return dnnl_unimplemented; // `any`, grouped, host scalar
    dnnl_dim_t off = parent->offset0;
    for (int d = 0; d < parent->ndims; ++d) {
        if (dims[d] < 0 || offsets[d] < 0 || offsets[d] + dims[d] > parent->dims[d]) return dnnl_invalid_arguments;
        off += offsets[d] * parent->strides[d];
    }
    // two 4-bit elements share a byte: the window has to start on a byte
    if (dt_bits(parent->data_type) == 4 && off % 2 != 0) return dnnl_invalid_arguments;
    auto *md = new dnnl_memory_desc(*parent);
    for (int d = 0; d < parent->ndims; ++d) md->dims[d] = dims[d];
    md->offset0 = off;
    *memory_desc = md;
    return dnnl_success;
}

/* ---- everything else dnnl.h declares: not part of this library ------------- */
#define QMM_STUB(name) \
    dnnl_status_t name(void) { return dnnl_unimplemented; }
QMM_STUB(dnnl_augru_backward_primitive_desc_create)
QMM_STUB(dnnl_augru_forward_primitive_desc_create)
QMM_STUB(dnnl_batch_normalization_backward_primitive_desc_create)
QMM_STUB(dnnl_batch_normalization_forward_primitive_desc_create)
QMM_STUB(dnnl_binary_primitive_desc_create)
QMM_STUB(dnnl_binary_primitive_desc_create_v2)
QMM_STUB(dnnl_concat_primitive_desc_create)
QMM_STUB(dnnl_convolution_backward_data_primitive_desc_create)
QMM_STUB(dnnl_convolution_backward_weights_primitive_desc_create)
QMM_STUB(dnnl_convolution_forward_primitive_desc_create)
QMM_STUB(dnnl_deconvolution_backward_data_primitive_desc_create)
QMM_STUB(dnnl_deconvolution_backward_weights_primitive_desc_create)
QMM_STUB(dnnl_deconvolution_forward_primitive_desc_create)
QMM_STUB(dnnl_eltwise_backward_primitive_desc_create)
QMM_STUB(dnnl_eltwise_forward_primitive_desc_create)
QMM_STUB(dnnl_gemm_s8s8s32)
QMM_STUB(dnnl_gemm_u8s8s32)
QMM_STUB(dnnl_group_normalization_backward_primitive_desc_create)
QMM_STUB(dnnl_group_normalization_forward_primitive_desc_create)
QMM_STUB(dnnl_gru_backward_primitive_desc_create)
QMM_STUB(dnnl_gru_forward_primitive_desc_create)
QMM_STUB(dnnl_inner_product_backward_data_primitive_desc_create)
QMM_STUB(dnnl_inner_product_backward_weights_primitive_desc_create)
QMM_STUB(dnnl_inner_product_forward_primitive_desc_create)
QMM_STUB(dnnl_layer_normalization_backward_primitive_desc_create)
QMM_STUB(dnnl_layer_normalization_backward_primitive_desc_create_v2)
QMM_STUB(dnnl_layer_normalization_forward_primitive_desc_create)
QMM_STUB(dnnl_layer_normalization_forward_primitive_desc_create_v2)
QMM_STUB(dnnl_lbr_augru_backward_primitive_desc_create)
QMM_STUB(dnnl_lbr_augru_forward_primitive_desc_create)
QMM_STUB(dnnl_lbr_gru_backward_primitive_desc_create)
QMM_STUB(dnnl_lbr_gru_forward_primitive_desc_create)
QMM_STUB(dnnl_lrn_backward_primitive_desc_create)
QMM_STUB(dnnl_lrn_forward_primitive_desc_create)
QMM_STUB(dnnl_lstm_backward_primitive_desc_create)
QMM_STUB(dnnl_lstm_forward_primitive_desc_create)
QMM_STUB(dnnl_memory_desc_create_with_blob)
QMM_STUB(dnnl_memory_desc_create_with_coo_encoding)
QMM_STUB(dnnl_memory_desc_create_with_csr_encoding)
QMM_STUB(dnnl_memory_desc_create_with_packed_encoding)
QMM_STUB(dnnl_memory_desc_get_blob)
QMM_STUB(dnnl_pooling_backward_primitive_desc_create)
QMM_STUB(dnnl_pooling_forward_primitive_desc_create)
QMM_STUB(dnnl_post_ops_append_dw)
QMM_STUB(dnnl_post_ops_get_params_dw)
QMM_STUB(dnnl_prelu_backward_primitive_desc_create)
QMM_STUB(dnnl_prelu_forward_primitive_desc_create)
QMM_STUB(dnnl_primitive_attr_get_dropout)
QMM_STUB(dnnl_primitive_attr_get_dropout_v2)
QMM_STUB(dnnl_primitive_attr_get_rnn_data_qparams)
QMM_STUB(dnnl_primitive_attr_get_rnn_weights_projection_qparams)
QMM_STUB(dnnl_primitive_attr_get_rnn_weights_qparams)
QMM_STUB(dnnl_primitive_attr_set_dropout)
QMM_STUB(dnnl_primitive_attr_set_dropout_v2)
QMM_STUB(dnnl_primitive_attr_set_rnn_data_qparams)
QMM_STUB(dnnl_primitive_attr_set_rnn_weights_projection_qparams)
QMM_STUB(dnnl_primitive_attr_set_rnn_weights_qparams)
QMM_STUB(dnnl_reduction_primitive_desc_create)
QMM_STUB(dnnl_resampling_backward_primitive_desc_create)
QMM_STUB(dnnl_resampling_forward_primitive_desc_create)
QMM_STUB(dnnl_sgemm)
QMM_STUB(dnnl_gemm_bf16bf16f32)
QMM_STUB(dnnl_impl_zero_pad) // plain layouts have no padding to clear
QMM_STUB(dnnl_shuffle_backward_primitive_desc_create)
QMM_STUB(dnnl_shuffle_forward_primitive_desc_create)
QMM_STUB(dnnl_softmax_backward_primitive_desc_create)
QMM_STUB(dnnl_softmax_forward_primitive_desc_create)
QMM_STUB(dnnl_sum_primitive_desc_create)
QMM_STUB(dnnl_vanilla_rnn_backward_primitive_desc_create)
QMM_STUB(dnnl_vanilla_rnn_forward_primitive_desc_create)
/* dnnl_ocl.h: the generated dnnl_config.h names the OpenCL runtime class so that programs fill GPU
   memory through map / unmap; there is no OpenCL behind it */
QMM_STUB(dnnl_ocl_interop_engine_create)
QMM_STUB(dnnl_ocl_interop_engine_create_from_cache_blob)
QMM_STUB(dnnl_ocl_interop_engine_get_cache_blob)
QMM_STUB(dnnl_ocl_interop_engine_get_cache_blob_id)
QMM_STUB(dnnl_ocl_interop_engine_get_context)
QMM_STUB(dnnl_ocl_interop_get_device)
QMM_STUB(dnnl_ocl_interop_memory_create)
QMM_STUB(dnnl_ocl_interop_memory_create_v2)
QMM_STUB(dnnl_ocl_interop_memory_get_mem_object)
QMM_STUB(dnnl_ocl_interop_memory_get_memory_kind)
QMM_STUB(dnnl_ocl_interop_memory_set_mem_object)
QMM_STUB(dnnl_ocl_interop_primitive_execute)
QMM_STUB(dnnl_ocl_interop_stream_create)
QMM_STUB(dnnl_ocl_interop_stream_get_command_queue)
#undef QMM_STUB

/* CPU-only service calls (dnnl.h:3960-4048): there is no CPU engine; they succeed and change nothing,
   except the ISA controls, which have nothing to act on */
dnnl_status_t dnnl_set_jit_dump(int) { return dnnl_success; }
dnnl_status_t dnnl_set_jit_profiling_flags(unsigned) { return dnnl_success; }
dnnl_status_t dnnl_set_jit_profiling_jitdumpdir(const char *) { return dnnl_success; }
dnnl_status_t dnnl_set_max_cpu_isa(int) { return dnnl_unimplemented; }
int dnnl_get_effective_cpu_isa(void) { return 0; /* dnnl_cpu_isa_default */ }
dnnl_status_t dnnl_set_cpu_isa_hints(int) { return dnnl_unimplemented; }
int dnnl_get_cpu_isa_hints(void) { return 0; /* dnnl_cpu_isa_no_hints */ }

} // extern "C"
