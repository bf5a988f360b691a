// Definitions of the opaque handle types of the C API (engine, stream,
// memory descriptor, memory, attributes, post-ops, primitive descriptor,
// primitive).  The counterparts in oneDNN are src/common/engine.hpp,
// stream.hpp, memory_desc.hpp, memory.hpp, primitive_attr.hpp,
// primitive_desc_iface.hpp and primitive_iface.hpp.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "dnnl_b200.h"
#include "kernel_args.h"

struct dnnl_engine {
    int device = 0;
    int sm_count = 0;
    std::atomic<int> refs {1};
    int *status_word = nullptr; // device word written by kernels on errors
};

struct dnnl_stream {
    dnnl_engine_t engine = nullptr;
    cudaStream_t stream = nullptr;
    bool owned = true;
    unsigned flags = 0;
    // dnnl_stream_profiling: one (start, stop) event pair per executed primitive
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof;
    std::mutex prof_mu;
    bool prof_open = false;
};

struct dnnl_memory_desc {
    int ndims = 0;
    dnnl_dims_t dims = {};
    dnnl_data_type_t data_type = dnnl_data_type_undef;
    dnnl_format_kind_t format_kind = dnnl_format_kind_undef;
    dnnl_dims_t strides = {}; // elements; valid when format_kind == blocked
    dnnl_dim_t offset0 = 0;
    // grouped encoding (format_kind == sparse)
    dnnl_sparse_encoding_t encoding = dnnl_sparse_encoding_undef;
    int variable_dim_idx = 0;
    dnnl_dim_t group_count = 0;
    dnnl_data_type_t offsets_dt = dnnl_data_type_undef;

    bool is_grouped() const { return format_kind == dnnl_format_kind_sparse && encoding == dnnl_grouped; }
    // a dim (or a stride that depends on one) left open until execution: DNNL_RUNTIME_DIM_VAL
    bool has_runtime_dims() const {
        for (int i = 0; i < ndims; ++i)
            if (dims[i] == DNNL_RUNTIME_DIM_VAL || (format_kind == dnnl_blocked && strides[i] == DNNL_RUNTIME_DIM_VAL))
                return true;
        return false;
    }
    bool is_zero() const { return ndims == 0; }
    dnnl_dim_t nelems() const {
        if (ndims == 0) return 0;
        dnnl_dim_t n = 1;
        for (int i = 0; i < ndims; ++i) n *= dims[i];
        return n;
    }
    bool has_zero_dim() const { return nelems() == 0; }
};

struct dnnl_memory {
    dnnl_memory_desc md;
    dnnl_engine_t engine = nullptr;
    void *handles[2] = {nullptr, nullptr};
    bool owned[2] = {false, false};
    void *mapped[2] = {nullptr, nullptr}; // host staging while mapped
    double host_scalar = 0; // storage of a host-scalar memory (<= 8 bytes)
    bool is_host_scalar = false;
};

struct quant_entry_t {
    bool set = false;
    int mask = 0;
    dnnl_data_type_t dt = dnnl_data_type_undef;
    int group_ndims = 0;
    dnnl_dim_t groups[2] = {1, 1};
    bool on_host = false;
    dnnl_quantization_mode_t qmode = dnnl_quantization_mode_static_sazp;
    dnnl_dim_t group(int d) const { // negative d counts from the end
        if (group_ndims == 0) return 1;
        if (d < 0) d += group_ndims;
        return (d < 0 || d >= group_ndims) ? 0 : groups[d];
    }
    bool operator==(const quant_entry_t &o) const {
        return set == o.set && mask == o.mask && dt == o.dt && group_ndims == o.group_ndims
                && groups[0] == o.groups[0] && groups[1] == o.groups[1] && on_host == o.on_host
                && qmode == o.qmode;
    }
};

struct post_op_entry_t {
    dnnl_primitive_kind_t kind = dnnl_undefined_primitive;
    dnnl_alg_kind_t alg = dnnl_alg_kind_undef;
    float alpha = 0, beta = 0, scale = 1.f;
    int32_t zero_point = 0; // sum
    dnnl_data_type_t sum_dt = dnnl_data_type_undef;
    dnnl_memory_desc src1; // binary
    int prelu_mask = 0;
};

struct dnnl_post_ops {
    std::vector<post_op_entry_t> entries;
};

struct dnnl_primitive_attr {
    dnnl_fpmath_mode_t fpmath = dnnl_fpmath_mode_strict;
    bool apply_to_int = false;
    dnnl_accumulation_mode_t acc_mode = dnnl_accumulation_mode_strict;
    bool deterministic = false;
    dnnl_scratchpad_mode_t scratchpad_mode = dnnl_scratchpad_mode_library;
    std::map<int, quant_entry_t> scales, zero_points, reductions;
    std::map<int, dnnl_rounding_mode_t> rounding;
    dnnl_post_ops post_ops;

    const quant_entry_t &get(const std::map<int, quant_entry_t> &m, int arg) const {
        static const quant_entry_t dflt;
        auto it = m.find(arg);
        return it == m.end() ? dflt : it->second;
    }
    const quant_entry_t &scale(int arg) const { return get(scales, arg); }
    const quant_entry_t &zp(int arg) const { return get(zero_points, arg); }
    const quant_entry_t &pr(int arg) const { return get(reductions, arg); }
    bool has_default_values() const {
        return fpmath == dnnl_fpmath_mode_strict && !apply_to_int && acc_mode == dnnl_accumulation_mode_strict
                && !deterministic && scratchpad_mode == dnnl_scratchpad_mode_library && scales.empty()
                && zero_points.empty() && reductions.empty() && rounding.empty() && post_ops.entries.empty();
    }
};

// One entry of the implementation list walked by primitive_desc_next_impl.
enum impl_id_t : int {
    IMPL_TCGEN05_GEMM = 0, // tensor-core int8 / fp8 GEMM
    IMPL_WOQ_TC, // int4 weight decompression through tensor memory (M <= 32)
    IMPL_WOQ_GEMV, // weight-decompression skinny GEMM (M <= 32), mma.sync
    IMPL_GROUPED_TC, // grouped (MoE) tensor-core GEMM
    IMPL_REF, // generic kernels, every attribute
    IMPL_COUNT
};

struct dnnl_primitive_desc {
    dnnl_primitive_kind_t kind = dnnl_matmul; // dnnl_reorder: only src, dst and attr are used
    dnnl_engine_t engine = nullptr;
    dnnl_memory_desc src, wei, bias, dst, scratchpad;
    dnnl_primitive_attr attr;
    bool grouped = false;
    // some of M, K, N (or strides) are DNNL_RUNTIME_DIM_VAL: shapes, implementation and scratch are
    // settled per execution from the memory objects' descriptors (impl / impl_name describe the
    // stand-in shape the descriptor was checked with at creation)
    bool runtime_m = false;
    bool batched = false; // ndims > 2: the implementation runs once per matrix of the batch
    int impl = IMPL_REF;
    std::string impl_name;
    std::map<int, dnnl_memory_desc> quant_mds; // exec-arg id -> parameter md
    size_t scratch_bytes = 0; // device scratch the chosen implementation needs
    dnnl_dim_t M() const { return dst.dims[dst.ndims - 2]; }
    dnnl_dim_t N() const { return dst.dims[dst.ndims - 1]; }
    dnnl_dim_t K() const { return src.dims[src.ndims - 1]; }
};

struct dnnl_primitive {
    dnnl_primitive_desc pd;
    // scratch owned by the primitive (scratchpad_mode_library); like oneDNN's
    // library scratchpad it makes concurrent execute calls of ONE primitive
    // object unsafe
    mutable void *scratch = nullptr;
    mutable size_t scratch_cap = 0; // bytes behind `scratch` (grows for runtime-M primitives)
    // dnnl_cuda_interop_primitive_replicate_dst: where the next executions repeat their dst stores
    mutable qmm::PeerReplication peers {};
    mutable const char *peers_own_base = nullptr;
    mutable size_t peers_bytes = 0;
};

namespace qmm {
void set_last_error(const std::string &s);
bool cuda_ok(cudaError_t e, const char *what);
int verbose_level();
size_t dt_bits(dnnl_data_type_t dt);
size_t md_bytes(const dnnl_memory_desc &md, int index);
const char *dt_name(int dt);
// api_misc.cu: the fields of a verbose line that describe the primitive, and the line itself
std::string pd_info_string(const dnnl_primitive_desc &pd);
void verbose_line(const char *operation, const dnnl_primitive_desc &pd, double ms);
// api_misc.cu: event pair around one primitive on a profiling stream
void profiling_begin(dnnl_stream_t s);
void profiling_end(dnnl_stream_t s);
void profiling_clear(dnnl_stream_t s);
// reorder.cu: enqueues the reorder described by pd on the stream
dnnl_status_t execute_reorder(const dnnl_primitive_desc &pd, dnnl_stream_t stream, int nargs,
        const dnnl_exec_arg_t *args);
} // namespace qmm
