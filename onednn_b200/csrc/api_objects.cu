// C API: engine, stream, memory descriptors, memory objects, attributes and
// post-ops.  Mirrors the behaviour (argument checks, status codes, ownership)
// of oneDNN's src/common/{engine,stream,memory_desc,memory,primitive_attr}.cpp
// for the subset the quantized matmul path uses.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "objects.hpp"
#include "launch.h"

using namespace qmm;

namespace {
thread_local std::string g_last_error;
std::atomic<uint64_t> g_launches {0};
int g_verbose = -1;
dnnl_fpmath_mode_t g_default_fpmath = dnnl_fpmath_mode_strict;
int g_cache_capacity = 0;
} // namespace

namespace qmm {
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
void set_last_error(const std::string &s) { g_last_error = s; }
bool cuda_ok(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return true;
    g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return false;
}
int verbose_level() {
    if (g_verbose < 0) {
        const char *v = getenv("ONEDNN_VERBOSE");
        if (!v) v = getenv("DNNL_VERBOSE");
        g_verbose = v ? atoi(v) : 0;
    }
    return g_verbose;
}
size_t dt_bits(dnnl_data_type_t dt) {
    switch (dt) {
        case dnnl_f32: case dnnl_s32: return 32;
        case dnnl_f16: case dnnl_bf16: return 16;
        case dnnl_s8: case dnnl_u8: case dnnl_f8_e5m2: case dnnl_f8_e4m3: case dnnl_e8m0: case dnnl_boolean: return 8;
        case dnnl_s4: case dnnl_u4: case dnnl_f4_e2m1: case dnnl_f4_e3m0: return 4;
        case dnnl_f64: case dnnl_s64: return 64;
        default: return 0;
    }
}
// bytes of a dense-or-strided blocked descriptor (sub-byte types round up)
size_t md_bytes(const dnnl_memory_desc &md, int index) {
    if (md.format_kind == dnnl_format_kind_host_scalar) return index == 0 ? dt_bits(md.data_type) / 8 : 0;
    if (md.ndims == 0) return 0;
    if (md.has_runtime_dims()) return (size_t)DNNL_RUNTIME_DIM_VAL; // DNNL_RUNTIME_SIZE_VAL
    if (md.has_zero_dim()) return 0;
    if (md.is_grouped()) {
        if (index == 0) return ((size_t)md.nelems() * dt_bits(md.data_type) + 7) / 8;
        if (index == 1) return (size_t)md.group_count * dt_bits(md.offsets_dt) / 8;
        return 0;
    }
    if (md.format_kind != dnnl_blocked || index != 0) return 0;
    size_t span = 1;
    for (int i = 0; i < md.ndims; ++i) span += (size_t)(md.dims[i] - 1) * (size_t)md.strides[i];
    return (span * dt_bits(md.data_type) + 7) / 8;
}
} // namespace qmm

static bool valid_dt(dnnl_data_type_t dt) { return dt_bits(dt) != 0; }

extern "C" {

/* ------------------------------------------------------------------ engine */
size_t dnnl_engine_get_count(dnnl_engine_kind_t kind) {
    if (kind != dnnl_gpu) return 0; // there is no CPU engine
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return (size_t)n;
}

dnnl_status_t dnnl_engine_create(dnnl_engine_t *engine, dnnl_engine_kind_t kind, size_t index) {
    if (!engine) return dnnl_invalid_arguments;
    if (kind != dnnl_gpu) return dnnl_invalid_arguments;
    // Host-logic testing without a GPU: a device-less engine on which
    // descriptors, attributes and primitive descriptors can be created and
    // queried.  It owns no memory and executes nothing (runtime_error).
    if (getenv("DNNL_B200_NO_DEVICE") && index == 0 && dnnl_engine_get_count(kind) == 0) {
        auto *e = new dnnl_engine;
        e->device = -1;
        *engine = e;
        return dnnl_success;
    }
    if (index >= dnnl_engine_get_count(kind)) return dnnl_invalid_arguments;
    cudaDeviceProp prop;
    if (!cuda_ok(cudaGetDeviceProperties(&prop, (int)index), "cudaGetDeviceProperties")) return dnnl_runtime_error;
    if (prop.major != 10) {
        set_last_error("the CUDA engine requires a compute capability 10.x device");
        return dnnl_unimplemented;
    }
    if (!cuda_ok(cudaSetDevice((int)index), "cudaSetDevice")) return dnnl_runtime_error;
    auto *e = new dnnl_engine;
    e->device = (int)index;
    e->sm_count = prop.multiProcessorCount;
    if (!cuda_ok(cudaMalloc(&e->status_word, sizeof(int)), "cudaMalloc")
            || !cuda_ok(cudaMemset(e->status_word, 0, sizeof(int)), "cudaMemset")) {
        delete e;
        return dnnl_out_of_memory;
    }
    *engine = e;
    return dnnl_success;
}

dnnl_status_t dnnl_cuda_interop_engine_create(dnnl_engine_t *engine, int device) {
    if (device < 0) return dnnl_invalid_arguments;
    return dnnl_engine_create(engine, dnnl_gpu, (size_t)device);
}

dnnl_status_t dnnl_cuda_interop_engine_get_device(dnnl_engine_t engine, int *device) {
    if (!engine || !device) return dnnl_invalid_arguments;
    *device = engine->device;
    return dnnl_success;
}

dnnl_status_t dnnl_engine_get_kind(dnnl_engine_t engine, dnnl_engine_kind_t *kind) {
    if (!engine || !kind) return dnnl_invalid_arguments;
    *kind = dnnl_gpu;
    return dnnl_success;
}

dnnl_status_t dnnl_engine_destroy(dnnl_engine_t engine) {
    if (!engine) return dnnl_success;
    if (engine->refs.fetch_sub(1) == 1) {
        if (engine->status_word) cudaFree(engine->status_word);
        delete engine;
    }
    return dnnl_success;
}

/* ------------------------------------------------------------------ stream */
dnnl_status_t dnnl_stream_create(dnnl_stream_t *stream, dnnl_engine_t engine, unsigned flags) {
    if (!stream || !engine) return dnnl_invalid_arguments;
    if (flags & ~(unsigned)(dnnl_stream_in_order | dnnl_stream_out_of_order | 0x4u)) return dnnl_invalid_arguments;
    auto *s = new dnnl_stream;
    s->engine = engine;
    s->flags = flags;
    if (engine->device < 0) { // device-less engine: a stream that runs nothing
        s->owned = false;
        engine->refs.fetch_add(1);
        *stream = s;
        return dnnl_success;
    }
    cudaSetDevice(engine->device);
    // out-of-order streams are accepted and executed in order
    if (!cuda_ok(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking), "cudaStreamCreate")) {
        delete s;
        return dnnl_runtime_error;
    }
    engine->refs.fetch_add(1);
    *stream = s;
    return dnnl_success;
}

dnnl_status_t dnnl_cuda_interop_stream_create(dnnl_stream_t *stream, dnnl_engine_t engine, void *cuda_stream) {
    if (!stream || !engine) return dnnl_invalid_arguments;
    auto *s = new dnnl_stream;
    s->engine = engine;
    s->flags = dnnl_stream_in_order;
    s->stream = (cudaStream_t)cuda_stream;
    s->owned = false;
    engine->refs.fetch_add(1);
    *stream = s;
    return dnnl_success;
}

dnnl_status_t dnnl_cuda_interop_stream_get_cuda_stream(dnnl_stream_t stream, void **cuda_stream) {
    if (!stream || !cuda_stream) return dnnl_invalid_arguments;
    *cuda_stream = (void *)stream->stream;
    return dnnl_success;
}

dnnl_status_t dnnl_stream_get_engine(const_dnnl_stream_t stream, dnnl_engine_t *engine) {
    if (!stream || !engine) return dnnl_invalid_arguments;
    *engine = stream->engine;
    return dnnl_success;
}

dnnl_status_t dnnl_stream_wait(dnnl_stream_t stream) {
    if (!stream) return dnnl_invalid_arguments;
    if (stream->engine->device < 0) return dnnl_success;
    if (!cuda_ok(cudaStreamSynchronize(stream->stream), "cudaStreamSynchronize")) return dnnl_runtime_error;
    // surface errors recorded by kernels (e.g. invalid grouped offsets)
    int st = 0;
    if (!cuda_ok(cudaMemcpy(&st, stream->engine->status_word, sizeof(int), cudaMemcpyDeviceToHost), "status read"))
        return dnnl_runtime_error;
    if (st != 0) {
        cudaMemset(stream->engine->status_word, 0, sizeof(int));
        set_last_error("a kernel reported status " + std::to_string(st));
        return (dnnl_status_t)st;
    }
    return dnnl_success;
}

dnnl_status_t dnnl_stream_destroy(dnnl_stream_t stream) {
    if (!stream) return dnnl_success;
    if (stream->owned && stream->stream) {
        cudaStreamSynchronize(stream->stream);
        cudaStreamDestroy(stream->stream);
    }
    profiling_clear(stream);
    dnnl_engine_destroy(stream->engine);
    delete stream;
    return dnnl_success;
}

/* ----------------------------------------------------------------- service */
const dnnl_version_t *dnnl_version(void) {
    static const dnnl_version_t v = {3, 14, 0, "b200-native", 0u /* no CPU runtime */, DNNL_RUNTIME_CUDA};
    return &v;
}
dnnl_status_t dnnl_set_verbose(int level) {
    if (level < 0) return dnnl_invalid_arguments;
    g_verbose = level;
    return dnnl_success;
}
dnnl_status_t dnnl_get_default_fpmath_mode(dnnl_fpmath_mode_t *mode) {
    if (!mode) return dnnl_invalid_arguments;
    *mode = g_default_fpmath;
    return dnnl_success;
}
dnnl_status_t dnnl_set_default_fpmath_mode(dnnl_fpmath_mode_t mode) {
    if ((int)mode < 0 || (int)mode > (int)dnnl_fpmath_mode_tf32) return dnnl_invalid_arguments;
    g_default_fpmath = mode;
    return dnnl_success;
}
dnnl_status_t dnnl_get_primitive_cache_capacity(int *capacity) {
    if (!capacity) return dnnl_invalid_arguments;
    *capacity = g_cache_capacity;
    return dnnl_success;
}
dnnl_status_t dnnl_set_primitive_cache_capacity(int capacity) {
    if (capacity < 0) return dnnl_invalid_arguments;
    g_cache_capacity = capacity; // primitives hold no compiled state: nothing to cache
    return dnnl_success;
}
uint64_t dnnl_cuda_interop_launch_count(void) { return g_launches.load(); }
const char *dnnl_cuda_interop_last_error(void) { return g_last_error.c_str(); }

/* ------------------------------------------------------- memory descriptor */
static dnnl_status_t md_check_common(int ndims, const dnnl_dims_t dims, dnnl_data_type_t dt) {
    if (ndims == 0) return dnnl_success;
    if (ndims < 0 || ndims > DNNL_MAX_NDIMS || !dims || !valid_dt(dt)) return dnnl_invalid_arguments;
    for (int i = 0; i < ndims; ++i)
        if (dims[i] < 0 && dims[i] != DNNL_RUNTIME_DIM_VAL) return dnnl_invalid_arguments;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_create_with_strides(dnnl_memory_desc_t *memory_desc, int ndims,
        const dnnl_dims_t dims, dnnl_data_type_t data_type, const dnnl_dims_t strides) {
    if (!memory_desc) return dnnl_invalid_arguments;
    dnnl_status_t st = md_check_common(ndims, dims, data_type);
    if (st != dnnl_success) return st;
    auto *md = new dnnl_memory_desc;
    if (ndims == 0) { *memory_desc = md; return dnnl_success; }
    md->ndims = ndims;
    md->data_type = data_type;
    md->format_kind = dnnl_blocked;
    bool runtime = false; // open dims, or open strides of known dims
    for (int i = 0; i < ndims; ++i) {
        runtime = runtime || dims[i] == DNNL_RUNTIME_DIM_VAL || (strides && strides[i] == DNNL_RUNTIME_DIM_VAL);
        md->dims[i] = dims[i];
    }
    if (runtime) {
        // dims left open until execution (src/common/memory_desc.cpp:245-300): the given strides
        // are taken as they are; dense strides are known up to the first open dim from the right
        dnnl_dim_t acc = 1;
        for (int i = ndims - 1; i >= 0; --i) {
            if (strides) {
                if (strides[i] < 0 && strides[i] != DNNL_RUNTIME_DIM_VAL) { delete md; return dnnl_invalid_arguments; }
                md->strides[i] = strides[i];
            } else {
                md->strides[i] = acc;
                if (acc != DNNL_RUNTIME_DIM_VAL)
                    acc = md->dims[i] == DNNL_RUNTIME_DIM_VAL ? DNNL_RUNTIME_DIM_VAL : acc * (md->dims[i] == 0 ? 1 : md->dims[i]);
            }
        }
        *memory_desc = md;
        return dnnl_success;
    }
    if (strides) {
        for (int i = 0; i < ndims; ++i) {
            if (strides[i] < 0) { delete md; return dnnl_invalid_arguments; }
            md->strides[i] = strides[i];
        }
        // Dense-in-some-order check: going from the smallest stride up, each
        // stride must be at least the extent covered so far (a zero stride is
        // a broadcast, a unit dim is exempt); sub-byte types need even strides
        // above 1 (src/common/memory_desc.cpp:163-191).
        int perm[DNNL_MAX_NDIMS];
        for (int i = 0; i < ndims; ++i) perm[i] = i;
        for (int i = 0; i < ndims; ++i)
            for (int j = i + 1; j < ndims; ++j)
                if (md->strides[perm[j]] < md->strides[perm[i]]) std::swap(perm[i], perm[j]);
        dnnl_dim_t min_stride = 1;
        bool empty = false; // a tensor without elements has no layout to check
        for (int i = 0; i < ndims; ++i) empty = empty || md->dims[i] == 0;
        for (int idx = 0; idx < ndims && !empty; ++idx) {
            const int d = perm[idx];
            if (md->strides[d] == 0 || md->dims[d] == 1) continue;
            if (md->strides[d] < min_stride) { delete md; return dnnl_invalid_arguments; }
            if (dt_bits(data_type) == 4 && md->strides[d] > 1 && (md->strides[d] % 2)) {
                delete md;
                return dnnl_invalid_arguments;
            }
            min_stride = md->strides[d] * md->dims[d];
        }
    } else {
        dnnl_dim_t acc = 1;
        for (int i = ndims - 1; i >= 0; --i) {
            md->strides[i] = acc;
            acc *= md->dims[i] == 0 ? 1 : md->dims[i];
        }
    }
    *memory_desc = md;
    return dnnl_success;
}

// The two entry points the reference's test driver declares for itself (src/common/memory_desc.cpp:1140-1158):
// a descriptor from a tag written as letters, outermost dim first ("acb"), and a data type changed in place.
// Plain permutations only: a tag with blocks (capital letters, digits) is unimplemented.
dnnl_status_t dnnl_memory_desc_create_with_string_tag(dnnl_memory_desc_t *memory_desc, int ndims, const dnnl_dims_t dims,
        dnnl_data_type_t data_type, const char *tag) {
    if (!memory_desc || !tag) return dnnl_invalid_arguments;
    dnnl_status_t st = md_check_common(ndims, dims, data_type);
    if (st != dnnl_success) return st;
    if ((int)std::strlen(tag) != ndims || ndims == 0) return dnnl_invalid_arguments;
    int order[DNNL_MAX_NDIMS];
    bool seen[DNNL_MAX_NDIMS] = {};
    for (int i = 0; i < ndims; ++i) {
        const char c = tag[i];
        if (c >= 'A' && c <= 'L') return dnnl_unimplemented;
        if (c < 'a' || c >= 'a' + ndims || seen[c - 'a']) return dnnl_invalid_arguments;
        seen[c - 'a'] = true;
        order[i] = c - 'a';
    }
    dnnl_dims_t strides = {};
    dnnl_dim_t acc = 1;
    for (int i = ndims - 1; i >= 0; --i) {
        strides[order[i]] = acc;
        const dnnl_dim_t d = dims[order[i]];
        acc = (acc == DNNL_RUNTIME_DIM_VAL || d == DNNL_RUNTIME_DIM_VAL) ? DNNL_RUNTIME_DIM_VAL : acc * (d == 0 ? 1 : d);
    }
    return dnnl_memory_desc_create_with_strides(memory_desc, ndims, dims, data_type, strides);
}
dnnl_status_t dnnl_memory_desc_set_data_type(dnnl_memory_desc_t memory_desc, dnnl_data_type_t data_type) {
    if (!memory_desc) return dnnl_invalid_arguments;
    memory_desc->data_type = data_type;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_create_with_tag(dnnl_memory_desc_t *memory_desc, int ndims,
        const dnnl_dims_t dims, dnnl_data_type_t data_type, dnnl_format_tag_t tag) {
    if (!memory_desc) return dnnl_invalid_arguments;
    dnnl_status_t st = md_check_common(ndims, dims, data_type);
    if (st != dnnl_success) return st;
    if (ndims == 0 || tag == dnnl_format_tag_undef) {
        if (ndims != 0 && tag == dnnl_format_tag_undef) return dnnl_invalid_arguments;
        *memory_desc = new dnnl_memory_desc;
        return dnnl_success;
    }
    if (tag == dnnl_format_tag_any) {
        // a layout the library is to choose needs the dims (src/common/memory_desc.cpp: `any` with
        // run-time dims is refused)
        for (int i = 0; i < ndims; ++i)
            if (dims[i] == DNNL_RUNTIME_DIM_VAL) return dnnl_invalid_arguments;
        auto *md = new dnnl_memory_desc;
        md->ndims = ndims;
        md->data_type = data_type;
        md->format_kind = dnnl_format_kind_any;
        for (int i = 0; i < ndims; ++i) md->dims[i] = dims[i];
        *memory_desc = md;
        return dnnl_success;
    }
    // permutation of the plain tags: order[i] = logical dim at position i,
    // outermost first
    int order[4];
    int tag_ndims = 0;
    auto set = [&](int n, int a, int b, int c, int d) { tag_ndims = n; order[0] = a; order[1] = b; order[2] = c; order[3] = d; };
    switch ((int)tag) {
        case dnnl_a: set(1, 0, 0, 0, 0); break;
        case dnnl_ab: set(2, 0, 1, 0, 0); break;
        case dnnl_ba: set(2, 1, 0, 0, 0); break;
        case dnnl_abc: set(3, 0, 1, 2, 0); break;
        case dnnl_acb: set(3, 0, 2, 1, 0); break;
        case dnnl_bac: set(3, 1, 0, 2, 0); break;
        case dnnl_bca: set(3, 1, 2, 0, 0); break;
        case dnnl_cab: set(3, 2, 0, 1, 0); break;
        case dnnl_cba: set(3, 2, 1, 0, 0); break;
        case dnnl_abcd: set(4, 0, 1, 2, 3); break;
        default: return dnnl_unimplemented; // blocked layouts are not part of this path
    }
    if (tag_ndims != ndims) return dnnl_invalid_arguments;
    dnnl_dims_t strides = {};
    dnnl_dim_t acc = 1;
    for (int i = ndims - 1; i >= 0; --i) { // a stride beyond an open dim is open too
        strides[order[i]] = acc;
        const dnnl_dim_t d = dims[order[i]];
        acc = (acc == DNNL_RUNTIME_DIM_VAL || d == DNNL_RUNTIME_DIM_VAL) ? DNNL_RUNTIME_DIM_VAL : acc * (d == 0 ? 1 : d);
    }
    return dnnl_memory_desc_create_with_strides(memory_desc, ndims, dims, data_type, strides);
}

// src/common/memory_desc.cpp:417-473: 2D only, s32 offsets, one variable dim
dnnl_status_t dnnl_memory_desc_create_with_grouped_encoding(dnnl_memory_desc_t *memory_desc, int ndims,
        const dnnl_dims_t dims, dnnl_data_type_t data_type, int variable_dim_idx, dnnl_dim_t group_count,
        dnnl_data_type_t offsets_dt) {
    if (!memory_desc) return dnnl_invalid_arguments;
    dnnl_status_t st = md_check_common(ndims, dims, data_type);
    if (st != dnnl_success) return st;
    if (ndims != 2) return dnnl_unimplemented;
    if (group_count <= 0) return dnnl_invalid_arguments;
    if (variable_dim_idx < 0 || variable_dim_idx >= ndims) return dnnl_invalid_arguments;
    if (offsets_dt != dnnl_s32) return dnnl_unimplemented;
    auto *md = new dnnl_memory_desc;
    md->ndims = ndims;
    md->data_type = data_type;
    md->format_kind = dnnl_format_kind_sparse;
    md->encoding = dnnl_grouped;
    md->variable_dim_idx = variable_dim_idx;
    md->group_count = group_count;
    md->offsets_dt = offsets_dt;
    for (int i = 0; i < ndims; ++i) md->dims[i] = dims[i];
    // values are concatenated along the variable dim: row-major when it is 0
    if (variable_dim_idx == 0) { md->strides[0] = dims[1]; md->strides[1] = 1; }
    else { md->strides[0] = 1; md->strides[1] = dims[0]; }
    *memory_desc = md;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_create_host_scalar(dnnl_memory_desc_t *memory_desc, dnnl_data_type_t data_type) {
    if (!memory_desc || !valid_dt(data_type) || dt_bits(data_type) < 8) return dnnl_invalid_arguments;
    auto *md = new dnnl_memory_desc;
    md->ndims = 1;
    md->dims[0] = 1;
    md->strides[0] = 1;
    md->data_type = data_type;
    md->format_kind = dnnl_format_kind_host_scalar;
    *memory_desc = md;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_clone(dnnl_memory_desc_t *memory_desc, const_dnnl_memory_desc_t existing) {
    if (!memory_desc || !existing) return dnnl_invalid_arguments;
    *memory_desc = new dnnl_memory_desc(*existing);
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_destroy(dnnl_memory_desc_t memory_desc) {
    delete memory_desc;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_reshape(dnnl_memory_desc_t *out, const_dnnl_memory_desc_t in, int ndims,
        const dnnl_dims_t dims) {
    if (!out || !in || !dims || ndims <= 0 || ndims > DNNL_MAX_NDIMS) return dnnl_invalid_arguments;
    if (in->format_kind != dnnl_blocked) return dnnl_invalid_arguments;
    dnnl_dim_t n = 1;
    for (int i = 0; i < ndims; ++i) n *= dims[i];
    if (n != in->nelems()) return dnnl_invalid_arguments;
    if (in->has_runtime_dims()) return dnnl_invalid_arguments;
    // dense row-major: the new shape is dense row-major too
    bool dense = true;
    dnnl_dim_t acc = 1;
    for (int i = in->ndims - 1; i >= 0; --i) {
        if (in->dims[i] != 1 && in->strides[i] != acc) dense = false;
        acc *= in->dims[i];
    }
    if (dense || n == 0) return dnnl_memory_desc_create_with_strides(out, ndims, dims, in->data_type, nullptr);
    // Any other plain layout: old and new dims are matched from the left in groups of equal
    // products (unit dims come and go freely); the old dims of a group must follow one another in
    // memory without gaps, and the new dims of the group then split that run.
    dnnl_dims_t st = {};
    bool assigned[DNNL_MAX_NDIMS] = {};
    int i = 0, j = 0;
    while (true) {
        while (i < in->ndims && in->dims[i] == 1) ++i;
        while (j < ndims && dims[j] == 1) ++j;
        if (i >= in->ndims || j >= ndims) break;
        int i1 = i, j1 = j;
        dnnl_dim_t po = in->dims[i], pn = dims[j];
        while (po != pn) {
            if (po < pn) {
                if (++i1 >= in->ndims) return dnnl_invalid_arguments;
                po *= in->dims[i1];
            } else {
                if (++j1 >= ndims) return dnnl_invalid_arguments;
                pn *= dims[j1];
            }
        }
        int last = i1; // the innermost old dim of the group that is not a unit dim
        while (in->dims[last] == 1) --last;
        dnnl_dim_t run = in->strides[last] * in->dims[last];
        for (int k = last - 1; k >= i; --k) {
            if (in->dims[k] == 1) continue;
            if (in->strides[k] != run) return dnnl_invalid_arguments; // a gap or another order inside the group
            run *= in->dims[k];
        }
        dnnl_dim_t s = in->strides[last];
        for (int t = j1; t >= j; --t) {
            st[t] = s;
            assigned[t] = true;
            s *= dims[t];
        }
        i = i1 + 1;
        j = j1 + 1;
    }
    if (i < in->ndims || j < ndims) return dnnl_invalid_arguments;
    for (int t = ndims - 1; t >= 0; --t) // unit dims: the extent of what lies to their right
        if (!assigned[t]) st[t] = t + 1 < ndims ? st[t + 1] * dims[t + 1] : 1;
    return dnnl_memory_desc_create_with_strides(out, ndims, dims, in->data_type, st);
}

dnnl_status_t dnnl_memory_desc_permute_axes(dnnl_memory_desc_t *out, const_dnnl_memory_desc_t in, const int *perm) {
    if (!out || !in || !perm) return dnnl_invalid_arguments;
    if (in->format_kind != dnnl_blocked) return dnnl_invalid_arguments;
    bool seen[DNNL_MAX_NDIMS] = {};
    for (int i = 0; i < in->ndims; ++i) {
        if (perm[i] < 0 || perm[i] >= in->ndims || seen[perm[i]]) return dnnl_invalid_arguments;
        seen[perm[i]] = true;
    }
    auto *md = new dnnl_memory_desc(*in);
    for (int i = 0; i < in->ndims; ++i) { // dim i of `in` becomes dim perm[i]
        md->dims[perm[i]] = in->dims[i];
        md->strides[perm[i]] = in->strides[i];
    }
    *out = md;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_query_v2(const_dnnl_memory_desc_t md, dnnl_query_t what, int index, void *result) {
    if (!md || !result) return dnnl_invalid_arguments;
    static const dnnl_dims_t zero_dims = {};
    switch ((int)what) {
        case dnnl_query_ndims_s32: *(int *)result = md->ndims; break;
        case dnnl_query_dims: *(const dnnl_dims_t **)result = &md->dims; break;
        case dnnl_query_padded_dims: *(const dnnl_dims_t **)result = &md->dims; break;
        case dnnl_query_padded_offsets: *(const dnnl_dims_t **)result = &zero_dims; break;
        case dnnl_query_data_type:
            if (index == 0) *(dnnl_data_type_t *)result = md->data_type;
            else if (index == 1 && md->is_grouped()) *(dnnl_data_type_t *)result = md->offsets_dt;
            else return dnnl_invalid_arguments;
            break;
        case dnnl_query_submemory_offset_s64: *(dnnl_dim_t *)result = md->offset0; break;
        case dnnl_query_format_kind: *(dnnl_format_kind_t *)result = md->format_kind; break;
        case dnnl_query_strides:
            if (md->format_kind != dnnl_blocked) return dnnl_invalid_arguments;
            *(const dnnl_dims_t **)result = &md->strides;
            break;
        case dnnl_query_inner_nblks_s32:
            if (md->format_kind != dnnl_blocked) return dnnl_invalid_arguments;
            *(int *)result = 0;
            break;
        case dnnl_query_inner_blks:
        case dnnl_query_inner_idxs:
            if (md->format_kind != dnnl_blocked) return dnnl_invalid_arguments;
            *(const dnnl_dims_t **)result = &zero_dims;
            break;
        case dnnl_query_sparse_encoding: *(dnnl_sparse_encoding_t *)result = md->encoding; break;
        case dnnl_query_nnz_s64: *(dnnl_dim_t *)result = 0; break;
        case dnnl_query_num_handles_s32: *(int *)result = md->is_grouped() ? 2 : (md->ndims ? 1 : 0); break;
        default: return dnnl_unimplemented;
    }
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_query(const_dnnl_memory_desc_t md, dnnl_query_t what, void *result) {
    return dnnl_memory_desc_query_v2(md, what, 0, result);
}

int dnnl_memory_desc_equal(const_dnnl_memory_desc_t a, const_dnnl_memory_desc_t b) {
    if (a == b) return 1;
    if (!a || !b) return 0;
    if (a->ndims != b->ndims || a->data_type != b->data_type || a->format_kind != b->format_kind) return 0;
    for (int i = 0; i < a->ndims; ++i) {
        if (a->dims[i] != b->dims[i]) return 0;
        if (a->format_kind == dnnl_blocked && a->strides[i] != b->strides[i]) return 0;
    }
    if (a->is_grouped())
        return a->variable_dim_idx == b->variable_dim_idx && a->group_count == b->group_count
                && a->offsets_dt == b->offsets_dt;
    return a->offset0 == b->offset0;
}

size_t dnnl_memory_desc_get_size_v2(const_dnnl_memory_desc_t md, int index) { return md ? md_bytes(*md, index) : 0; }
size_t dnnl_memory_desc_get_size(const_dnnl_memory_desc_t md) { return dnnl_memory_desc_get_size_v2(md, 0); }
size_t dnnl_data_type_size(dnnl_data_type_t dt) {
    const size_t b = dt_bits(dt);
    return b == 4 ? 1 : b / 8; // sub-byte types report one byte
}

/* ------------------------------------------------------------------ memory */
dnnl_status_t dnnl_memory_create_v2(dnnl_memory_t *memory, const_dnnl_memory_desc_t md, dnnl_engine_t engine,
        int nhandles, void **handles) {
    if (!memory || !md || !engine) return dnnl_invalid_arguments;
    if (md->format_kind == dnnl_format_kind_any) return dnnl_invalid_arguments;
    if (md->format_kind == dnnl_format_kind_host_scalar) return dnnl_invalid_arguments;
    const int expected = md->is_grouped() ? 2 : (md->ndims ? 1 : 0);
    if (nhandles != expected && !(expected == 0 && nhandles <= 1)) return dnnl_invalid_arguments;
    if (nhandles > 0 && !handles) return dnnl_invalid_arguments;
    auto *m = new dnnl_memory;
    m->md = *md;
    m->engine = engine;
    if (engine->device >= 0) cudaSetDevice(engine->device);
    for (int i = 0; i < nhandles && i < 2; ++i) {
        if (handles[i] == DNNL_MEMORY_ALLOCATE) {
            const size_t bytes = md_bytes(*md, i);
            if (bytes && engine->device < 0) {
                set_last_error("a device-less engine cannot allocate memory");
                delete m;
                return dnnl_runtime_error;
            }
            if (bytes) {
                if (!cuda_ok(cudaMalloc(&m->handles[i], bytes), "cudaMalloc")) {
                    for (int j = 0; j < i; ++j)
                        if (m->owned[j]) cudaFree(m->handles[j]);
                    delete m;
                    return dnnl_out_of_memory;
                }
                m->owned[i] = true;
            }
        } else {
            m->handles[i] = handles[i]; // user device pointer (or NONE)
        }
    }
    engine->refs.fetch_add(1);
    *memory = m;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_create(dnnl_memory_t *memory, const_dnnl_memory_desc_t md, dnnl_engine_t engine, void *handle) {
    if (!md) return dnnl_invalid_arguments;
    if (md->is_grouped()) return dnnl_invalid_arguments; // needs two handles: use _v2
    void *h[1] = {handle};
    return dnnl_memory_create_v2(memory, md, engine, md->ndims ? 1 : 0, h);
}

dnnl_status_t dnnl_cuda_interop_memory_create(dnnl_memory_t *memory, const_dnnl_memory_desc_t md,
        dnnl_engine_t engine, void *device_ptr) {
    return dnnl_memory_create(memory, md, engine, device_ptr);
}

dnnl_status_t dnnl_memory_create_host_scalar(dnnl_memory_t *memory, const_dnnl_memory_desc_t md, void *scalar_ptr) {
    if (!memory || !md || !scalar_ptr) return dnnl_invalid_arguments;
    if (md->format_kind != dnnl_format_kind_host_scalar) return dnnl_invalid_arguments;
    auto *m = new dnnl_memory;
    m->md = *md;
    m->is_host_scalar = true;
    memcpy(&m->host_scalar, scalar_ptr, dt_bits(md->data_type) / 8);
    *memory = m;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_get_host_scalar_value(const_dnnl_memory_t memory, void *value) {
    if (!memory || !value || !memory->is_host_scalar) return dnnl_invalid_arguments;
    memcpy(value, &memory->host_scalar, dt_bits(memory->md.data_type) / 8);
    return dnnl_success;
}

dnnl_status_t dnnl_memory_set_host_scalar_value(dnnl_memory_t memory, const void *value) {
    if (!memory || !value || !memory->is_host_scalar) return dnnl_invalid_arguments;
    memcpy(&memory->host_scalar, value, dt_bits(memory->md.data_type) / 8);
    return dnnl_success;
}

dnnl_status_t dnnl_memory_get_memory_desc(const_dnnl_memory_t memory, const_dnnl_memory_desc_t *md) {
    if (!memory || !md) return dnnl_invalid_arguments;
    *md = &memory->md;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_get_engine(const_dnnl_memory_t memory, dnnl_engine_t *engine) {
    if (!memory || !engine) return dnnl_invalid_arguments;
    *engine = memory->engine;
    return dnnl_success;
}

// map: the device buffer is copied to a host staging buffer the caller may
// read and write; unmap copies it back and releases it.
dnnl_status_t dnnl_memory_map_data_v2(const_dnnl_memory_t cmem, void **mapped_ptr, int index) {
    auto *memory = const_cast<dnnl_memory_t>(cmem);
    if (!memory || !mapped_ptr || index < 0 || index > 1) return dnnl_invalid_arguments;
    if (memory->is_host_scalar) return dnnl_invalid_arguments;
    if (memory->mapped[index]) return dnnl_invalid_arguments; // already mapped
    const size_t bytes = md_bytes(memory->md, index);
    if (!memory->handles[index] || bytes == 0) { *mapped_ptr = nullptr; return dnnl_success; }
    cudaSetDevice(memory->engine->device);
    void *host = malloc(bytes);
    if (!host) return dnnl_out_of_memory;
    if (!cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize")
            || !cuda_ok(cudaMemcpy(host, memory->handles[index], bytes, cudaMemcpyDeviceToHost), "map copy")) {
        free(host);
        return dnnl_runtime_error;
    }
    memory->mapped[index] = host;
    *mapped_ptr = host;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_unmap_data_v2(const_dnnl_memory_t cmem, void *mapped_ptr, int index) {
    auto *memory = const_cast<dnnl_memory_t>(cmem);
    if (!memory || index < 0 || index > 1) return dnnl_invalid_arguments;
    if (!mapped_ptr && !memory->mapped[index]) return dnnl_success;
    if (memory->mapped[index] != mapped_ptr) return dnnl_invalid_arguments;
    const size_t bytes = md_bytes(memory->md, index);
    cudaSetDevice(memory->engine->device);
    const bool ok = cuda_ok(cudaMemcpy(memory->handles[index], mapped_ptr, bytes, cudaMemcpyHostToDevice), "unmap copy");
    free(mapped_ptr);
    memory->mapped[index] = nullptr;
    return ok ? dnnl_success : dnnl_runtime_error;
}

dnnl_status_t dnnl_memory_map_data(const_dnnl_memory_t memory, void **mapped_ptr) {
    return dnnl_memory_map_data_v2(memory, mapped_ptr, 0);
}
dnnl_status_t dnnl_memory_unmap_data(const_dnnl_memory_t memory, void *mapped_ptr) {
    return dnnl_memory_unmap_data_v2(memory, mapped_ptr, 0);
}

dnnl_status_t dnnl_memory_get_data_handle_v2(const_dnnl_memory_t memory, void **handle, int index) {
    if (!memory || !handle || index < 0 || index > 1) return dnnl_invalid_arguments;
    *handle = memory->is_host_scalar ? (void *)&memory->host_scalar : memory->handles[index];
    return dnnl_success;
}

dnnl_status_t dnnl_memory_set_data_handle_v2(dnnl_memory_t memory, void *handle, int index) {
    if (!memory || index < 0 || index > 1 || memory->is_host_scalar) return dnnl_invalid_arguments;
    if (memory->owned[index]) {
        cudaFree(memory->handles[index]);
        memory->owned[index] = false;
    }
    memory->handles[index] = handle;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_get_data_handle(const_dnnl_memory_t memory, void **handle) {
    return dnnl_memory_get_data_handle_v2(memory, handle, 0);
}
dnnl_status_t dnnl_memory_set_data_handle(dnnl_memory_t memory, void *handle) {
    return dnnl_memory_set_data_handle_v2(memory, handle, 0);
}

dnnl_status_t dnnl_memory_destroy(dnnl_memory_t memory) {
    if (!memory) return dnnl_success;
    for (int i = 0; i < 2; ++i) {
        if (memory->mapped[i]) free(memory->mapped[i]);
        if (memory->owned[i]) cudaFree(memory->handles[i]);
    }
    if (memory->engine) dnnl_engine_destroy(memory->engine);
    delete memory;
    return dnnl_success;
}

/* -------------------------------------------------------------- attributes */
dnnl_status_t dnnl_primitive_attr_create(dnnl_primitive_attr_t *attr) {
    if (!attr) return dnnl_invalid_arguments;
    *attr = new dnnl_primitive_attr;
    (*attr)->fpmath = g_default_fpmath;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_clone(dnnl_primitive_attr_t *attr, const_dnnl_primitive_attr_t existing) {
    if (!attr || !existing) return dnnl_invalid_arguments;
    *attr = new dnnl_primitive_attr(*existing);
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_destroy(dnnl_primitive_attr_t attr) {
    delete attr;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_fpmath_mode_v2(const_dnnl_primitive_attr_t attr, dnnl_fpmath_mode_t *mode, int *apply_to_int) {
    if (!attr) return dnnl_invalid_arguments;
    if (mode) *mode = attr->fpmath;
    if (apply_to_int) *apply_to_int = attr->apply_to_int;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_fpmath_mode(const_dnnl_primitive_attr_t attr, dnnl_fpmath_mode_t *mode) {
    if (!attr || !mode) return dnnl_invalid_arguments;
    *mode = attr->fpmath;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_fpmath_mode_v2(dnnl_primitive_attr_t attr, dnnl_fpmath_mode_t mode, int apply_to_int) {
    if (!attr) return dnnl_invalid_arguments;
    if ((int)mode < 0 || (int)mode > (int)dnnl_fpmath_mode_tf32) return dnnl_invalid_arguments;
    attr->fpmath = mode;
    attr->apply_to_int = apply_to_int != 0;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_fpmath_mode(dnnl_primitive_attr_t attr, dnnl_fpmath_mode_t mode) {
    return dnnl_primitive_attr_set_fpmath_mode_v2(attr, mode, 0);
}
dnnl_status_t dnnl_primitive_attr_get_deterministic(const_dnnl_primitive_attr_t attr, int *value) {
    if (!attr || !value) return dnnl_invalid_arguments;
    *value = attr->deterministic;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_deterministic(dnnl_primitive_attr_t attr, int value) {
    if (!attr) return dnnl_invalid_arguments;
    attr->deterministic = value != 0;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_accumulation_mode(const_dnnl_primitive_attr_t attr, dnnl_accumulation_mode_t *mode) {
    if (!attr || !mode) return dnnl_invalid_arguments;
    *mode = attr->acc_mode;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_accumulation_mode(dnnl_primitive_attr_t attr, dnnl_accumulation_mode_t mode) {
    if (!attr) return dnnl_invalid_arguments;
    if ((int)mode < 0 || (int)mode > (int)dnnl_accumulation_mode_f16) return dnnl_invalid_arguments;
    attr->acc_mode = mode;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_scratchpad_mode(const_dnnl_primitive_attr_t attr, dnnl_scratchpad_mode_t *mode) {
    if (!attr || !mode) return dnnl_invalid_arguments;
    *mode = attr->scratchpad_mode;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_scratchpad_mode(dnnl_primitive_attr_t attr, dnnl_scratchpad_mode_t mode) {
    if (!attr) return dnnl_invalid_arguments;
    if (mode != dnnl_scratchpad_mode_library && mode != dnnl_scratchpad_mode_user) return dnnl_invalid_arguments;
    attr->scratchpad_mode = mode;
    return dnnl_success;
}

static dnnl_status_t set_quant(std::map<int, quant_entry_t> &m, int arg, int mask, int group_ndims,
        const dnnl_dims_t group_dims, dnnl_data_type_t dt, int on_host, dnnl_quantization_mode_t qmode) {
    if (group_ndims != 0 && group_ndims != 2) return dnnl_invalid_arguments;
    if (group_ndims) {
        if (!group_dims) return dnnl_invalid_arguments;
        for (int i = 0; i < group_ndims; ++i)
            if (group_dims[i] <= 0) return dnnl_invalid_arguments;
        if (mask <= 0) return dnnl_invalid_arguments;
    }
    if (on_host && (mask != 0 || group_ndims != 0)) return dnnl_invalid_arguments;
    quant_entry_t e;
    e.set = true;
    e.mask = mask;
    e.dt = dt;
    e.group_ndims = group_ndims;
    if (group_ndims) { e.groups[0] = group_dims[0]; e.groups[1] = group_dims[1]; }
    e.on_host = on_host != 0;
    e.qmode = qmode;
    m[arg] = e;
    return dnnl_success;
}

// the arguments scales / zero-points may be set for (src/common/primitive_attr_quant.hpp:337-359, 390-406)
static bool scales_arg_ok(int arg) {
    if (arg == DNNL_ARG_SRC || arg == DNNL_ARG_WEIGHTS || arg == DNNL_ARG_DST || arg == DNNL_ARG_SRC_1 || arg == DNNL_ARG_SRC_2
            || arg == DNNL_ARG_WEIGHTS_1 || arg == DNNL_ARG_WEIGHTS_2)
        return true;
    if (arg & DNNL_ARG_MULTIPLE_SRC) return true;
    for (int a : {DNNL_ARG_SRC, DNNL_ARG_WEIGHTS, DNNL_ARG_DST})
        if (arg == (DNNL_ARG_ATTR_POST_OP_DW | a)) return true;
    return false;
}
static bool zero_points_arg_ok(int arg) {
    return arg == DNNL_ARG_SRC || arg == DNNL_ARG_WEIGHTS || arg == DNNL_ARG_DST || arg == DNNL_ARG_SRC_2
            || arg == DNNL_ARG_WEIGHTS_1 || arg == DNNL_ARG_WEIGHTS_2;
}

dnnl_status_t dnnl_primitive_attr_set_scales_v3(dnnl_primitive_attr_t attr, int arg, int mask, int ndims,
        const dnnl_dims_t group_dims, dnnl_data_type_t dt, int is_on_host, dnnl_quantization_mode_t qmode) {
    if (!attr || arg < 0 || mask < 0 || !scales_arg_ok(arg)) return dnnl_invalid_arguments;
    if (qmode != dnnl_quantization_mode_static_sazp && qmode != dnnl_quantization_mode_dynamic_mx
            && qmode != dnnl_quantization_mode_dynamic_fp)
        return dnnl_invalid_arguments;
    if (dt != dnnl_f32 && dt != dnnl_bf16 && dt != dnnl_f16 && dt != dnnl_e8m0 && dt != dnnl_f8_e4m3)
        return dnnl_invalid_arguments;
    if ((dt == dnnl_e8m0 || dt == dnnl_f8_e4m3) && mask <= 0) return dnnl_invalid_arguments;
    return set_quant(attr->scales, arg, mask, ndims, group_dims, dt, is_on_host, qmode);
}
dnnl_status_t dnnl_primitive_attr_set_scales_v2(dnnl_primitive_attr_t attr, int arg, int mask, int ndims,
        const dnnl_dims_t group_dims, dnnl_data_type_t dt, int is_on_host) {
    return dnnl_primitive_attr_set_scales_v3(attr, arg, mask, ndims, group_dims, dt, is_on_host, dnnl_quantization_mode_static_sazp);
}
dnnl_status_t dnnl_primitive_attr_set_scales(dnnl_primitive_attr_t attr, int arg, int mask, int group_ndims,
        const dnnl_dims_t group_dims, dnnl_data_type_t dt) {
    return dnnl_primitive_attr_set_scales_v3(attr, arg, mask, group_ndims, group_dims, dt, 0, dnnl_quantization_mode_static_sazp);
}
dnnl_status_t dnnl_primitive_attr_set_scales_mask(dnnl_primitive_attr_t attr, int arg, int mask) {
    if (!attr || arg < 0 || mask < 0 || !scales_arg_ok(arg)) return dnnl_invalid_arguments;
    return set_quant(attr->scales, arg, mask, 0, nullptr, dnnl_f32, 0, dnnl_quantization_mode_static_sazp);
}
dnnl_status_t dnnl_primitive_attr_set_zero_points_v2(dnnl_primitive_attr_t attr, int arg, int mask, int ndims,
        const dnnl_dims_t group_dims, dnnl_data_type_t dt, int is_on_host) {
    if (!attr || arg < 0 || mask < 0 || !zero_points_arg_ok(arg)) return dnnl_invalid_arguments;
    if (dt != dnnl_s32 && dt != dnnl_s8 && dt != dnnl_u8 && dt != dnnl_s4 && dt != dnnl_u4) return dnnl_invalid_arguments;
    if ((dt == dnnl_s4 || dt == dnnl_u4) && mask <= 0) return dnnl_invalid_arguments;
    if (arg != DNNL_ARG_SRC && arg != DNNL_ARG_WEIGHTS && !(dt == dnnl_s32 && ndims == 0)) return dnnl_invalid_arguments;
    return set_quant(attr->zero_points, arg, mask, ndims, group_dims, dt, is_on_host, dnnl_quantization_mode_static_sazp);
}
dnnl_status_t dnnl_primitive_attr_set_zero_points(dnnl_primitive_attr_t attr, int arg, int mask, int group_ndims,
        const dnnl_dims_t group_dims, dnnl_data_type_t dt) {
    return dnnl_primitive_attr_set_zero_points_v2(attr, arg, mask, group_ndims, group_dims, dt, 0);
}
dnnl_status_t dnnl_primitive_attr_set_zero_points_mask(dnnl_primitive_attr_t attr, int arg, int mask) {
    if (!attr || mask < 0 || !zero_points_arg_ok(arg)) return dnnl_invalid_arguments;
    return set_quant(attr->zero_points, arg, mask, 0, nullptr, dnnl_s32, 0, dnnl_quantization_mode_static_sazp);
}
dnnl_status_t dnnl_primitive_attr_set_precomputed_reductions(dnnl_primitive_attr_t attr, int arg, int mask,
        int group_ndims, const dnnl_dims_t group_dims, dnnl_data_type_t dt) {
    if (!attr || mask < 0 || group_ndims < 0) return dnnl_invalid_arguments;
    if (arg != DNNL_ARG_SRC && arg != DNNL_ARG_WEIGHTS) return dnnl_invalid_arguments;
    if (dt != dnnl_s32) return dnnl_invalid_arguments;
    return set_quant(attr->reductions, arg, mask, group_ndims, group_dims, dt, 0, dnnl_quantization_mode_static_sazp);
}
dnnl_status_t dnnl_primitive_attr_set_rounding(dnnl_primitive_attr_t attr, int arg, dnnl_rounding_mode_t mode) {
    if (!attr) return dnnl_invalid_arguments;
    if (mode == dnnl_rounding_mode_environment) attr->rounding.erase(arg);
    else attr->rounding[arg] = mode;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_rounding(dnnl_primitive_attr_t attr, int arg, dnnl_rounding_mode_t *mode) {
    if (!attr || !mode) return dnnl_invalid_arguments;
    auto it = attr->rounding.find(arg);
    *mode = it == attr->rounding.end() ? dnnl_rounding_mode_environment : it->second;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_post_ops(const_dnnl_primitive_attr_t attr, const_dnnl_post_ops_t *post_ops) {
    if (!attr || !post_ops) return dnnl_invalid_arguments;
    *post_ops = &attr->post_ops;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_post_ops(dnnl_primitive_attr_t attr, const_dnnl_post_ops_t post_ops) {
    if (!attr || !post_ops) return dnnl_invalid_arguments;
    attr->post_ops = *post_ops;
    return dnnl_success;
}

/* ---------------------------------------------------------------- post-ops */
dnnl_status_t dnnl_post_ops_create(dnnl_post_ops_t *post_ops) {
    if (!post_ops) return dnnl_invalid_arguments;
    *post_ops = new dnnl_post_ops;
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_clone(dnnl_post_ops_t *post_ops, const_dnnl_post_ops_t existing) {
    if (!post_ops || !existing) return dnnl_invalid_arguments;
    *post_ops = new dnnl_post_ops(*existing);
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_destroy(dnnl_post_ops_t post_ops) {
    delete post_ops;
    return dnnl_success;
}
int dnnl_post_ops_len(const_dnnl_post_ops_t post_ops) { return post_ops ? (int)post_ops->entries.size() : 0; }
dnnl_primitive_kind_t dnnl_post_ops_get_kind(const_dnnl_post_ops_t post_ops, int index) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_undefined_primitive;
    return post_ops->entries[index].kind;
}
static bool po_has_room(dnnl_post_ops_t po) { return po && (int)po->entries.size() < MAX_POST_OPS; }

dnnl_status_t dnnl_post_ops_append_sum(dnnl_post_ops_t post_ops, float scale, int32_t zero_point, dnnl_data_type_t dt) {
    if (!po_has_room(post_ops)) return post_ops ? dnnl_out_of_memory : dnnl_invalid_arguments;
    post_op_entry_t e;
    e.kind = dnnl_sum;
    e.scale = scale;
    e.zero_point = zero_point;
    e.sum_dt = dt;
    post_ops->entries.push_back(e);
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_get_params_sum(const_dnnl_post_ops_t post_ops, int index, float *scale,
        int32_t *zero_point, dnnl_data_type_t *dt) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_invalid_arguments;
    const auto &e = post_ops->entries[index];
    if (e.kind != dnnl_sum) return dnnl_invalid_arguments;
    if (scale) *scale = e.scale;
    if (zero_point) *zero_point = e.zero_point;
    if (dt) *dt = e.sum_dt;
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_append_eltwise(dnnl_post_ops_t post_ops, dnnl_alg_kind_t alg, float alpha, float beta) {
    if (!po_has_room(post_ops)) return post_ops ? dnnl_out_of_memory : dnnl_invalid_arguments;
    if ((int)alg < (int)dnnl_eltwise_relu || (int)alg > (int)dnnl_eltwise_hardswish) return dnnl_invalid_arguments;
    if ((alg == dnnl_eltwise_clip || alg == dnnl_eltwise_clip_v2) && beta < alpha) return dnnl_invalid_arguments;
    post_op_entry_t e;
    e.kind = dnnl_eltwise;
    e.alg = alg;
    e.alpha = alpha;
    e.beta = beta;
    e.scale = 1.f;
    post_ops->entries.push_back(e);
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_get_params_eltwise(const_dnnl_post_ops_t post_ops, int index, dnnl_alg_kind_t *alg,
        float *alpha, float *beta) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_invalid_arguments;
    const auto &e = post_ops->entries[index];
    if (e.kind != dnnl_eltwise) return dnnl_invalid_arguments;
    if (alg) *alg = e.alg;
    if (alpha) *alpha = e.alpha;
    if (beta) *beta = e.beta;
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_append_binary(dnnl_post_ops_t post_ops, dnnl_alg_kind_t alg, const_dnnl_memory_desc_t src1) {
    if (!po_has_room(post_ops)) return post_ops ? dnnl_out_of_memory : dnnl_invalid_arguments;
    if (!src1) return dnnl_invalid_arguments;
    if ((int)alg < (int)dnnl_binary_add || (int)alg > (int)dnnl_binary_ne) return dnnl_invalid_arguments;
    // `any` is allowed as in the reference (src/common/primitive_attr.cpp:228-258): the primitive
    // descriptor resolves it to the plain row-major layout
    post_op_entry_t e;
    e.kind = dnnl_binary;
    e.alg = alg;
    e.src1 = *src1;
    post_ops->entries.push_back(e);
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_get_params_binary(const_dnnl_post_ops_t post_ops, int index, dnnl_alg_kind_t *alg,
        const_dnnl_memory_desc_t *src1) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_invalid_arguments;
    const auto &e = post_ops->entries[index];
    if (e.kind != dnnl_binary) return dnnl_invalid_arguments;
    if (alg) *alg = e.alg;
    if (src1) *src1 = &e.src1;
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_append_prelu(dnnl_post_ops_t post_ops, int mask) {
    if (!po_has_room(post_ops)) return post_ops ? dnnl_out_of_memory : dnnl_invalid_arguments;
    post_op_entry_t e;
    e.kind = dnnl_prelu;
    e.prelu_mask = mask;
    post_ops->entries.push_back(e);
    return dnnl_success;
}

} // extern "C"
