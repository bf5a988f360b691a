// dnnl::reorder on the CUDA engine ("cuda:ref:reorder"): a quantizing /
// dequantizing copy between two plain strided layouts of one logical tensor,
//   dst = cvt((src_scale * (src - src_zp) [+ beta * dst]) / dst_scale + dst_zp)
// in the reference's operation order
// (src/cpu/reorder/simple_reorder.hpp:2621-2676; 4-bit sources :2391-2421,
// 4-bit targets :2256-2277), so results equal the reference's bit for bit.
// Descriptor checks follow src/common/reorder.cpp:67-150.
//
// One thread per element (per byte for 4-bit targets).  Threads walk the
// tensor in the order of the dst strides, smallest first, so the stores of a
// warp are contiguous whatever the src layout is; the work is a single pass
// over both tensors, bound by HBM.  When both tensors are dense in the same
// dim order (the quantization of weights and activations before a matmul) a
// thread takes four neighbours with 16-byte loads and one packed store.
#include <cstdio>

#include "device_math.cuh"
#include "launch.h"
#include "objects.hpp"

using namespace qmm;

namespace {

constexpr int RMAX = 6; // tensor dims the kernel handles

struct RQuant {
    const void *ptr;
    int dt;
    int64_t grp[RMAX]; // group size per dim (1 except, possibly, the last two)
    int64_t str[RMAX]; // stride of the parameter tensor per dim, 0 where the mask bit is clear
};

struct ReorderArgs {
    int ndims;
    int order[RMAX]; // dims from the fastest varying thread index to the slowest
    int64_t dims[RMAX], sstr[RMAX], dstr[RMAX];
    int64_t work; // elements, or element pairs for 4-bit targets
    int tx; // dense kernel: column chunks per CTA row
    const void *src;
    void *dst;
    int src_dt, dst_dt;
    RQuant src_scale, dst_scale, src_zp;
    const int *dst_zp;
    float beta;
};

__device__ __forceinline__ bool dt_is_int(int dt) { return dt == DT_S32 || dt == DT_S8 || dt == DT_U8; }

__device__ __forceinline__ unsigned quantize_nibble(float v, bool sgn) {
    v = fminf(fmaxf(v, sgn ? -8.f : 0.f), sgn ? 7.f : 15.f);
    return (unsigned)__float2int_rn(v) & 0xFu;
}

// IDX: the type the linear index is decomposed in (32-bit division where the tensor allows it)
template <typename IDX>
__global__ void __launch_bounds__(256) reorder_kernel(const __grid_constant__ ReorderArgs a) {
    const bool dst4 = a.dst_dt == DT_S4 || a.dst_dt == DT_U4;
    const bool src4 = a.src_dt == DT_S4 || a.src_dt == DT_U4;
    const int dst_zp = a.dst_zp ? __ldg(a.dst_zp) : 0;
    for (int64_t l = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; l < a.work;
            l += (int64_t)gridDim.x * blockDim.x) {
        IDX rem = (IDX)l;
        int64_t i_off = 0, o_off = 0, q_ss = 0, q_ds = 0, q_sz = 0; // tensor and parameter offsets
#pragma unroll
        for (int k = 0; k < RMAX; ++k) {
            if (k >= a.ndims) break;
            const int d = a.order[k];
            IDX extent = (IDX)a.dims[d];
            if (dst4 && k == 0) extent >>= 1; // a thread owns elements (2j, 2j+1) of the innermost dim
            IDX i = rem % extent;
            rem /= extent;
            if (dst4 && k == 0) i *= 2;
            i_off += (int64_t)i * a.sstr[d];
            o_off += (int64_t)i * a.dstr[d];
            // groups exist on the last two dims only; elsewhere the divisor is 1
            q_ss += (int64_t)(a.src_scale.grp[d] == 1 ? i : i / (IDX)a.src_scale.grp[d]) * a.src_scale.str[d];
            q_ds += (int64_t)i * a.dst_scale.str[d];
            q_sz += (int64_t)(a.src_zp.grp[d] == 1 ? i : i / (IDX)a.src_zp.grp[d]) * a.src_zp.str[d];
        }
        if (dst4) {
            const int64_t s1 = a.sstr[a.order[0]];
            const float v0 = ((const float *)a.src)[i_off], v1 = ((const float *)a.src)[i_off + s1];
            const bool sgn = a.dst_dt == DT_S4;
            ((unsigned char *)a.dst)[o_off >> 1] = (unsigned char)(quantize_nibble(v0, sgn) | (quantize_nibble(v1, sgn) << 4));
            continue;
        }
        float src_scale = 1.f, dst_scale = 1.f;
        if (a.src_scale.ptr) src_scale = load_float(a.src_scale.dt, a.src_scale.ptr, q_ss);
        if (a.dst_scale.ptr) dst_scale = __ldg((const float *)a.dst_scale.ptr + q_ds);
        int zp = 0;
        if (a.src_zp.ptr) zp = (int)load_float(a.src_zp.dt, a.src_zp.ptr, q_sz);
        // integer sources subtract in integer arithmetic, the others (and 4-bit ones, which the
        // reference widens to the floating-point dst type first) in float
        float diff;
        if (dt_is_int(a.src_dt)) diff = (float)(load_int(a.src_dt, a.src, i_off) - zp);
        else diff = __fsub_rn(load_float(a.src_dt, a.src, i_off), (float)zp);
        float d = __fmul_rn(src_scale, diff);
        if (!src4) {
            if (a.beta != 0.f) d = __fadd_rn(d, __fmul_rn(a.beta, load_float(a.dst_dt, a.dst, o_off)));
            d = __fdiv_rn(d, dst_scale);
            // like the reference: its JIT reorders add a zero-point only when one is set (-0 stays
            // -0), its scalar one, which serves reorders with a sum, always does
            if (a.dst_zp || a.beta != 0.f) d = __fadd_rn(d, (float)dst_zp);
        }
        store_float(a.dst_dt, d, a.dst, o_off);
    }
}

// ---- both tensors dense in the same dim order: four neighbours per thread, 16-byte accesses
// elements off .. off+3 (off a multiple of 4) as floats, and as ints for integer types
__device__ __forceinline__ void load4(int dt, const void *p, int64_t off, float (&f)[4], int (&iv)[4]) {
    if (dt == DT_F32) {
        const float4 v = __ldg((const float4 *)p + (off >> 2));
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    } else if (dt == DT_S32) {
        const int4 v = __ldg((const int4 *)p + (off >> 2));
        iv[0] = v.x; iv[1] = v.y; iv[2] = v.z; iv[3] = v.w;
    } else if (dt == DT_BF16 || dt == DT_F16) {
        const uint2 v = __ldg((const uint2 *)p + (off >> 2));
        const unsigned short h[4] = {(unsigned short)(v.x & 0xffffu), (unsigned short)(v.x >> 16),
                (unsigned short)(v.y & 0xffffu), (unsigned short)(v.y >> 16)};
#pragma unroll
        for (int e = 0; e < 4; ++e) f[e] = dt == DT_BF16 ? bf16_bits_to_f32(h[e]) : __half2float(__ushort_as_half(h[e]));
    } else {
        const unsigned v = __ldg((const unsigned *)p + (off >> 2));
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const unsigned b = (v >> (8 * e)) & 0xffu;
            if (dt == DT_S8) iv[e] = (int)(signed char)b;
            else if (dt == DT_U8) iv[e] = (int)b;
            else f[e] = dt == DT_F8_E4M3 ? e4m3_to_f32((unsigned char)b) : e5m2_to_f32((unsigned char)b);
        }
    }
}

__device__ __forceinline__ void store4(int dt, const float (&d)[4], void *p, int64_t off) {
    if (dt == DT_F32) {
        ((float4 *)p)[off >> 2] = make_float4(d[0], d[1], d[2], d[3]);
    } else if (dt == DT_S32) {
        int q[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float v = fminf(fmaxf(d[e], -2147483648.f), 2147483520.f);
            q[e] = (v != v) ? (int)0x80000000 : __float2int_rn(v);
        }
        ((int4 *)p)[off >> 2] = make_int4(q[0], q[1], q[2], q[3]);
    } else if (dt == DT_BF16 || dt == DT_F16) {
        unsigned h[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            h[e] = dt == DT_BF16 ? (unsigned)f32_to_bf16_bits(d[e]) : (unsigned)__half_as_ushort(__float2half_rn(d[e]));
        ((uint2 *)p)[off >> 2] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
    } else {
        unsigned w = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            unsigned b;
            if (dt == DT_F8_E4M3) b = f32_to_e4m3_bits(d[e]);
            else if (dt == DT_F8_E5M2) b = f32_to_e5m2_bits(d[e]);
            else {
                const float v = dt == DT_S8 ? fminf(fmaxf(d[e], -128.f), 127.f) : fminf(fmaxf(d[e], 0.f), 255.f);
                b = (unsigned)__float2int_rn(v) & 0xffu;
            }
            w |= b << (8 * e);
        }
        ((unsigned *)p)[off >> 2] = w;
    }
}

__global__ void __launch_bounds__(256) reorder_dense4_kernel(const __grid_constant__ ReorderArgs a) {
    // A thread keeps its four columns (indices i0 .. i0+3 of the contiguous dim d0) and walks over
    // the rows (all other dims collapsed): parameters that vary only along d0 -- per-column scales,
    // the usual case -- are loaded once, and no index is decomposed inside the loop.
    const int dst_zp = a.dst_zp ? __ldg(a.dst_zp) : 0;
    const int d0 = a.order[0];
    const int64_t cols = a.dims[d0], rows = a.work * 4 / cols;
    // a CTA is tx column chunks wide and 256 / tx rows high (tx a power of two, narrow tensors get tall CTAs)
    const int tx = a.tx, ty = 256 / tx;
    const int64_t i0 = ((int64_t)blockIdx.x * tx + threadIdx.x % tx) * 4;
    if (i0 >= cols) return;
    int64_t c_ss[4], c_ds[4], c_sz[4]; // parameter offsets contributed by the column
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        c_ss[e] = ((i0 + e) / a.src_scale.grp[d0]) * a.src_scale.str[d0];
        c_ds[e] = ((i0 + e) / a.dst_scale.grp[d0]) * a.dst_scale.str[d0];
        c_sz[e] = ((i0 + e) / a.src_zp.grp[d0]) * a.src_zp.str[d0];
    }
    bool outer = false; // does a parameter vary along another dim than d0?
    for (int k = 1; k < a.ndims; ++k) {
        const int d = a.order[k];
        outer |= a.src_scale.str[d] != 0 || a.dst_scale.str[d] != 0 || a.src_zp.str[d] != 0;
    }
    float ss[4], ds[4];
    int zps[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        ss[e] = (a.src_scale.ptr && !outer) ? load_float(a.src_scale.dt, a.src_scale.ptr, c_ss[e]) : 1.f;
        ds[e] = (a.dst_scale.ptr && !outer) ? __ldg((const float *)a.dst_scale.ptr + c_ds[e]) : 1.f;
        zps[e] = (a.src_zp.ptr && !outer) ? (int)load_float(a.src_zp.dt, a.src_zp.ptr, c_sz[e]) : 0;
    }
#pragma unroll 2
    for (int64_t r = (int64_t)blockIdx.y * ty + threadIdx.x / tx; r < rows; r += (int64_t)gridDim.y * ty) {
        const int64_t off = r * cols + i0;
        int64_t o_ss = 0, o_ds = 0, o_sz = 0; // parameter offsets contributed by the row
        if (outer) {
            int64_t rem = r;
#pragma unroll
            for (int k = 1; k < RMAX; ++k) {
                if (k >= a.ndims) break;
                const int d = a.order[k];
                const int64_t i = rem % a.dims[d];
                rem /= a.dims[d];
                o_ss += (i / a.src_scale.grp[d]) * a.src_scale.str[d];
                o_ds += (i / a.dst_scale.grp[d]) * a.dst_scale.str[d];
                o_sz += (i / a.src_zp.grp[d]) * a.src_zp.str[d];
            }
        }
        float f[4], old[4], out[4];
        int iv[4], unused[4];
        load4(a.src_dt, a.src, off, f, iv);
        if (a.beta != 0.f) {
            load4(a.dst_dt, a.dst, off, old, unused);
            if (dt_is_int(a.dst_dt))
#pragma unroll
                for (int e = 0; e < 4; ++e) old[e] = (float)unused[e];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float src_scale = ss[e], dst_scale = ds[e];
            int zp = zps[e];
            if (outer) {
                if (a.src_scale.ptr) src_scale = load_float(a.src_scale.dt, a.src_scale.ptr, o_ss + c_ss[e]);
                if (a.dst_scale.ptr) dst_scale = __ldg((const float *)a.dst_scale.ptr + o_ds + c_ds[e]);
                if (a.src_zp.ptr) zp = (int)load_float(a.src_zp.dt, a.src_zp.ptr, o_sz + c_sz[e]);
            }
            const float diff = dt_is_int(a.src_dt) ? (float)(iv[e] - zp) : __fsub_rn(f[e], (float)zp);
            float d = __fmul_rn(src_scale, diff);
            if (a.beta != 0.f) d = __fadd_rn(d, __fmul_rn(a.beta, old[e]));
            if (a.dst_scale.ptr) d = __fdiv_rn(d, dst_scale); // x / 1 = x: skipped without dst scales
            out[e] = (a.dst_zp || a.beta != 0.f) ? __fadd_rn(d, (float)dst_zp) : d;
        }
        store4(a.dst_dt, out, a.dst, off);
    }
}

// The same walk with the data types known at compile time, for reorders whose parameters vary only
// along the contiguous dim and that have no sum: four rows in flight per thread, conversions
// without run-time type switches.  This is the quantization / dequantization of a weight or
// activation matrix with per-tensor or per-column parameters.
template <int SDT, int DDT>
__global__ void __launch_bounds__(256) reorder_cols4_kernel(const __grid_constant__ ReorderArgs a) {
    const int dst_zp = a.dst_zp ? __ldg(a.dst_zp) : 0;
    const int d0 = a.order[0];
    const int64_t cols = a.dims[d0], rows = a.work * 4 / cols;
    const int tx = a.tx, ty = 256 / tx;
    const int64_t i0 = ((int64_t)blockIdx.x * tx + threadIdx.x % tx) * 4;
    if (i0 >= cols) return;
    float ss[4], ds[4];
    int zps[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        ss[e] = a.src_scale.ptr ? load_float(a.src_scale.dt, a.src_scale.ptr,
                                          ((i0 + e) / a.src_scale.grp[d0]) * a.src_scale.str[d0])
                                : 1.f;
        ds[e] = a.dst_scale.ptr ? __ldg((const float *)a.dst_scale.ptr + ((i0 + e) / a.dst_scale.grp[d0]) * a.dst_scale.str[d0])
                                : 1.f;
        zps[e] = a.src_zp.ptr ? (int)load_float(a.src_zp.dt, a.src_zp.ptr, ((i0 + e) / a.src_zp.grp[d0]) * a.src_zp.str[d0])
                              : 0;
    }
    const bool has_ds = a.dst_scale.ptr != nullptr, has_zp = a.dst_zp != nullptr;
    auto convert = [&](const float (&f)[4], const int (&iv)[4], int64_t off) {
        float out[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float diff = dt_is_int(SDT) ? (float)(iv[e] - zps[e]) : __fsub_rn(f[e], (float)zps[e]);
            float d = __fmul_rn(ss[e], diff);
            if (has_ds) d = __fdiv_rn(d, ds[e]);
            out[e] = has_zp ? __fadd_rn(d, (float)dst_zp) : d;
        }
        store4(DDT, out, a.dst, off);
    };
    const int64_t step = (int64_t)gridDim.y * ty;
    int64_t r = (int64_t)blockIdx.y * ty + threadIdx.x / tx;
    for (; r + 3 * step < rows; r += 4 * step) {
        float f[4][4];
        int iv[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) load4(SDT, a.src, (r + u * step) * cols + i0, f[u], iv[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u) convert(f[u], iv[u], (r + u * step) * cols + i0);
    }
    for (; r < rows; r += step) {
        float f[4];
        int iv[4];
        load4(SDT, a.src, r * cols + i0, f, iv);
        convert(f, iv, r * cols + i0);
    }
}

// Layout-changing reorder of a matrix (or a batch of them): the src is contiguous along dim dr,
// the dst along dim dc.  A CTA converts a 32 x 32 tile, reading along dr and, after a trip
// through shared memory, writing along dc, so both sides move whole sectors.  No sum.
__global__ void __launch_bounds__(256)
reorder_transpose_kernel(const __grid_constant__ ReorderArgs a, int dr, int dc, int db) {
    __shared__ float tile[32][33];
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    const int64_t r0 = (int64_t)blockIdx.x * 32, c0 = (int64_t)blockIdx.y * 32, b = blockIdx.z;
    const int dst_zp = a.dst_zp ? __ldg(a.dst_zp) : 0;
    int64_t sb = 0, ob = 0, q_ss = 0, q_ds = 0, q_sz = 0; // the batch index's share of every offset
    if (db >= 0) {
        sb = b * a.sstr[db];
        ob = b * a.dstr[db];
        q_ss = b * a.src_scale.str[db];
        q_ds = b * a.dst_scale.str[db];
        q_sz = b * a.src_zp.str[db];
    }
    const int64_t r = r0 + tx;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int64_t c = c0 + ty + 8 * j;
        if (r >= a.dims[dr] || c >= a.dims[dc]) continue;
        const int64_t i_off = sb + r * a.sstr[dr] + c * a.sstr[dc];
        float src_scale = 1.f, dst_scale = 1.f;
        int zp = 0;
        if (a.src_scale.ptr)
            src_scale = load_float(a.src_scale.dt, a.src_scale.ptr,
                    q_ss + (r / a.src_scale.grp[dr]) * a.src_scale.str[dr] + (c / a.src_scale.grp[dc]) * a.src_scale.str[dc]);
        if (a.dst_scale.ptr) dst_scale = __ldg((const float *)a.dst_scale.ptr + q_ds + r * a.dst_scale.str[dr] + c * a.dst_scale.str[dc]);
        if (a.src_zp.ptr)
            zp = (int)load_float(a.src_zp.dt, a.src_zp.ptr,
                    q_sz + (r / a.src_zp.grp[dr]) * a.src_zp.str[dr] + (c / a.src_zp.grp[dc]) * a.src_zp.str[dc]);
        const float diff = dt_is_int(a.src_dt) ? (float)(load_int(a.src_dt, a.src, i_off) - zp)
                                                : __fsub_rn(load_float(a.src_dt, a.src, i_off), (float)zp);
        float d = __fmul_rn(src_scale, diff);
        if (a.dst_scale.ptr) d = __fdiv_rn(d, dst_scale); // x / 1 = x
        if (a.dst_zp) d = __fadd_rn(d, (float)dst_zp);
        tile[ty + 8 * j][tx] = d;
    }
    __syncthreads();
    const int64_t c = c0 + tx;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int64_t rr = r0 + ty + 8 * j;
        if (rr >= a.dims[dr] || c >= a.dims[dc]) continue;
        store_float(a.dst_dt, tile[tx][ty + 8 * j], a.dst, ob + rr * a.dstr[dr] + c * a.dstr[dc]);
    }
}

typedef void (*reorder_kernel_fn)(const ReorderArgs);

template <int SDT>
reorder_kernel_fn cols4_for_dst(int ddt) {
    switch (ddt) {
        case DT_F32: return reorder_cols4_kernel<SDT, DT_F32>;
        case DT_BF16: return reorder_cols4_kernel<SDT, DT_BF16>;
        case DT_F16: return reorder_cols4_kernel<SDT, DT_F16>;
        case DT_S8: return reorder_cols4_kernel<SDT, DT_S8>;
        case DT_U8: return reorder_cols4_kernel<SDT, DT_U8>;
        case DT_F8_E4M3: return reorder_cols4_kernel<SDT, DT_F8_E4M3>;
        case DT_F8_E5M2: return reorder_cols4_kernel<SDT, DT_F8_E5M2>;
        default: return nullptr;
    }
}
reorder_kernel_fn cols4_kernel(int sdt, int ddt) {
    switch (sdt) {
        case DT_F32: return cols4_for_dst<DT_F32>(ddt);
        case DT_BF16: return cols4_for_dst<DT_BF16>(ddt);
        case DT_F16: return cols4_for_dst<DT_F16>(ddt);
        case DT_S8: return cols4_for_dst<DT_S8>(ddt);
        case DT_U8: return cols4_for_dst<DT_U8>(ddt);
        default: return nullptr;
    }
}

bool one_of_dt(dnnl_data_type_t v, std::initializer_list<dnnl_data_type_t> l) {
    for (auto x : l)
        if (v == x) return true;
    return false;
}

bool is_integral(dnnl_data_type_t dt) { return one_of_dt(dt, {dnnl_s32, dnnl_s8, dnnl_u8, dnnl_s4, dnnl_u4}); }

// memory descriptor of a scale / zero-point buffer: the tensor's dims under the mask, the
// last two divided by the groups, dense row-major (quant_entry_t::get_md,
// src/common/primitive_attr_quant.hpp:116-140)
dnnl_memory_desc quant_md(const quant_entry_t &e, const dnnl_memory_desc &t) {
    dnnl_memory_desc md;
    md.ndims = t.ndims;
    md.data_type = e.dt;
    md.format_kind = dnnl_blocked;
    for (int d = 0; d < t.ndims; ++d) {
        dnnl_dim_t g = 1;
        if (e.group_ndims && t.ndims >= 2 && d == t.ndims - 1) g = e.groups[1];
        if (e.group_ndims && t.ndims >= 2 && d == t.ndims - 2) g = e.groups[0];
        md.dims[d] = ((e.mask >> d) & 1) ? t.dims[d] / g : 1;
    }
    dnnl_dim_t acc = 1;
    for (int d = t.ndims - 1; d >= 0; --d) {
        md.strides[d] = acc;
        acc *= md.dims[d];
    }
    return md;
}

dnnl_status_t bind_rquant(RQuant &q, const quant_entry_t &e, const dnnl_memory_desc &t, dnnl_memory_t mem) {
    q = RQuant {};
    for (int d = 0; d < RMAX; ++d) q.grp[d] = 1;
    if (!e.set) return dnnl_success;
    if (!mem || mem->is_host_scalar || !mem->handles[0]) return dnnl_invalid_arguments;
    const dnnl_memory_desc md = quant_md(e, t);
    q.ptr = mem->handles[0];
    q.dt = e.dt;
    for (int d = 0; d < t.ndims; ++d) {
        if (e.group_ndims && t.ndims >= 2 && d == t.ndims - 1) q.grp[d] = e.groups[1];
        if (e.group_ndims && t.ndims >= 2 && d == t.ndims - 2) q.grp[d] = e.groups[0];
        q.str[d] = ((e.mask >> d) & 1) ? md.strides[d] : 0;
    }
    return dnnl_success;
}

bool plain(const dnnl_memory_desc &md) { return md.format_kind == dnnl_blocked; }

} // namespace

extern "C" dnnl_status_t dnnl_reorder_primitive_desc_create(dnnl_primitive_desc_t *reorder_primitive_desc,
        const_dnnl_memory_desc_t src_desc, dnnl_engine_t src_engine, const_dnnl_memory_desc_t dst_desc,
        dnnl_engine_t dst_engine, const_dnnl_primitive_attr_t attr) {
    if (!reorder_primitive_desc || !src_desc || !src_engine || !dst_desc || !dst_engine) return dnnl_invalid_arguments;
    // one engine kind here, so a cross-engine reorder can only be between two devices: not provided
    if (src_engine != dst_engine && src_engine->device != dst_engine->device) return dnnl_unimplemented;
    if (!plain(*src_desc) || !plain(*dst_desc)) {
        // format_any is an error, sparse / grouped encodings have no reorder on a GPU engine
        const bool any = src_desc->format_kind == dnnl_format_kind_any || dst_desc->format_kind == dnnl_format_kind_any;
        return any ? dnnl_invalid_arguments : dnnl_unimplemented;
    }
    const int nd = src_desc->ndims;
    if (nd != dst_desc->ndims || nd < 1) return dnnl_invalid_arguments;
    for (int d = 0; d < nd; ++d)
        if (src_desc->dims[d] != dst_desc->dims[d]) return dnnl_invalid_arguments;

    auto pd = new dnnl_primitive_desc;
    pd->kind = dnnl_reorder;
    pd->engine = src_engine;
    pd->src = *src_desc;
    pd->dst = *dst_desc;
    if (attr) pd->attr = *attr;
    const auto &at = pd->attr;
    const dnnl_data_type_t si = src_desc->data_type, di = dst_desc->data_type;

    auto fail = [&](dnnl_status_t st) {
        delete pd;
        return st;
    };
    // src/common/reorder.cpp:95-147
    if (!is_integral(si) && at.zp(DNNL_ARG_SRC).set) return fail(dnnl_invalid_arguments);
    if (!is_integral(di) && at.zp(DNNL_ARG_DST).set) return fail(dnnl_invalid_arguments);
    for (const auto &kv : at.scales)
        if (kv.first != DNNL_ARG_SRC && kv.first != DNNL_ARG_DST) return fail(dnnl_unimplemented);
    const quant_entry_t &ss = at.scale(DNNL_ARG_SRC), &ds = at.scale(DNNL_ARG_DST);
    const quant_entry_t &sz = at.zp(DNNL_ARG_SRC), &dz = at.zp(DNNL_ARG_DST);
    const bool src4 = si == dnnl_s4 || si == dnnl_u4, dst4 = di == dnnl_s4 || di == dnnl_u4;
    if (src4 && ss.set && ss.mask == 0) return fail(dnnl_invalid_arguments);
    for (const quant_entry_t *q : {&ss, &sz}) {
        if (!q->set || !q->group_ndims) continue;
        if (nd < 2) return fail(dnnl_invalid_arguments);
        if ((q->groups[0] > 1 && src_desc->dims[nd - 2] % q->groups[0])
                || (q->groups[1] > 1 && src_desc->dims[nd - 1] % q->groups[1]))
            return fail(dnnl_invalid_arguments);
        if (!((q->mask >> (nd - 1)) & 1) || !((q->mask >> (nd - 2)) & 1)) return fail(dnnl_invalid_arguments);
    }
    if (ds.set && ds.group_ndims) return fail(dnnl_invalid_arguments);

    // what the kernel covers (the reference's simple_reorder reference implementations)
    const std::initializer_list<dnnl_data_type_t> in_types
            = {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_s32, dnnl_s8, dnnl_u8, dnnl_f8_e4m3, dnnl_f8_e5m2, dnnl_s4, dnnl_u4};
    const std::initializer_list<dnnl_data_type_t> out_types
            = {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_s32, dnnl_s8, dnnl_u8, dnnl_f8_e4m3, dnnl_f8_e5m2, dnnl_s4, dnnl_u4};
    if (nd > RMAX || !one_of_dt(si, in_types) || !one_of_dt(di, out_types)) return fail(dnnl_unimplemented);
    if (src_desc->offset0 || dst_desc->offset0) return fail(dnnl_unimplemented);
    for (const quant_entry_t *q : {&ss, &ds, &sz, &dz})
        if (q->set && q->on_host) return fail(dnnl_unimplemented);
    if (at.fpmath != dnnl_fpmath_mode_strict || at.apply_to_int || !at.reductions.empty() || !at.rounding.empty())
        return fail(dnnl_unimplemented);
    if (ss.set && !one_of_dt(ss.dt, {dnnl_f32, dnnl_bf16, dnnl_f16})) return fail(dnnl_unimplemented);
    if (ds.set && ds.dt != dnnl_f32) return fail(dnnl_unimplemented);
    if (sz.set && !is_integral(sz.dt)) return fail(dnnl_unimplemented);
    if (dz.set && (dz.mask != 0 || dz.dt != dnnl_s32 || dz.group_ndims)) return fail(dnnl_unimplemented);
    const auto &po = at.post_ops.entries;
    if (po.size() > 1 || (po.size() == 1 && (po[0].kind != dnnl_sum || po[0].zero_point != 0)))
        return fail(dnnl_unimplemented);
    const bool has_sum = po.size() == 1;
    if (has_sum && po[0].sum_dt != dnnl_data_type_undef && po[0].sum_dt != di) return fail(dnnl_unimplemented);
    if (dst4) {
        // plain conversion of f32 into a buffer whose innermost dim is dense and even, so that two
        // neighbours share a byte no other thread touches
        if (si != dnnl_f32 || ss.set || ds.set || sz.set || dz.set || has_sum) return fail(dnnl_unimplemented);
        if (dst_desc->strides[nd - 1] != 1 || dst_desc->dims[nd - 1] % 2) return fail(dnnl_unimplemented);
        for (int d = 0; d < nd - 1; ++d)
            if (dst_desc->strides[d] % 2) return fail(dnnl_unimplemented);
    }
    if (src4) {
        if (!one_of_dt(di, {dnnl_f32, dnnl_bf16, dnnl_f16}) || ds.set || dz.set || has_sum) return fail(dnnl_unimplemented);
    }

    pd->impl = IMPL_REF;
    pd->impl_name = "cuda:ref:reorder";
    if (ss.set) pd->quant_mds[DNNL_ARG_ATTR_SCALES | DNNL_ARG_SRC] = quant_md(ss, pd->src);
    if (ds.set) pd->quant_mds[DNNL_ARG_ATTR_SCALES | DNNL_ARG_DST] = quant_md(ds, pd->src);
    if (sz.set) pd->quant_mds[DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_SRC] = quant_md(sz, pd->src);
    if (dz.set) pd->quant_mds[DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_DST] = quant_md(dz, pd->src);
    *reorder_primitive_desc = pd;
    return dnnl_success;
}

dnnl_status_t qmm::execute_reorder(const dnnl_primitive_desc &pd, dnnl_stream_t stream, int nargs,
        const dnnl_exec_arg_t *args) {
    auto find = [&](int key) -> dnnl_memory_t {
        for (int i = 0; i < nargs; ++i)
            if (args[i].arg == key) return args[i].memory;
        return nullptr;
    };
    dnnl_memory_t src = find(DNNL_ARG_FROM), dst = find(DNNL_ARG_TO);
    if (!src || !dst) return dnnl_invalid_arguments;
    const auto &at = pd.attr;
    ReorderArgs a {};
    a.ndims = pd.src.ndims;
    int64_t nelems = 1;
    for (int d = 0; d < a.ndims; ++d) {
        a.dims[d] = pd.src.dims[d];
        a.sstr[d] = pd.src.strides[d];
        a.dstr[d] = pd.dst.strides[d];
        a.order[d] = d;
        nelems *= a.dims[d];
    }
    // dims by increasing dst stride (insertion sort; ties keep the later dim first, as row-major does)
    for (int i = 0; i < a.ndims; ++i) a.order[i] = a.ndims - 1 - i;
    for (int i = 1; i < a.ndims; ++i)
        for (int j = i; j > 0 && a.dstr[a.order[j]] < a.dstr[a.order[j - 1]]; --j) {
            const int t = a.order[j];
            a.order[j] = a.order[j - 1];
            a.order[j - 1] = t;
        }
    a.src = src->handles[0];
    a.dst = dst->handles[0];
    a.src_dt = pd.src.data_type;
    a.dst_dt = pd.dst.data_type;
    const bool dst4 = a.dst_dt == DT_S4 || a.dst_dt == DT_U4;
    a.work = dst4 ? nelems / 2 : nelems;
    if (nelems == 0) return dnnl_success;
    if (!a.src || !a.dst) return dnnl_invalid_arguments;
    dnnl_status_t st;
    st = bind_rquant(a.src_scale, at.scale(DNNL_ARG_SRC), pd.src, find(DNNL_ARG_ATTR_SCALES | DNNL_ARG_SRC));
    if (st != dnnl_success) return st;
    st = bind_rquant(a.dst_scale, at.scale(DNNL_ARG_DST), pd.src, find(DNNL_ARG_ATTR_SCALES | DNNL_ARG_DST));
    if (st != dnnl_success) return st;
    st = bind_rquant(a.src_zp, at.zp(DNNL_ARG_SRC), pd.src, find(DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_SRC));
    if (st != dnnl_success) return st;
    if (at.zp(DNNL_ARG_DST).set) {
        dnnl_memory_t m = find(DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_DST);
        if (!m || m->is_host_scalar || !m->handles[0]) return dnnl_invalid_arguments;
        a.dst_zp = (const int *)m->handles[0];
    }
    if (!at.post_ops.entries.empty()) a.beta = at.post_ops.entries[0].scale;
    if (pd.engine->device < 0) {
        set_last_error("a device-less engine cannot execute primitives");
        return dnnl_runtime_error;
    }
    cudaSetDevice(pd.engine->device);
    // Both tensors dense in the same dim order, the contiguous dim a multiple of four, buffers
    // aligned for four elements: the kernel with 16-byte accesses.
    const bool src4 = a.src_dt == DT_S4 || a.src_dt == DT_U4;
    bool dense4 = !src4 && !dst4 && a.dims[a.order[0]] % 4 == 0;
    int64_t expect = 1;
    for (int k = 0; k < a.ndims && dense4; ++k) {
        const int d = a.order[k];
        if (a.dims[d] != 1 && (a.dstr[d] != expect || a.sstr[d] != expect)) dense4 = false;
        expect *= a.dims[d];
    }
    auto width = [](int dt) { return (dt == DT_F32 || dt == DT_S32) ? 4 : (dt == DT_BF16 || dt == DT_F16) ? 2 : 1; };
    if ((uintptr_t)a.src % (4 * width(a.src_dt)) || (uintptr_t)a.dst % (4 * width(a.dst_dt))) dense4 = false;
    if (dense4) a.work = nelems / 4;
    const int sms = pd.engine->sm_count > 0 ? pd.engine->sm_count : 148;
    int64_t blocks = (a.work + 255) / 256;
    if (blocks > (int64_t)sms * 32) blocks = (int64_t)sms * 32; // grid-stride beyond 32 CTAs per SM
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    const bool verbose = verbose_level() >= 1;
    if (verbose) {
        cudaEventCreate(&ev0); cudaEventCreate(&ev1);
        cudaEventRecord(ev0, stream->stream);
    }
    profiling_begin(stream);
    if (dense4) {
        // x: the columns in chunks of four; y: as many row walkers as fill the SMs eight CTAs deep
        const int64_t cols = a.dims[a.order[0]], rows = nelems / cols;
        a.tx = 256;
        while (a.tx > 1 && a.tx / 2 >= cols / 4) a.tx /= 2;
        const int ty = 256 / a.tx;
        const int64_t gx = (cols / 4 + a.tx - 1) / a.tx;
        int64_t gy = ((int64_t)sms * 8 + gx - 1) / gx;
        if (gy > (rows + ty - 1) / ty) gy = (rows + ty - 1) / ty;
        if (gy > 65535) gy = 65535;
        if (gx > 0x7fffffff) return dnnl_unimplemented;
        bool outer = false; // a parameter that varies along another dim than the contiguous one
        for (int k = 1; k < a.ndims; ++k) {
            const int d = a.order[k];
            outer |= a.src_scale.str[d] != 0 || a.dst_scale.str[d] != 0 || a.src_zp.str[d] != 0;
        }
        reorder_kernel_fn typed = (!outer && a.beta == 0.f) ? cols4_kernel(a.src_dt, a.dst_dt) : nullptr;
        if (typed) typed<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, stream->stream>>>(a);
        else reorder_dense4_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, stream->stream>>>(a);
    } else {
        // a matrix (or a batch of matrices) whose contiguous dim changes: the tiled kernel
        int dr = -1, dc = -1;
        if (!src4 && !dst4 && a.beta == 0.f && (a.ndims == 2 || a.ndims == 3)) {
            for (int d = a.ndims - 2; d < a.ndims; ++d) {
                if (a.sstr[d] == 1 && a.dims[d] > 1) dr = d;
                if (a.dstr[d] == 1 && a.dims[d] > 1) dc = d;
            }
        }
        const int64_t gy = dc >= 0 ? (a.dims[dc] + 31) / 32 : 0, gz = a.ndims == 3 ? a.dims[0] : 1;
        if (dr >= 0 && dc >= 0 && dr != dc && gy <= 65535 && gz <= 65535) {
            const dim3 grid((unsigned)((a.dims[dr] + 31) / 32), (unsigned)gy, (unsigned)gz);
            reorder_transpose_kernel<<<grid, 256, 0, stream->stream>>>(a, dr, dc, a.ndims == 3 ? 0 : -1);
        } else if (nelems < ((int64_t)1 << 31)) {
            reorder_kernel<unsigned><<<(unsigned)blocks, 256, 0, stream->stream>>>(a);
        } else {
            reorder_kernel<int64_t><<<(unsigned)blocks, 256, 0, stream->stream>>>(a);
        }
    }
    count_launch();
    const bool ok = cudaGetLastError() == cudaSuccess;
    profiling_end(stream);
    if (verbose) {
        cudaEventRecord(ev1, stream->stream);
        cudaEventSynchronize(ev1);
        float ms = 0;
        cudaEventElapsedTime(&ms, ev0, ev1);
        cudaEventDestroy(ev0); cudaEventDestroy(ev1);
        verbose_line("exec", pd, ms);
    }
    if (!ok) {
        set_last_error("kernel launch: reorder");
        return dnnl_runtime_error;
    }
    return dnnl_success;
}
