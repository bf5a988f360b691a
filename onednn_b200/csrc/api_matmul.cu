// C API: matmul primitive descriptor (validation + implementation list),
// primitive creation and execution.  The checks restate oneDNN's
// src/common/matmul.cpp (matmul_desc_init :630-744, matmul_attr_check
// :261-624, grouped variants :53-258), matmul_pd.hpp and the acceptance
// conditions of its reference implementations (ref_matmul.hpp:44-123,
// ref_matmul_int8.hpp:44-92, ref_grouped_gemm.hpp:67-246).
#include <chrono>
#include <cstdio>
#include <cstring>

#include "launch.h"
#include "objects.hpp"

using namespace qmm;

namespace {

bool one_of(int v, std::initializer_list<int> l) {
    for (int x : l)
        if (v == x) return true;
    return false;
}
bool is_int8(dnnl_data_type_t dt) { return dt == dnnl_s8 || dt == dnnl_u8; }
bool is_int_wei(dnnl_data_type_t dt) { return one_of(dt, {dnnl_s8, dnnl_u8, dnnl_s4, dnnl_u4}); }
bool is_fp8(dnnl_data_type_t dt) { return dt == dnnl_f8_e4m3 || dt == dnnl_f8_e5m2; }

#define UNIMPL_IF(cond) do { if (cond) return dnnl_unimplemented; } while (0)
#define INVALID_IF(cond) do { if (cond) return dnnl_invalid_arguments; } while (0)

// row-major strides for a descriptor created with format_tag::any
void set_default_format(dnnl_memory_desc &md) {
    if (md.format_kind != dnnl_format_kind_any) return;
    md.format_kind = dnnl_blocked;
    dnnl_dim_t acc = 1;
    for (int i = md.ndims - 1; i >= 0; --i) {
        md.strides[i] = acc;
        acc *= md.dims[i] == 0 ? 1 : md.dims[i];
    }
}

// types::default_accum_data_type (src/common/type_helpers.hpp:515-548): the
// combination must have a defined accumulation type
bool dt_combo_ok(dnnl_data_type_t s, dnnl_data_type_t w, dnnl_data_type_t d) {
    if (s == dnnl_f32 && w == dnnl_f32) return true;
    if (is_int8(s) && is_int_wei(w)) return true;
    if (s == dnnl_f16 || w == dnnl_f16) return true;
    if (one_of(s, {dnnl_bf16, dnnl_f32}) && is_int_wei(w)) return true; // weights decompression
    for (dnnl_data_type_t t : {s, w, d})
        if (one_of(t, {dnnl_f4_e2m1, dnnl_f8_e5m2, dnnl_f8_e4m3, dnnl_bf16, dnnl_f16})) return true;
    return false; // no accumulation type: the descriptor is invalid, not merely without an implementation
}

dnnl_status_t dense_desc_check(const dnnl_memory_desc &src, const dnnl_memory_desc &wei,
        const dnnl_memory_desc *bias, const dnnl_memory_desc &dst) {
    const int ndims = dst.ndims;
    INVALID_IF(ndims < 2 || ndims > DNNL_MAX_NDIMS);
    INVALID_IF(src.ndims != ndims || wei.ndims != ndims);
    INVALID_IF(bias && bias->ndims != ndims);
    const int m = ndims - 2, n = ndims - 1;
    INVALID_IF(dst.dims[m] != src.dims[m]);
    INVALID_IF(dst.dims[n] != wei.dims[n]);
    INVALID_IF(src.dims[n] != wei.dims[m]);
    if (bias) {
        INVALID_IF(bias->dims[n] != 1 && bias->dims[n] != dst.dims[n]);
        INVALID_IF(bias->dims[m] != 1 && bias->dims[m] != dst.dims[m]);
    }
    for (int d = 0; d < ndims - 2; ++d) {
        const dnnl_dim_t s = src.dims[d], w = wei.dims[d], o = dst.dims[d];
        if (!(s == w && w == o)) INVALID_IF(s != 1 && w != 1);
        if (s == 1) INVALID_IF(o != w);
        if (w == 1) INVALID_IF(o != s);
        if (bias) INVALID_IF(bias->dims[d] != 1 && bias->dims[d] != o);
    }
    INVALID_IF(!dt_combo_ok(src.data_type, wei.data_type, dst.data_type));
    return dnnl_success;
}

dnnl_status_t dense_attr_check(const dnnl_primitive_desc &pd) {
    const auto &attr = pd.attr;
    if (attr.has_default_values()) return dnnl_success;
    const auto src_dt = pd.src.data_type, wei_dt = pd.wei.data_type, dst_dt = pd.dst.data_type;
    const bool src_int8 = is_int8(src_dt), src_fp8 = is_fp8(src_dt);
    const bool wei_int = is_int_wei(wei_dt), wei_fp8 = is_fp8(wei_dt);
    const int nd = pd.src.ndims;
    const dnnl_dim_t K = pd.K(), N = pd.N();
    const int qM = 1 << (nd - 2), qK = 1 << (nd - 1); // src masks; weights: K = qM, N = qK
    const int full = (1 << nd) - 1;

    UNIMPL_IF(!attr.rounding.empty());
    // zero-points only for int8/fp8 sources, or as part of weights decompression
    for (auto &kv : attr.zero_points) {
        if (kv.first == DNNL_ARG_WEIGHTS && (wei_int || wei_fp8)) continue;
        UNIMPL_IF(!(src_int8 || src_fp8));
        // non-weights zero-points: plain s32, no groups, unless the weights
        // are low precision
        if (!(wei_int || wei_fp8)) UNIMPL_IF(kv.second.dt != dnnl_s32 || kv.second.group_ndims != 0);
    }
    UNIMPL_IF(!attr.reductions.empty() && !src_int8);
    for (auto &kv : attr.scales)
        if (kv.second.group_ndims && kv.first != DNNL_ARG_DST) UNIMPL_IF(!(wei_int || wei_fp8));

    auto divisible = [](dnnl_dim_t a, dnnl_dim_t b) { return !(a > 1 && b > 1) || a % b == 0 || b % a == 0; };

    dnnl_dim_t ssg_k = 1, wsg_k = 1, wsg_n = 1;
    const auto &ss = attr.scale(DNNL_ARG_SRC);
    if (ss.set) {
        // per tensor, per row, or per K group (with or without the rows): what the reference's
        // matmuls take for src (attr_scales_ok with src_qmask_M, src/cpu/matmul/ref_matmul_int8.hpp:79-82)
        UNIMPL_IF(!(ss.mask == 0 || (ss.mask == qM && !ss.group_ndims)
                || (one_of(ss.mask, {qK, qM + qK}) && ss.group_ndims)));
        if (ss.group_ndims && (ss.mask & qK)) ssg_k = ss.group(1);
        UNIMPL_IF(ssg_k > 1 && ssg_k < K && ssg_k % 16 != 0);
    }
    const auto &ws = attr.scale(DNNL_ARG_WEIGHTS);
    if (ws.set) {
        if (ws.group_ndims) {
            if (ws.mask & qM) wsg_k = ws.group(0);
            if (ws.mask & qK) wsg_n = ws.group(1);
        }
        UNIMPL_IF(wsg_k > 1 && wsg_k < K && wsg_k % 16 != 0);
        UNIMPL_IF(wsg_n > 1 && wsg_n < N && wsg_n % 16 != 0);
    }
    const auto &ds = attr.scale(DNNL_ARG_DST);
    if (ds.set) {
        UNIMPL_IF(!one_of(ds.mask, {0, qK, qM, qM + qK, full}));
        UNIMPL_IF(ds.qmode != dnnl_quantization_mode_static_sazp); // dynamic (MX) dst scales
    }
    UNIMPL_IF(ssg_k > 1 && !((src_int8 || src_fp8) && divisible(ssg_k, wsg_k)));
    for (auto &kv : attr.scales) UNIMPL_IF(!one_of(kv.first, {DNNL_ARG_SRC, DNNL_ARG_WEIGHTS, DNNL_ARG_DST}));

    dnnl_dim_t szg_k = 1, wzg_k = 1, wzg_n = 1;
    const auto &sz = attr.zp(DNNL_ARG_SRC);
    if (sz.set) {
        UNIMPL_IF(!one_of(sz.mask, {0, qK, qM + qK, full}));
        if (sz.group_ndims && (sz.mask & qK)) szg_k = sz.group(1);
        UNIMPL_IF(szg_k > 1 && szg_k < K && szg_k % 32 != 0);
    }
    const auto &wz = attr.zp(DNNL_ARG_WEIGHTS);
    if (wz.set) {
        if (wz.group_ndims) {
            if (wz.mask & qM) wzg_k = wz.group(0);
            if (wz.mask & qK) wzg_n = wz.group(1);
        }
        UNIMPL_IF(wzg_n > 1 && !attr.apply_to_int);
        UNIMPL_IF(wzg_k > 1 && wzg_k < K && wzg_k % 16 != 0);
        UNIMPL_IF(wzg_n > 1 && wzg_n < N && wzg_n % 16 != 0);
        if (wz.dt == dnnl_s4 || wz.dt == dnnl_u4) {
            UNIMPL_IF((wz.mask & qM) && K % 2 != 0);
            UNIMPL_IF((wz.mask & qK) && N % 2 != 0);
        }
    }
    const auto &dz = attr.zp(DNNL_ARG_DST);
    if (dz.set) UNIMPL_IF(!(dz.mask == 0 || (nd == 2 && dz.mask == 2)));
    UNIMPL_IF(szg_k > 1 && !(src_int8 && divisible(szg_k, wzg_k)));
    for (auto &kv : attr.zero_points) UNIMPL_IF(!one_of(kv.first, {DNNL_ARG_SRC, DNNL_ARG_WEIGHTS, DNNL_ARG_DST}));

    if (!attr.reductions.empty()) {
        for (auto &kv : attr.reductions) UNIMPL_IF(kv.first != DNNL_ARG_SRC);
        const auto &pr = attr.pr(DNNL_ARG_SRC);
        UNIMPL_IF(!wz.set);
        UNIMPL_IF(pr.mask != full);
        UNIMPL_IF(pr.dt != dnnl_s32);
        if (pr.group_ndims) {
            const dnnl_dim_t prg = pr.group(1);
            dnnl_dim_t min_g = INT64_MAX, wzk = 1;
            if (wz.group_ndims) { wzk = wz.group(-2); min_g = std::min(min_g, wzk); }
            if (sz.group_ndims) min_g = std::min(min_g, sz.group(-1));
            if (ws.group_ndims) min_g = std::min(min_g, ws.group(-2));
            if (ss.group_ndims) min_g = std::min(min_g, ss.group(-1));
            INVALID_IF(prg > 1 && !src_int8);
            INVALID_IF(prg > 1 && !divisible(prg, wzk));
            INVALID_IF(prg > 1 && prg > min_g);
        }
    }

    // post-ops: binary / eltwise / prelu / sum only; src1 must have dst's
    // rank and broadcast-compatible dims (src/common/primitive_attr.cpp:389-412)
    for (const auto &e : attr.post_ops.entries) {
        UNIMPL_IF(!one_of(e.kind, {dnnl_binary, dnnl_eltwise, dnnl_prelu, dnnl_sum}));
        if (e.kind == dnnl_sum) {
            // the sum data type must have the size of the dst type
            if (e.sum_dt != dnnl_data_type_undef) UNIMPL_IF(dt_bits(e.sum_dt) != dt_bits(dst_dt));
            // a sum zero-point belongs to integer problems and an integer sum type
            // (src/common/primitive_attr.cpp:366-380)
            UNIMPL_IF(e.zero_point != 0 && !src_int8);
            const auto sum_dt = e.sum_dt != dnnl_data_type_undef ? e.sum_dt : dst_dt;
            UNIMPL_IF(e.zero_point != 0 && !one_of(sum_dt, {dnnl_s8, dnnl_u8, dnnl_s32}));
        }
        if (e.kind == dnnl_binary) {
            INVALID_IF(e.src1.ndims != pd.dst.ndims);
            for (int d = 0; d < pd.dst.ndims; ++d)
                INVALID_IF(e.src1.dims[d] != 1 && e.src1.dims[d] != pd.dst.dims[d]);
        }
    }
    return dnnl_success;
}

dnnl_status_t grouped_desc_check(const dnnl_memory_desc &src, const dnnl_memory_desc &wei,
        const dnnl_memory_desc *bias, const dnnl_memory_desc &dst) {
    UNIMPL_IF(!src.is_grouped());
    // 2D x 3D (variable M) only; the 2D x 2D variable-K form is not built
    UNIMPL_IF(!(dst.is_grouped() && !wei.is_grouped()));
    UNIMPL_IF(src.variable_dim_idx != 0 || dst.variable_dim_idx != 0);
    UNIMPL_IF(src.group_count != dst.group_count);
    UNIMPL_IF(src.offsets_dt != dnnl_s32 || dst.offsets_dt != dnnl_s32);
    UNIMPL_IF(src.ndims != 2 || wei.ndims != 3 || dst.ndims != 2);
    UNIMPL_IF(wei.dims[0] != src.group_count);
    UNIMPL_IF(src.dims[0] != dst.dims[0]);
    UNIMPL_IF(src.dims[1] != wei.dims[1]);
    UNIMPL_IF(dst.dims[1] != wei.dims[2]);
    if (wei.format_kind == dnnl_blocked) {
        const dnnl_dim_t K = wei.dims[1], N = wei.dims[2];
        const bool abc = wei.strides[2] == 1 && wei.strides[1] == N && wei.strides[0] == K * N;
        const bool acb = wei.strides[1] == 1 && wei.strides[2] == K && wei.strides[0] == K * N;
        UNIMPL_IF(!abc && !acb);
    }
    if (bias) {
        UNIMPL_IF(bias->is_grouped() || bias->ndims != 2);
        UNIMPL_IF(bias->dims[0] != src.group_count || bias->dims[1] != wei.dims[2]);
    }
    UNIMPL_IF(!dt_combo_ok(src.data_type, wei.data_type, dst.data_type));
    return dnnl_success;
}

dnnl_status_t grouped_attr_check(const dnnl_primitive_desc &pd) {
    const auto &attr = pd.attr;
    if (attr.has_default_values()) return dnnl_success;
    UNIMPL_IF(!attr.reductions.empty() || !attr.rounding.empty() || attr.deterministic);
    UNIMPL_IF(attr.acc_mode != dnnl_accumulation_mode_strict);
    const auto s = pd.src.data_type, w = pd.wei.data_type;
    UNIMPL_IF(one_of(s, {dnnl_f32, dnnl_bf16, dnnl_f16}) && attr.scale(DNNL_ARG_SRC).set);
    UNIMPL_IF(one_of(w, {dnnl_f32, dnnl_bf16, dnnl_f16}) && attr.scale(DNNL_ARG_WEIGHTS).set);
    UNIMPL_IF(attr.scale(DNNL_ARG_DST).set);
    for (const auto &e : attr.post_ops.entries) {
        UNIMPL_IF(e.kind != dnnl_eltwise && e.kind != dnnl_binary);
        if (e.kind == dnnl_binary) {
            UNIMPL_IF(e.alg != dnnl_binary_mul);
            INVALID_IF(e.src1.ndims != pd.dst.ndims);
            UNIMPL_IF(e.src1.is_grouped()); // grouped binary operands are not built
            const dnnl_dim_t bM = e.src1.dims[0], bN = e.src1.dims[1];
            const dnnl_dim_t gc = pd.dst.group_count, tM = pd.dst.dims[0];
            UNIMPL_IF(!(bN == 1 || (e.src1.strides[1] == 1 && e.src1.strides[0] == bN)));
            UNIMPL_IF(!((bM == gc || bM == tM) && (bM != gc || bM == tM || bN == 1)));
            UNIMPL_IF(bN != 1 && bN != pd.dst.dims[1]);
        }
    }
    return dnnl_success;
}

// ---- acceptance of each implementation (the pd_t::init of oneDNN) ---------

dnnl_status_t ref_dense_accepts(const dnnl_primitive_desc &pd) {
    const auto s = pd.src.data_type, w = pd.wei.data_type, d = pd.dst.data_type;
    const auto &attr = pd.attr;
    UNIMPL_IF(pd.src.ndims != 2); // a batched problem comes here as its 2D core (batch_core)
    const bool with_bias = pd.bias.ndims != 0;
    const dnnl_dim_t K = pd.K();
    if (is_int8(s)) { // ref_matmul_int8.hpp:44-92
        UNIMPL_IF(!is_int_wei(w));
        UNIMPL_IF(with_bias && !one_of(pd.bias.data_type, {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_s32, dnnl_s8, dnnl_u8}));
        UNIMPL_IF(!one_of(d, {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_s32, dnnl_s8, dnnl_u8}));
    } else { // ref_matmul.hpp:44-123
        UNIMPL_IF(!one_of(s, {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_f8_e5m2, dnnl_f8_e4m3}));
        UNIMPL_IF(!one_of(w, {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_f8_e5m2, dnnl_f8_e4m3, dnnl_u8, dnnl_s8, dnnl_u4, dnnl_s4}));
        // sub-byte float destinations are not built; 8-bit float ones go to the generic kernel
        UNIMPL_IF(!one_of(d, {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_f8_e5m2, dnnl_f8_e4m3, dnnl_u8, dnnl_s8}));
        UNIMPL_IF(!(s == w || one_of(w, {dnnl_bf16, dnnl_f16, dnnl_f8_e5m2, dnnl_f8_e4m3, dnnl_u8, dnnl_s8, dnnl_u4, dnnl_s4})));
        // integer weights convert to the src type only with apply_to_int and
        // an fpmath mode that covers that type (primitive_attr_t::mayiconvert,
        // src/common/primitive_attr.hpp:697-737)
        if (is_int_wei(w)) {
            UNIMPL_IF(!attr.apply_to_int);
            bool ok = false;
            switch (attr.fpmath) {
                case dnnl_fpmath_mode_strict: ok = s == dnnl_f32; break;
                case dnnl_fpmath_mode_any: ok = true; break;
                case dnnl_fpmath_mode_bf16: ok = s == dnnl_bf16 || s == dnnl_f32; break;
                case dnnl_fpmath_mode_f16: ok = s == dnnl_f16 || s == dnnl_f32; break;
                case dnnl_fpmath_mode_tf32: ok = s == dnnl_f32; break;
            }
            UNIMPL_IF(!ok);
        }
        UNIMPL_IF(s == dnnl_f16 && !one_of(d, {dnnl_f32, dnnl_f16, dnnl_u8, dnnl_s8}));
        if (with_bias) {
            const auto b = pd.bias.data_type;
            UNIMPL_IF(!one_of(b, {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_f8_e5m2, dnnl_f8_e4m3}));
            UNIMPL_IF(w == dnnl_f32 && b != dnnl_f32);
            UNIMPL_IF(w == dnnl_f16 && !one_of(b, {dnnl_f32, dnnl_f16}));
            UNIMPL_IF(w == dnnl_bf16 && !one_of(b, {dnnl_f32, dnnl_bf16}));
        }
        // this reference path has no src / dst zero-points and no reductions
        UNIMPL_IF(attr.zp(DNNL_ARG_SRC).set || attr.zp(DNNL_ARG_DST).set || !attr.reductions.empty());
    }
    // matmul_pd_t::attr_scales_ok / attr_zero_points_ok (matmul_pd.hpp:209-397)
    const auto &ss = attr.scale(DNNL_ARG_SRC);
    const auto &ws = attr.scale(DNNL_ARG_WEIGHTS);
    const auto &ds = attr.scale(DNNL_ARG_DST);
    if (ss.set) {
        // mask M alone is accepted by the int8 reference only
        if (ss.mask == 1) UNIMPL_IF(!is_int8(s));
        if (ss.group_ndims) UNIMPL_IF(ss.group(0) != 1 || K % ss.group(1) != 0);
    }
    if (ws.set) {
        // a K-dependent weights scale only for weights decompression or
        // together with grouped src scales
        if (ws.mask & 1) UNIMPL_IF(!(is_int_wei(w) || is_fp8(w)));
        if (ws.group_ndims) UNIMPL_IF(K % ws.group(0) != 0 || pd.N() % ws.group(1) != 0);
        else if (ws.mask & 1) UNIMPL_IF(false);
    }
    if (ds.set) UNIMPL_IF(ds.mask != 0 || ds.group_ndims != 0);
    const auto &wz = attr.zp(DNNL_ARG_WEIGHTS);
    if (wz.set && wz.group_ndims) UNIMPL_IF(K % wz.group(0) != 0 || pd.N() % wz.group(1) != 0);
    const auto &sz = attr.zp(DNNL_ARG_SRC);
    if (sz.set && sz.group_ndims) UNIMPL_IF(sz.group(0) != 1 || K % sz.group(1) != 0);
    // strided plain layouts only
    UNIMPL_IF(pd.src.format_kind != dnnl_blocked || pd.wei.format_kind != dnnl_blocked
            || pd.dst.format_kind != dnnl_blocked);
    return dnnl_success;
}

dnnl_status_t ref_grouped_accepts(const dnnl_primitive_desc &pd) {
    const auto s = pd.src.data_type, w = pd.wei.data_type, d = pd.dst.data_type;
    const auto &attr = pd.attr;
    const bool fp_s = one_of(s, {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_f8_e5m2, dnnl_f8_e4m3});
    const bool fp_w = one_of(w, {dnnl_f32, dnnl_bf16, dnnl_f16, dnnl_f8_e5m2, dnnl_f8_e4m3});
    const bool int_s = is_int8(s), int_w = is_int_wei(w);
    UNIMPL_IF(!(fp_s || int_s) || !(fp_w || int_w));
    UNIMPL_IF(!one_of(d, {dnnl_f32, dnnl_bf16, dnnl_f16}));
    UNIMPL_IF(int_s && !int_w);
    UNIMPL_IF(fp_s && int_w && !attr.scale(DNNL_ARG_WEIGHTS).set);
    UNIMPL_IF(fp_s && int_w && !attr.apply_to_int);
    const dnnl_dim_t K = pd.K();
    const auto &ss = attr.scale(DNNL_ARG_SRC);
    if (ss.set) {
        UNIMPL_IF(ss.mask != 1 && ss.mask != 3);
        if (ss.group_ndims) UNIMPL_IF(ss.group(-2) != 1 || ss.group(-1) <= 1 || K % ss.group(-1) != 0);
    }
    const auto &ws = attr.scale(DNNL_ARG_WEIGHTS);
    if (ws.set) {
        UNIMPL_IF(ws.mask != 0b101 && ws.mask != 0b111);
        if (ws.group_ndims) UNIMPL_IF(ws.group(-2) <= 1 || K % ws.group(-2) != 0 || ws.group(-1) != 1);
    }
    UNIMPL_IF(attr.zp(DNNL_ARG_DST).set);
    const auto &sz = attr.zp(DNNL_ARG_SRC);
    if (sz.set) {
        UNIMPL_IF(!int_s || !one_of(sz.dt, {dnnl_u8, dnnl_s8, dnnl_s32}));
        UNIMPL_IF(sz.mask != 1 && sz.mask != 3);
        if (sz.group_ndims) UNIMPL_IF(sz.group(-2) != 1 || sz.group(-1) <= 1 || K % sz.group(-1) != 0);
    }
    const auto &wz = attr.zp(DNNL_ARG_WEIGHTS);
    if (wz.set) {
        UNIMPL_IF(!int_w);
        UNIMPL_IF(wz.mask != 0b101 && wz.mask != 0b111);
        if (wz.group_ndims) UNIMPL_IF(wz.group(-2) <= 1 || K % wz.group(-2) != 0 || wz.group(-1) != 1);
    }
    if (ss.set && ss.group_ndims && ws.set && ws.group_ndims)
        UNIMPL_IF(!(ss.group(-1) % ws.group(-2) == 0 || ws.group(-2) % ss.group(-1) == 0));
    if (ws.set && wz.set) UNIMPL_IF(ws.group(-2) != wz.group(-2));
    return dnnl_success;
}

// tcgen05 GEMM: dense 2D, 8-bit x 8-bit, quantization parameters constant
// along K; everything the reference implementation of the same problem
// accepts, minus K-grouped parameters and precomputed reductions.
dnnl_status_t tc_accepts(const dnnl_primitive_desc &pd) {
    if (ref_dense_accepts(pd) != dnnl_success) return dnnl_unimplemented;
    const auto s = pd.src.data_type, w = pd.wei.data_type;
    const auto &attr = pd.attr;
    const bool int_path = is_int8(s);
    UNIMPL_IF(!((int_path && is_int8(w)) || (is_fp8(s) && is_fp8(w))));
    UNIMPL_IF(is_fp8(pd.dst.data_type) || (pd.bias.ndims && is_fp8(pd.bias.data_type))); // no 8-bit float stores / bias here
    const dnnl_dim_t M = pd.M(), N = pd.N(), K = pd.K();
    UNIMPL_IF(M == 0 || N == 0 || K == 0);
    UNIMPL_IF(M >= (1LL << 31) || N >= (1LL << 31) || K >= (1LL << 31));
    // TMA: rows of 16-byte multiples; src K-contiguous, weights `ab` or `ba`
    UNIMPL_IF(pd.src.strides[1] != 1 || pd.src.strides[0] % 16 != 0 || pd.src.strides[0] < K);
    const bool ab = pd.wei.strides[1] == 1 && pd.wei.strides[0] % 16 == 0 && pd.wei.strides[0] >= N;
    const bool ba = pd.wei.strides[0] == 1 && pd.wei.strides[1] % 16 == 0 && pd.wei.strides[1] >= K && N > 1;
    UNIMPL_IF(!ab && !ba);
    const auto &ss = attr.scale(DNNL_ARG_SRC), &ws = attr.scale(DNNL_ARG_WEIGHTS);
    if (ss.set) UNIMPL_IF(ss.group_ndims || !(ss.mask == 0 || (ss.mask == 1 && int_path)));
    if (ws.set) UNIMPL_IF(ws.group_ndims || !(ws.mask == 0 || ws.mask == 2));
    const auto &sz = attr.zp(DNNL_ARG_SRC), &wz = attr.zp(DNNL_ARG_WEIGHTS);
    if (sz.set) UNIMPL_IF(sz.group_ndims || sz.mask != 0 || sz.dt != dnnl_s32 || sz.on_host);
    if (wz.set) UNIMPL_IF(wz.group_ndims || !(wz.mask == 0 || wz.mask == 2) || wz.on_host);
    UNIMPL_IF(!attr.reductions.empty());
    // The kernel adds K products of 8-bit values in s32 and subtracts the zero-point terms afterwards;
    // the reference adds (s - zs)(w - zw) directly.  Both stay inside s32, and so agree, while
    // K * 255 * 255 < 2^31; longer sums go to the generic kernel, which adds in the reference's order.
    UNIMPL_IF(int_path && K > 33025);
    return dnnl_success;
}

// Skinny weight-decompression GEMM: few src rows (decode), bf16/f16 src,
// s4/u4 `ab` weights, weight scales per N or per (K-group, N), optional
// zero-points with the same grouping (or per tensor).
dnnl_status_t woq_accepts(const dnnl_primitive_desc &pd) {
    if (ref_dense_accepts(pd) != dnnl_success) return dnnl_unimplemented;
    const auto s = pd.src.data_type, w = pd.wei.data_type;
    const auto &attr = pd.attr;
    UNIMPL_IF(!(s == dnnl_bf16 || s == dnnl_f16) || !(w == dnnl_s4 || w == dnnl_u4));
    UNIMPL_IF(is_fp8(pd.dst.data_type) || (pd.bias.ndims && is_fp8(pd.bias.data_type)));
    const dnnl_dim_t M = pd.M(), N = pd.N(), K = pd.K();
    UNIMPL_IF(M < 1 || M > 32 || N % 32 != 0 || K % 16 != 0 || K < 16);
    UNIMPL_IF(N >= (1LL << 31) || K >= (1LL << 31));
    UNIMPL_IF(pd.src.strides[1] != 1 || pd.src.strides[0] % 2 != 0);
    UNIMPL_IF(pd.wei.strides[1] != 1 || pd.wei.strides[0] % 32 != 0 || pd.wei.strides[0] < N);
    const auto &ws = attr.scale(DNNL_ARG_WEIGHTS), &ss = attr.scale(DNNL_ARG_SRC);
    UNIMPL_IF(!ws.set || ws.on_host);
    dnnl_dim_t group = K;
    if (ws.mask == 3) {
        UNIMPL_IF(!ws.group_ndims || ws.groups[1] != 1 || ws.groups[0] % 16 != 0);
        group = ws.groups[0];
    } else UNIMPL_IF(ws.mask != 2 || ws.group_ndims);
    if (ss.set) UNIMPL_IF(ss.mask != 0 || ss.group_ndims);
    const auto &wz = attr.zp(DNNL_ARG_WEIGHTS);
    if (wz.set) {
        UNIMPL_IF(wz.on_host);
        if (wz.mask == 3) {
            UNIMPL_IF(!wz.group_ndims || wz.groups[1] != 1 || wz.groups[0] != group);
        } else UNIMPL_IF(wz.mask != 0);
    }
    return dnnl_success;
}

// int4 decompression through tensor memory: what the skinny GEMM accepts, with
// the src rows reachable by TMA (16-byte row pitch unless there is one row)
dnnl_status_t woq_tc_accepts(const dnnl_primitive_desc &pd) {
    if (woq_accepts(pd) != dnnl_success) return dnnl_unimplemented;
    UNIMPL_IF(pd.M() > 1 && pd.src.strides[0] % 8 != 0);
    UNIMPL_IF(pd.wei.strides[0] % 32 != 0);
    // the scale / zero-point rows of a stage's groups must fit in the kernel's shared-memory ring
    const auto &ws = pd.attr.scale(DNNL_ARG_WEIGHTS);
    const auto &wz = pd.attr.zp(DNNL_ARG_WEIGHTS);
    const dnnl_dim_t group = ws.mask == 3 ? ws.groups[0] : pd.K();
    UNIMPL_IF(!woq_tc_fits(pd.M(), pd.K(), group, (int)ws.dt, (wz.set && wz.mask == 3) ? (int)wz.dt : -1));
    return dnnl_success;
}

// weight zero-points the s8-decompression tensor-core kernel handles: one per
// (expert, column) for grouped problems, one per tensor or per column otherwise
bool woq_tc_wei_zp_ok(const dnnl_primitive_desc &pd) {
    const auto &wz = pd.attr.zp(DNNL_ARG_WEIGHTS);
    if (!wz.set) return true;
    if (wz.on_host || wz.group_ndims || !one_of(wz.dt, {dnnl_s8, dnnl_u8, dnnl_s32})) return false;
    return pd.grouped ? wz.mask == 0b101 : (wz.mask == 0 || wz.mask == 2);
}

// tcgen05 grouped GEMM: bf16 src rows x s8 weights [G, K, N] (N contiguous)
// with one weight scale per (expert, column); optional bias [G, N] and
// eltwise / binary post-ops.
dnnl_status_t grouped_tc_accepts(const dnnl_primitive_desc &pd) {
    if (ref_grouped_accepts(pd) != dnnl_success) return dnnl_unimplemented;
    const auto &attr = pd.attr;
    UNIMPL_IF(pd.src.data_type != dnnl_bf16 || pd.wei.data_type != dnnl_s8);
    UNIMPL_IF(!one_of(pd.dst.data_type, {dnnl_bf16, dnnl_f16, dnnl_f32}));
    UNIMPL_IF(!attr.apply_to_int);
    for (const auto &e : attr.post_ops.entries) UNIMPL_IF(e.kind != dnnl_eltwise && e.kind != dnnl_binary); // no sum
    const auto &ws = attr.scale(DNNL_ARG_WEIGHTS);
    UNIMPL_IF(!ws.set || ws.on_host || ws.mask != 0b101 || ws.group_ndims);
    UNIMPL_IF(attr.scale(DNNL_ARG_SRC).set || attr.scale(DNNL_ARG_DST).set);
    UNIMPL_IF(attr.zp(DNNL_ARG_SRC).set || attr.zp(DNNL_ARG_DST).set || !woq_tc_wei_zp_ok(pd));
    const dnnl_dim_t N = pd.N(), K = pd.K();
    UNIMPL_IF(N >= (1LL << 31) || K >= (1LL << 31) || pd.M() >= (1LL << 31) || pd.src.group_count < 1);
    // TMA: unit inner strides, 16-byte multiples for the others
    UNIMPL_IF(pd.wei.strides[2] != 1 || pd.wei.strides[1] % 16 != 0 || pd.wei.strides[0] % 16 != 0
            || pd.wei.strides[1] < N);
    UNIMPL_IF(pd.src.strides[1] != 1 || pd.src.strides[0] % 8 != 0 || pd.dst.strides[1] != 1);
    return dnnl_success;
}

// Dense weight decompression on the tensor cores (prefill-sized M): bf16 src x
// s8 `ab` weights with one scale per tensor or per column; optional bias and
// eltwise / binary post-ops.
dnnl_status_t dense_woq8_accepts(const dnnl_primitive_desc &pd) {
    if (ref_dense_accepts(pd) != dnnl_success) return dnnl_unimplemented;
    const auto &attr = pd.attr;
    UNIMPL_IF(pd.src.ndims != 2);
    UNIMPL_IF(pd.src.data_type != dnnl_bf16 || pd.wei.data_type != dnnl_s8);
    UNIMPL_IF(!one_of(pd.dst.data_type, {dnnl_bf16, dnnl_f16, dnnl_f32}));
    UNIMPL_IF(!attr.apply_to_int);
    for (const auto &e : attr.post_ops.entries) UNIMPL_IF(e.kind != dnnl_eltwise && e.kind != dnnl_binary); // no sum
    const auto &ws = attr.scale(DNNL_ARG_WEIGHTS);
    UNIMPL_IF(!ws.set || ws.on_host || (ws.mask != 0 && ws.mask != 2) || ws.group_ndims);
    UNIMPL_IF(attr.scale(DNNL_ARG_SRC).set || attr.scale(DNNL_ARG_DST).set);
    UNIMPL_IF(attr.zp(DNNL_ARG_SRC).set || attr.zp(DNNL_ARG_DST).set || !woq_tc_wei_zp_ok(pd));
    const dnnl_dim_t N = pd.N(), K = pd.K();
    UNIMPL_IF(N >= (1LL << 31) || K >= (1LL << 31) || pd.M() >= (1LL << 31) || pd.M() < 1);
    UNIMPL_IF(pd.wei.strides[1] != 1 || pd.wei.strides[0] % 16 != 0 || pd.wei.strides[0] < N);
    UNIMPL_IF(pd.src.strides[1] != 1 || pd.src.strides[0] % 8 != 0 || pd.dst.strides[1] != 1);
    return dnnl_success;
}

dnnl_status_t impl_accepts(const dnnl_primitive_desc &pd, int impl, std::string &name) {
    switch (impl) {
        case IMPL_GROUPED_TC:
            if (!pd.grouped) { // the same kernel with the dense problem as its only group
                name = "cuda:tcgen05:woq8";
                return dense_woq8_accepts(pd);
            }
            name = "cuda:tcgen05:grouped";
            return grouped_tc_accepts(pd);
        case IMPL_WOQ_TC:
            if (pd.grouped) return dnnl_unimplemented;
            name = "cuda:tcgen05:woq4";
            return woq_tc_accepts(pd);
        case IMPL_WOQ_GEMV:
            if (pd.grouped) return dnnl_unimplemented;
            name = "cuda:woq:skinny";
            return woq_accepts(pd);
        case IMPL_TCGEN05_GEMM:
            if (pd.grouped) return dnnl_unimplemented;
            name = is_int8(pd.src.data_type) ? "cuda:tcgen05:int8" : "cuda:tcgen05:fp8";
            return tc_accepts(pd);
        case IMPL_REF:
            name = pd.grouped ? "cuda:ref_grouped:any" : is_int8(pd.src.data_type) ? "cuda:ref_int8:any" : "cuda:ref:any";
            return pd.grouped ? ref_grouped_accepts(pd) : ref_dense_accepts(pd);
        default: return dnnl_unimplemented;
    }
}

dnnl_status_t select_impl(dnnl_primitive_desc &pd, int first) {
    for (int i = first; i < IMPL_COUNT; ++i) {
        std::string name;
        if (impl_accepts(pd, i, name) == dnnl_success) {
            pd.impl = i;
            pd.impl_name = name;
            // scratchpad: the tensor-core GEMM keeps its zero-point
            // compensation sums there
            pd.scratch_bytes = 0;
            if (i == IMPL_TCGEN05_GEMM && (pd.attr.zp(DNNL_ARG_SRC).set || pd.attr.zp(DNNL_ARG_WEIGHTS).set))
                pd.scratch_bytes = gemm_tc_scratch_bytes(pd.M(), pd.N());
            // the skinny GEMM keeps split-K partial sums and arrival counters there
            if (i == IMPL_WOQ_TC)
                pd.scratch_bytes = woq_tc_scratch_bytes(
                        pd.M(), pd.N(), pd.K(), pd.engine->sm_count > 0 ? pd.engine->sm_count : 148);
            if (i == IMPL_WOQ_GEMV)
                pd.scratch_bytes = woq_skinny_scratch_bytes(
                        pd.N(), pd.K(), pd.engine->sm_count > 0 ? pd.engine->sm_count : 148);
            // the grouped GEMM keeps its per-expert tile ranges there
            if (i == IMPL_GROUPED_TC)
                pd.scratch_bytes = grouped_tc_scratch_bytes(pd.grouped ? (int)pd.src.group_count : 1, pd.M());
            pd.scratchpad = dnnl_memory_desc();
            if (pd.scratch_bytes && pd.attr.scratchpad_mode == dnnl_scratchpad_mode_user) {
                pd.scratchpad.ndims = 1;
                pd.scratchpad.dims[0] = (dnnl_dim_t)pd.scratch_bytes;
                pd.scratchpad.strides[0] = 1;
                pd.scratchpad.data_type = dnnl_u8;
                pd.scratchpad.format_kind = dnnl_blocked;
            }
            return dnnl_success;
        }
    }
    return first == 0 ? dnnl_unimplemented : dnnl_last_impl_reached;
}

// memory descriptor of a quantization parameter: tensor dims masked, the last
// two divided by the groups, dense row-major (primitive_attr_quant.hpp:116-140)
dnnl_memory_desc quant_md(const quant_entry_t &q, const dnnl_memory_desc &base) {
    dnnl_memory_desc md;
    if (q.on_host) {
        md.ndims = 1; md.dims[0] = 1; md.strides[0] = 1;
        md.data_type = q.dt; md.format_kind = dnnl_format_kind_host_scalar;
        return md;
    }
    md.ndims = base.ndims;
    md.data_type = q.dt;
    md.format_kind = dnnl_blocked;
    for (int i = 0; i < base.ndims; ++i) md.dims[i] = (q.mask & (1 << i)) ? base.dims[i] : 1;
    if (q.group_ndims) { // a dim left open until execution stays open
        if (md.dims[base.ndims - 2] != DNNL_RUNTIME_DIM_VAL) md.dims[base.ndims - 2] /= q.groups[0];
        if (md.dims[base.ndims - 1] != DNNL_RUNTIME_DIM_VAL) md.dims[base.ndims - 1] /= q.groups[1];
    }
    dnnl_dim_t acc = 1;
    for (int i = base.ndims - 1; i >= 0; --i) {
        md.strides[i] = acc;
        acc = (acc == DNNL_RUNTIME_DIM_VAL || md.dims[i] == DNNL_RUNTIME_DIM_VAL) ? DNNL_RUNTIME_DIM_VAL : acc * md.dims[i];
    }
    return md;
}

void fill_quant_mds(dnnl_primitive_desc &pd) {
    pd.quant_mds.clear();
    auto base = [&](int arg) -> const dnnl_memory_desc & {
        return arg == DNNL_ARG_SRC ? pd.src : arg == DNNL_ARG_WEIGHTS ? pd.wei : pd.dst;
    };
    for (auto &kv : pd.attr.scales) pd.quant_mds[DNNL_ARG_ATTR_SCALES | kv.first] = quant_md(kv.second, base(kv.first));
    for (auto &kv : pd.attr.zero_points)
        pd.quant_mds[DNNL_ARG_ATTR_ZERO_POINTS | kv.first] = quant_md(kv.second, base(kv.first));
    for (auto &kv : pd.attr.reductions)
        pd.quant_mds[DNNL_ARG_ATTR_PRECOMPUTED_REDUCTIONS | kv.first] = quant_md(kv.second, base(kv.first));
}

const dnnl_memory_desc g_zero_md;

// prelu: f32 weights over the dst dims its mask names, dense, with dim 1 innermost beyond two
// dims (ab, acb, acdb, acdeb: src/cpu/primitive_attr_postops.cpp:219-242); kept in src1 so that
// the kernels see it as a binary operand
void build_prelu_mds(dnnl_primitive_desc &pd) {
    for (auto &e : pd.attr.post_ops.entries)
        if (e.kind == dnnl_prelu && !pd.grouped) {
            const int nd = pd.dst.ndims;
            dnnl_memory_desc w;
            w.ndims = nd;
            w.data_type = dnnl_f32;
            w.format_kind = dnnl_blocked;
            for (int d = 0; d < nd; ++d) w.dims[d] = ((e.prelu_mask >> d) & 1) ? pd.dst.dims[d] : 1;
            int order[DNNL_MAX_NDIMS]; // outermost first
            int k = 0;
            if (nd <= 2) for (int d = 0; d < nd; ++d) order[k++] = d;
            else {
                order[k++] = 0;
                for (int d = 2; d < nd; ++d) order[k++] = d;
                order[k++] = 1;
            }
            dnnl_dim_t acc = 1;
            for (int i = nd - 1; i >= 0; --i) {
                w.strides[order[i]] = acc;
                acc *= w.dims[order[i]] == 0 ? 1 : w.dims[order[i]];
            }
            e.src1 = w;
        }
}

dnnl_dim_t lcm_of(dnnl_dim_t a, dnnl_dim_t b) {
    if (a <= 0 || b <= 0) return a > b ? a : b;
    dnnl_dim_t x = a, y = b;
    while (y) { const dnnl_dim_t t = x % y; x = y; y = t; }
    return a / x * b;
}

// A 2D descriptor with run-time dims, made concrete for the checks at creation and for the
// implementation list: every open dim takes the value another tensor gives it, else a stand-in
// (1, or the least common multiple of the groups that must divide it); open strides become dense
// row-major.  What executes is settled again from the memory objects.
void apply_stand_ins(dnnl_primitive_desc &pd) {
    const dnnl_dim_t RT = DNNL_RUNTIME_DIM_VAL;
    dnnl_dim_t M = RT, K = RT, N = RT;
    auto learn = [&](dnnl_dim_t &v, dnnl_dim_t d) { if (v == RT && d != RT) v = d; };
    learn(M, pd.src.dims[0]); learn(M, pd.dst.dims[0]);
    learn(K, pd.src.dims[1]); learn(K, pd.wei.dims[0]);
    learn(N, pd.wei.dims[1]); learn(N, pd.dst.dims[1]);
    // an operand that states a full extent (a residual with M rows while M is open) tells it too
    auto learn_from = [&](const dnnl_memory_desc &md) {
        if (md.ndims != 2) return;
        if (md.dims[0] != RT && md.dims[0] > 1) learn(M, md.dims[0]);
        if (md.dims[1] != RT && md.dims[1] > 1) learn(N, md.dims[1]);
    };
    learn_from(pd.bias);
    for (auto &e : pd.attr.post_ops.entries)
        if (e.kind == dnnl_binary) learn_from(e.src1);
    dnnl_dim_t gk = 1, gn = 1;
    for (auto *m : {&pd.attr.scales, &pd.attr.zero_points, &pd.attr.reductions})
        for (auto &kv : *m)
            if (kv.second.group_ndims) {
                if (kv.first == DNNL_ARG_SRC) gk = lcm_of(gk, kv.second.groups[1]);
                if (kv.first == DNNL_ARG_WEIGHTS) { gk = lcm_of(gk, kv.second.groups[0]); gn = lcm_of(gn, kv.second.groups[1]); }
                if (kv.first == DNNL_ARG_DST) gn = lcm_of(gn, kv.second.groups[1]);
            }
    if (M == RT) M = 1;
    if (K == RT) K = gk;
    if (N == RT) N = gn;
    // stated dims stay (contradictions between tensors are then found by the usual checks)
    auto fix = [&](dnnl_memory_desc &md, dnnl_dim_t d0, dnnl_dim_t d1) {
        if (md.ndims != 2) return;
        const bool open = md.has_runtime_dims();
        if (md.dims[0] == RT) md.dims[0] = d0;
        if (md.dims[1] == RT) md.dims[1] = d1;
        if (open || md.format_kind == dnnl_format_kind_any) {
            md.format_kind = dnnl_blocked;
            md.strides[1] = 1;
            md.strides[0] = md.dims[1] == 0 ? 1 : md.dims[1];
        }
    };
    fix(pd.src, M, K);
    fix(pd.wei, K, N);
    fix(pd.dst, M, N);
    fix(pd.bias, M, N);
    for (auto &e : pd.attr.post_ops.entries)
        if (e.kind == dnnl_binary) fix(e.src1, M, N);
}

// The 2D core of a batched descriptor: the last two dims of every tensor, quantization masks
// without the batch bits.  Parameters that vary along a batch dim are not built.
dnnl_status_t batch_core(const dnnl_primitive_desc &pd, dnnl_primitive_desc &core) {
    core = pd;
    core.batched = false;
    const int nd = pd.dst.ndims, nb = nd - 2;
    auto last2 = [&](dnnl_memory_desc &md) {
        if (md.ndims == 0) return;
        dnnl_memory_desc m = md;
        m.ndims = 2;
        for (int i = 0; i < 2; ++i) {
            m.dims[i] = md.dims[nb + i];
            m.strides[i] = md.strides[nb + i];
        }
        md = m;
    };
    last2(core.src); last2(core.wei); last2(core.dst); last2(core.bias);
    for (auto &e : core.attr.post_ops.entries)
        if (e.kind == dnnl_binary || e.kind == dnnl_prelu) {
            if (e.src1.ndims != nd) return dnnl_unimplemented;
            last2(e.src1);
        }
    const int batch_bits = (1 << nb) - 1;
    for (auto *m : {&core.attr.scales, &core.attr.zero_points, &core.attr.reductions})
        for (auto &kv : *m) {
            if (kv.second.mask & batch_bits) return dnnl_unimplemented;
            kv.second.mask >>= nb;
        }
    return dnnl_success;
}


} // namespace

extern "C" {

dnnl_status_t dnnl_matmul_primitive_desc_create(dnnl_primitive_desc_t *primitive_desc, dnnl_engine_t engine,
        const_dnnl_memory_desc_t src_desc, const_dnnl_memory_desc_t weights_desc,
        const_dnnl_memory_desc_t bias_desc, const_dnnl_memory_desc_t dst_desc,
        const_dnnl_primitive_attr_t attr) {
    if (!primitive_desc || !engine || !src_desc || !weights_desc || !dst_desc) return dnnl_invalid_arguments;
    for (auto *md : {src_desc, weights_desc, bias_desc, dst_desc})
        if (md && md->format_kind == dnnl_format_kind_host_scalar) return dnnl_invalid_arguments;
    const dnnl_memory_desc *bias = (bias_desc && bias_desc->ndims != 0) ? bias_desc : nullptr;

    auto pd = new dnnl_primitive_desc;
    pd->engine = engine;
    pd->src = *src_desc;
    pd->wei = *weights_desc;
    pd->dst = *dst_desc;
    if (bias) pd->bias = *bias;
    if (attr) pd->attr = *attr;
    pd->grouped = src_desc->is_grouped();

    // Run-time shapes (DNNL_RUNTIME_DIM_VAL, src/common/matmul.cpp:630-744) of a dense 2D problem:
    // any of M, K, N and the strides may be left open, in bias and binary operands too.  The
    // descriptor is checked, and its implementation list made, with stand-ins for the open dims;
    // what the queries report stays as the caller gave it; every execution settles the shapes
    // again from the memory objects.
    bool has_open = pd->src.has_runtime_dims() || pd->wei.has_runtime_dims() || pd->dst.has_runtime_dims()
            || pd->bias.has_runtime_dims();
    for (auto &e : pd->attr.post_ops.entries) has_open = has_open || (e.kind == dnnl_binary && e.src1.has_runtime_dims());
    if (has_open) {
        const bool ok = !pd->grouped && pd->src.ndims == 2 && pd->dst.ndims == 2 && pd->wei.ndims == 2
                && (pd->bias.ndims == 0 || pd->bias.ndims == 2);
        if (!ok) {
            delete pd;
            return dnnl_unimplemented;
        }
        for (auto &e : pd->attr.post_ops.entries) // `any` on an operand whose dims are known: row-major
            if (e.kind == dnnl_binary && !e.src1.has_runtime_dims()) set_default_format(e.src1);
        dnnl_primitive_desc chk = *pd;
        apply_stand_ins(chk);
        dnnl_status_t rst = dense_desc_check(chk.src, chk.wei, chk.bias.ndims ? &chk.bias : nullptr, chk.dst);
        if (rst == dnnl_success) {
            for (auto &e : chk.attr.post_ops.entries)
                if (e.kind == dnnl_sum && e.sum_dt == dnnl_data_type_undef) e.sum_dt = chk.dst.data_type;
            build_prelu_mds(chk);
            rst = dense_attr_check(chk);
        }
        if (rst == dnnl_success) rst = select_impl(chk, 0);
        if (rst != dnnl_success) {
            delete pd;
            return rst;
        }
        pd->runtime_m = true;
        pd->impl = chk.impl; pd->impl_name = chk.impl_name;
        pd->scratch_bytes = chk.scratch_bytes; pd->scratchpad = chk.scratchpad;
        for (auto &e : pd->attr.post_ops.entries)
            if (e.kind == dnnl_sum && e.sum_dt == dnnl_data_type_undef) e.sum_dt = pd->dst.data_type;
        // `any` resolves to row-major here as everywhere; strides that depend on an open dim stay open
        for (auto *md : {&pd->src, &pd->wei, &pd->dst, &pd->bias})
            if (md->ndims == 2 && md->format_kind == dnnl_format_kind_any) {
                md->format_kind = dnnl_blocked;
                md->strides[1] = 1;
                md->strides[0] = md->dims[1];
            }
        fill_quant_mds(*pd);
        *primitive_desc = pd;
        return dnnl_success;
    }

    dnnl_status_t st = pd->grouped ? grouped_desc_check(pd->src, pd->wei, bias, pd->dst)
                                   : dense_desc_check(pd->src, pd->wei, bias, pd->dst);
    if (st == dnnl_success) {
        // format_tag::any: this engine uses plain row-major layouts
        set_default_format(pd->src);
        set_default_format(pd->wei);
        set_default_format(pd->dst);
        set_default_format(pd->bias);
        for (auto &e : pd->attr.post_ops.entries)
            if (e.kind == dnnl_binary) set_default_format(e.src1);
        for (auto &e : pd->attr.post_ops.entries)
            if (e.kind == dnnl_sum && e.sum_dt == dnnl_data_type_undef) e.sum_dt = pd->dst.data_type;
        build_prelu_mds(*pd);
        st = pd->grouped ? grouped_attr_check(*pd) : dense_attr_check(*pd);
    }
    // Batched (ndims > 2, src/common/matmul.cpp:630-744 with broadcast of size-1 batch dims): the
    // implementation is chosen for the 2D core and run once per matrix of the batch.
    const bool batched = st == dnnl_success && !pd->grouped && pd->dst.ndims > 2;
    if (batched) {
        if (pd->src.format_kind != dnnl_blocked || pd->wei.format_kind != dnnl_blocked
                || pd->dst.format_kind != dnnl_blocked)
            st = dnnl_unimplemented;
        dnnl_primitive_desc core;
        if (st == dnnl_success) st = batch_core(*pd, core);
        if (st == dnnl_success) st = select_impl(core, 0);
        if (st == dnnl_success) {
            pd->batched = true;
            pd->impl = core.impl;
            pd->impl_name = core.impl_name;
            pd->scratch_bytes = core.scratch_bytes;
            pd->scratchpad = core.scratchpad;
        }
    } else if (st == dnnl_success) st = select_impl(*pd, 0);
    if (st != dnnl_success) {
        delete pd;
        return st;
    }
    fill_quant_mds(*pd);
    *primitive_desc = pd;
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_desc_next_impl(dnnl_primitive_desc_t pd) {
    if (!pd) return dnnl_invalid_arguments;
    if (pd->kind != dnnl_matmul) return dnnl_last_impl_reached; // one reorder implementation
    dnnl_primitive_desc tmp = *pd;
    if (tmp.runtime_m) {
        apply_stand_ins(tmp);
        build_prelu_mds(tmp);
    }
    if (pd->batched && batch_core(*pd, tmp) != dnnl_success) return dnnl_last_impl_reached;
    dnnl_status_t st = select_impl(tmp, pd->impl + 1);
    if (st != dnnl_success) return dnnl_last_impl_reached;
    pd->scratch_bytes = tmp.scratch_bytes;
    pd->scratchpad = tmp.scratchpad;
    pd->impl = tmp.impl;
    pd->impl_name = tmp.impl_name;
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_desc_clone(dnnl_primitive_desc_t *pd, const_dnnl_primitive_desc_t existing) {
    if (!pd || !existing) return dnnl_invalid_arguments;
    *pd = new dnnl_primitive_desc(*existing);
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_desc_get_attr(const_dnnl_primitive_desc_t pd, const_dnnl_primitive_attr_t *attr) {
    if (!pd || !attr) return dnnl_invalid_arguments;
    *attr = &pd->attr;
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_desc_destroy(dnnl_primitive_desc_t pd) {
    delete pd;
    return dnnl_success;
}

const_dnnl_memory_desc_t dnnl_primitive_desc_query_md(const_dnnl_primitive_desc_t pd, dnnl_query_t what, int index) {
    if (!pd) return nullptr;
    switch ((int)what) {
        case dnnl_query_src_md: return index == 0 ? &pd->src : nullptr;
        case dnnl_query_weights_md: return index == 0 ? &pd->wei : index == 1 ? &pd->bias : nullptr;
        case dnnl_query_dst_md: return index == 0 ? &pd->dst : nullptr;
        case dnnl_query_workspace_md: return &g_zero_md;
        case dnnl_query_scratchpad_md: return &pd->scratchpad;
        case dnnl_query_exec_arg_md: {
            if (index == DNNL_ARG_SRC) return &pd->src;
            if (index == DNNL_ARG_WEIGHTS) return &pd->wei;
            if (index == DNNL_ARG_BIAS) return &pd->bias;
            if (index == DNNL_ARG_DST) return &pd->dst;
            if (index == DNNL_ARG_SCRATCHPAD) return &pd->scratchpad;
            auto it = pd->quant_mds.find(index);
            if (it != pd->quant_mds.end()) return &it->second;
            const int n = (int)pd->attr.post_ops.entries.size();
            for (int i = 0; i < n; ++i)
                if (index == (DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_SRC_1)
                        && pd->attr.post_ops.entries[i].kind == dnnl_binary)
                    return &pd->attr.post_ops.entries[i].src1;
            return &g_zero_md;
        }
        default: return nullptr;
    }
}

dnnl_status_t dnnl_primitive_desc_query(const_dnnl_primitive_desc_t pd, dnnl_query_t what, int index, void *result) {
    if (!pd || !result) return dnnl_invalid_arguments;
    int n_binary = 0;
    for (const auto &e : pd->attr.post_ops.entries) n_binary += e.kind == dnnl_binary;
    switch ((int)what) {
        case dnnl_query_engine:
        case dnnl_query_scratchpad_engine: *(dnnl_engine_t *)result = pd->engine; break;
        case dnnl_query_primitive_kind: *(dnnl_primitive_kind_t *)result = pd->kind; break;
        case dnnl_query_num_of_inputs_s32:
            *(int *)result = pd->kind == dnnl_reorder ? 1 : 2 + (pd->bias.ndims != 0) + n_binary;
            break;
        case dnnl_query_num_of_outputs_s32: *(int *)result = 1; break;
        case dnnl_query_time_estimate_f64: *(double *)result = 0.0; break;
        case dnnl_query_memory_consumption_s64: *(dnnl_dim_t *)result = 0; break;
        case dnnl_query_impl_info_str: *(const char **)result = pd->impl_name.c_str(); break;
        case dnnl_query_prop_kind: *(int *)result = 0; break;
        default: {
            const_dnnl_memory_desc_t md = dnnl_primitive_desc_query_md(pd, what, index);
            if (!md) return dnnl_unimplemented;
            *(const_dnnl_memory_desc_t *)result = md;
        }
    }
    return dnnl_success;
}

int dnnl_primitive_desc_query_s32(const_dnnl_primitive_desc_t pd, dnnl_query_t what, int index) {
    int v = 0;
    if (what == dnnl_query_num_of_inputs_s32 || what == dnnl_query_num_of_outputs_s32)
        dnnl_primitive_desc_query(pd, what, index, &v);
    return v;
}

dnnl_status_t dnnl_primitive_create(dnnl_primitive_t *primitive, const_dnnl_primitive_desc_t pd) {
    if (!primitive || !pd) return dnnl_invalid_arguments;
    auto *p = new dnnl_primitive;
    p->pd = *pd;
    if (pd->runtime_m && pd->attr.scratchpad_mode == dnnl_scratchpad_mode_user) { // its size is not known yet
        delete p;
        return dnnl_unimplemented;
    }
    if (pd->scratch_bytes && !pd->runtime_m && pd->attr.scratchpad_mode == dnnl_scratchpad_mode_library) {
        if (pd->engine->device < 0) { /* device-less engine: nothing to allocate */ }
        else {
            cudaSetDevice(pd->engine->device);
            if (!cuda_ok(cudaMalloc(&p->scratch, pd->scratch_bytes), "cudaMalloc(scratchpad)")) {
                delete p;
                return dnnl_out_of_memory;
            }
            cudaMemset(p->scratch, 0, pd->scratch_bytes); // arrival counters start at zero
            p->scratch_cap = pd->scratch_bytes;
        }
    }
    *primitive = p;
    if (verbose_level() >= 2) verbose_line("create:cache_miss", p->pd, 0.0); // there is no primitive cache
    return dnnl_success;
}

// cache blobs exist for the OpenCL / Level-Zero engines only
// (src/common/primitive_iface.cpp:235-237)
dnnl_status_t dnnl_primitive_create_from_cache_blob(dnnl_primitive_t *, const_dnnl_primitive_desc_t, size_t, const uint8_t *) {
    return dnnl_unimplemented;
}
dnnl_status_t dnnl_primitive_get_cache_blob(const_dnnl_primitive_t, size_t *, uint8_t *) { return dnnl_unimplemented; }

dnnl_status_t dnnl_primitive_get_primitive_desc(const_dnnl_primitive_t primitive, const_dnnl_primitive_desc_t *pd) {
    if (!primitive || !pd) return dnnl_invalid_arguments;
    *pd = &primitive->pd;
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_destroy(dnnl_primitive_t primitive) {
    if (primitive && primitive->scratch) cudaFree(primitive->scratch);
    delete primitive;
    return dnnl_success;
}

} // extern "C"

// ---------------------------------------------------------------- execution
namespace {

struct arg_map_t {
    const dnnl_exec_arg_t *args;
    int n;
    dnnl_memory_t find(int key) const {
        for (int i = 0; i < n; ++i)
            if (args[i].arg == key) return args[i].memory;
        return nullptr;
    }
};

// fills one QParam; `two_d_mask` maps the tensor's mask to (dim0, dim1) bits
dnnl_status_t bind_quant(QParam &q, const quant_entry_t &e, dnnl_memory_t mem, int lead_dims, dnnl_dim_t d1,
        dnnl_dim_t gstride_rows) {
    q = QParam {};
    q.g0 = q.g1 = 1;
    if (!e.set) return dnnl_success;
    if (!mem) return dnnl_invalid_arguments; // the attribute promises a buffer at execution time
    q.dt = e.dt;
    q.mask = (e.mask >> lead_dims) & 3;
    if (e.group_ndims) { q.g0 = e.groups[0]; q.g1 = e.groups[1]; }
    q.ld = (q.mask & 2) ? d1 / q.g1 : 1;
    q.gstride = gstride_rows * q.ld;
    if (e.on_host) {
        if (!mem->is_host_scalar) return dnnl_invalid_arguments;
        q.on_host = 1;
        switch (e.dt) {
            case dnnl_f32: { float v; memcpy(&v, &mem->host_scalar, 4); q.host_value = v; } break;
            case dnnl_s32: { int v; memcpy(&v, &mem->host_scalar, 4); q.host_value = (float)v; } break;
            default: return dnnl_unimplemented;
        }
        return dnnl_success;
    }
    if (mem->is_host_scalar) return dnnl_invalid_arguments;
    q.ptr = mem->handles[0];
    if (!q.ptr) return dnnl_invalid_arguments;
    return dnnl_success;
}

} // namespace

// One 2D (or grouped) problem: `pd` holds two-dimensional descriptors; a descriptor's offset0 says
// where in the buffer its matrix begins (sub-memories, and the matrices of a batch).
static dnnl_status_t execute_matmul_2d(const_dnnl_primitive_t primitive, const dnnl_primitive_desc &pd,
        dnnl_stream_t stream, arg_map_t &am, int nargs, const dnnl_exec_arg_t *args) {
    const auto &attr = pd.attr;

    dnnl_memory_t src = am.find(DNNL_ARG_SRC), wei = am.find(DNNL_ARG_WEIGHTS), dst = am.find(DNNL_ARG_DST);
    dnnl_memory_t bias = am.find(DNNL_ARG_BIAS);
    if (!src || !wei || !dst) return dnnl_invalid_arguments;
    if ((pd.bias.ndims != 0) != (bias != nullptr)) return dnnl_invalid_arguments;
    // the number of inputs must match what the descriptor expects:
    // src, weights, [bias], one src1 per binary post-op
    int n_in = 0;
    for (int i = 0; i < nargs; ++i) {
        const int a = args[i].arg;
        if (a == DNNL_ARG_SRC || a == DNNL_ARG_WEIGHTS || a == DNNL_ARG_BIAS) ++n_in;
        if (a >= DNNL_ARG_ATTR_MULTIPLE_POST_OP_BASE && (a & 0xff) == DNNL_ARG_SRC_1) ++n_in;
    }
    int expect_in = 2 + (pd.bias.ndims != 0);
    for (const auto &e : attr.post_ops.entries) expect_in += e.kind == dnnl_binary;
    if (n_in != expect_in) return dnnl_invalid_arguments;

    // a descriptor made by dnnl_memory_desc_create_submemory starts offset0 elements into the buffer
    auto at_offset0 = [](void *h, const dnnl_memory_desc &md) -> void * {
        return h && md.offset0 ? (char *)h + md.offset0 * (dnnl_dim_t)dt_bits(md.data_type) / 8 : h;
    };
    MatmulArgs a {};
    a.M = pd.M(); a.N = pd.N(); a.K = pd.K();
    a.src = at_offset0(src->handles[0], pd.src); a.src_dt = pd.src.data_type;
    a.src_sm = pd.src.strides[0]; a.src_sk = pd.src.strides[1];
    a.wei = at_offset0(wei->handles[0], pd.wei); a.wei_dt = pd.wei.data_type;
    a.dst = at_offset0(dst->handles[0], pd.dst); a.dst_dt = pd.dst.data_type;
    a.dst_sm = pd.dst.strides[0]; a.dst_sn = pd.dst.strides[1];
    const int wl = pd.grouped ? 1 : 0; // leading (expert) dim of the weights
    a.wei_sk = pd.wei.strides[wl + 0]; a.wei_sn = pd.wei.strides[wl + 1];
    a.wei_sg = pd.grouped ? pd.wei.strides[0] : 0;
    if (bias) {
        a.bias = at_offset0(bias->handles[0], pd.bias); a.bias_dt = pd.bias.data_type;
        if (pd.grouped) { a.bias_sg = pd.bias.strides[0]; a.bias_sn = 1; }
        else {
            a.bias_sm = pd.bias.dims[0] > 1 ? pd.bias.strides[0] : 0;
            a.bias_sn = pd.bias.dims[1] > 1 ? pd.bias.strides[1] : 0;
        }
        if (!a.bias) return dnnl_invalid_arguments;
    }
    const bool empty = pd.src.has_zero_dim() || pd.wei.has_zero_dim() || pd.dst.has_zero_dim();
    if (!empty && (!a.src || !a.wei || !a.dst)) return dnnl_invalid_arguments;

    dnnl_status_t st;
#define BIND(field, map_get, key, lead, d1, gs) \
    st = bind_quant(a.field, attr.map_get, am.find(key), lead, d1, gs); \
    if (st != dnnl_success) return st;
    const dnnl_dim_t K = a.K, N = a.N;
    BIND(src_scale, scale(DNNL_ARG_SRC), DNNL_ARG_ATTR_SCALES | DNNL_ARG_SRC, 0, K, 0)
    BIND(wei_scale, scale(DNNL_ARG_WEIGHTS), DNNL_ARG_ATTR_SCALES | DNNL_ARG_WEIGHTS, wl, N,
            attr.scale(DNNL_ARG_WEIGHTS).group_ndims ? K / attr.scale(DNNL_ARG_WEIGHTS).groups[0] : 1)
    BIND(dst_scale, scale(DNNL_ARG_DST), DNNL_ARG_ATTR_SCALES | DNNL_ARG_DST, 0, N, 0)
    BIND(src_zp, zp(DNNL_ARG_SRC), DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_SRC, 0, K, 0)
    BIND(wei_zp, zp(DNNL_ARG_WEIGHTS), DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_WEIGHTS, wl, N,
            attr.zp(DNNL_ARG_WEIGHTS).group_ndims ? K / attr.zp(DNNL_ARG_WEIGHTS).groups[0] : 1)
    BIND(dst_zp, zp(DNNL_ARG_DST), DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_DST, 0, N, 0)
    BIND(src_pr, pr(DNNL_ARG_SRC), DNNL_ARG_ATTR_PRECOMPUTED_REDUCTIONS | DNNL_ARG_SRC, 0, K, 0)
#undef BIND
    // host-side zero-points become device-free constants only for scales;
    // integer host scalars are not supported by the kernels
    if (a.src_zp.on_host || a.wei_zp.on_host || a.dst_zp.on_host) return dnnl_unimplemented;

    a.apply_to_int = attr.apply_to_int;
    a.non_default_attr = !attr.has_default_values();
    a.sum_dt = pd.dst.data_type;
    a.n_po = (int)attr.post_ops.entries.size();
    for (int i = 0; i < a.n_po; ++i) {
        const auto &e = attr.post_ops.entries[i];
        PostOpArg &po = a.po[i];
        po = PostOpArg {};
        po.alg = e.alg; po.alpha = e.alpha; po.beta = e.beta; po.scale = e.scale; po.zero_point = e.zero_point;
        if (e.kind == dnnl_sum) { po.kind = PO_SUM; a.sum_dt = e.sum_dt; }
        else if (e.kind == dnnl_eltwise) po.kind = PO_ELTWISE;
        else if (e.kind == dnnl_binary || e.kind == dnnl_prelu) {
            po.kind = PO_BINARY;
            const bool prelu = e.kind == dnnl_prelu; // a binary operation on the weights tensor
            if (prelu) po.alg = ALG_PRELU;
            dnnl_memory_t m = am.find(DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | (prelu ? DNNL_ARG_WEIGHTS : DNNL_ARG_SRC_1));
            if (!m || !m->handles[0]) return dnnl_invalid_arguments;
            po.src1 = at_offset0(m->handles[0], e.src1);
            po.src1_dt = e.src1.data_type;
            po.sm = e.src1.dims[0] > 1 ? e.src1.strides[0] : 0;
            po.sn = e.src1.dims[1] > 1 ? e.src1.strides[1] : 0;
            if (pd.grouped && e.src1.dims[0] == pd.dst.group_count && e.src1.dims[1] == 1
                    && e.src1.dims[0] != pd.dst.dims[0]) {
                po.per_group = 1;
                po.sm = 1;
            }
        } else return dnnl_unimplemented;
    }
    if (pd.grouped) {
        a.group_count = (int)pd.src.group_count;
        a.offsets = (const int32_t *)src->handles[1];
        a.dst_offsets = (const int32_t *)dst->handles[1];
        if (!a.offsets || !a.dst_offsets) return dnnl_invalid_arguments;
    }
    a.status = pd.engine->status_word;
    if (empty) return dnnl_success; // nothing to compute (the reference returns early too)
    if (pd.engine->device < 0) {
        set_last_error("a device-less engine cannot execute primitives");
        return dnnl_runtime_error;
    }

    cudaSetDevice(pd.engine->device);
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    const bool verbose = verbose_level() >= 1;
    if (verbose) {
        cudaEventCreate(&ev0); cudaEventCreate(&ev1);
        cudaEventRecord(ev0, stream->stream);
    }
    profiling_begin(stream);
    void *scratch = primitive->scratch;
    if (pd.scratch_bytes && pd.attr.scratchpad_mode == dnnl_scratchpad_mode_user) {
        dnnl_memory_t sp = am.find(DNNL_ARG_SCRATCHPAD);
        if (!sp || !sp->handles[0]) return dnnl_invalid_arguments;
        scratch = sp->handles[0];
    }
    int rc;
    switch (pd.impl) {
        case IMPL_REF: rc = launch_ref(a, stream->stream); break;
        case IMPL_WOQ_TC:
            if (!woq_tc_pointers_ok(a)) {
                rc = launch_ref(a, stream->stream); // misaligned user pointers: generic kernel
            } else {
                if (pd.attr.scratchpad_mode == dnnl_scratchpad_mode_user) // counters of a user buffer
                    cudaMemsetAsync(scratch, 0, ((pd.N() + 255) / 256) * sizeof(int), stream->stream);
                rc = launch_woq_tc(a, scratch, pd.engine->sm_count, stream->stream);
            }
            break;
        case IMPL_WOQ_GEMV:
            if ((uintptr_t)a.wei % 16 || (uintptr_t)a.src % 4 || (uintptr_t)a.wei_scale.ptr % 16
                    || (a.wei_zp.ptr && (uintptr_t)a.wei_zp.ptr % 16)) {
                rc = launch_ref(a, stream->stream); // misaligned user pointers: generic kernel
            } else {
                if (pd.attr.scratchpad_mode == dnnl_scratchpad_mode_user) // counters of a user buffer
                    cudaMemsetAsync(scratch, 0, ((pd.N() + 255) / 256) * sizeof(int), stream->stream);
                rc = launch_woq_skinny(a, scratch, pd.engine->sm_count, stream->stream);
            }
            break;
        case IMPL_GROUPED_TC:
            if (!grouped_tc_pointers_ok(a)) rc = launch_ref(a, stream->stream);
            else rc = launch_grouped_tc(a, scratch, pd.engine->sm_count, stream->stream);
            break;
        case IMPL_TCGEN05_GEMM:
            // TMA needs 16-byte aligned base pointers; a misaligned user
            // pointer is served by the generic kernel instead
            if (primitive->peers.count) {
                // replicated dst: the memory must lie in this rank's buffer, so that the same offset
                // exists in every peer's; the generic kernel does not replicate
                const char *d = (const char *)a.dst;
                if (d < primitive->peers_own_base || d >= primitive->peers_own_base + primitive->peers_bytes
                        || !gemm_tc_pointers_ok(a)) {
                    set_last_error("replicated dst: the dst memory is outside the registered buffer or misaligned");
                    return dnnl_invalid_arguments;
                }
                a.peers = primitive->peers;
            }
            if (!gemm_tc_pointers_ok(a)) rc = launch_ref(a, stream->stream);
            else rc = launch_gemm_tc(a, scratch, pd.engine->sm_count, stream->stream);
            break;
        default: rc = dnnl_unimplemented;
    }
    profiling_end(stream);
    if (verbose) {
        cudaEventRecord(ev1, stream->stream);
        cudaEventSynchronize(ev1);
        float ms = 0;
        cudaEventElapsedTime(&ms, ev0, ev1);
        cudaEventDestroy(ev0); cudaEventDestroy(ev1);
        verbose_line("exec", pd, ms); // device time of the primitive's kernels
    }
    if (rc == 5) { // a launcher that saw the CUDA error itself has recorded it already
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) set_last_error(std::string("kernel launch: ") + cudaGetErrorString(e));
    }
    return (dnnl_status_t)rc;
}

extern "C" dnnl_status_t dnnl_primitive_execute(const_dnnl_primitive_t primitive, dnnl_stream_t stream, int nargs,
        const dnnl_exec_arg_t *args) {
    if (!primitive || !stream || nargs < 0 || (nargs > 0 && !args)) return dnnl_invalid_arguments;
    if (stream->engine != primitive->pd.engine && stream->engine->device != primitive->pd.engine->device)
        return dnnl_invalid_arguments;
    for (int i = 0; i < nargs; ++i)
        if (!args[i].memory) return dnnl_invalid_arguments;
    if (primitive->pd.kind == dnnl_reorder) return execute_reorder(primitive->pd, stream, nargs, args);
    arg_map_t am {args, nargs};
    // A primitive created with dims left open takes them from the memory objects: every descriptor
    // must agree with what the primitive descriptor does state (rank, data type, the known dims);
    // then the shapes are checked together and the implementation (and its scratch) chosen.
    dnnl_primitive_desc settled;
    if (primitive->pd.runtime_m) {
        settled = primitive->pd;
        settled.runtime_m = false;
        auto take = [&](dnnl_memory_desc &want, int arg) -> bool {
            dnnl_memory_t m = am.find(arg);
            if (!m) return false;
            const dnnl_memory_desc &got = m->md;
            if (got.ndims != want.ndims || got.has_runtime_dims() || got.data_type != want.data_type
                    || got.format_kind != dnnl_blocked)
                return false;
            for (int d = 0; d < want.ndims; ++d)
                if (want.dims[d] != DNNL_RUNTIME_DIM_VAL && want.dims[d] != got.dims[d]) return false;
            want = got;
            return true;
        };
        if (!take(settled.src, DNNL_ARG_SRC) || !take(settled.wei, DNNL_ARG_WEIGHTS) || !take(settled.dst, DNNL_ARG_DST))
            return dnnl_invalid_arguments;
        if (settled.bias.ndims && !take(settled.bias, DNNL_ARG_BIAS)) return dnnl_invalid_arguments;
        for (size_t i = 0; i < settled.attr.post_ops.entries.size(); ++i) {
            auto &e = settled.attr.post_ops.entries[i];
            if (e.kind == dnnl_binary && e.src1.has_runtime_dims()
                    && !take(e.src1, DNNL_ARG_ATTR_MULTIPLE_POST_OP((int)i) | DNNL_ARG_SRC_1))
                return dnnl_invalid_arguments;
        }
        build_prelu_mds(settled);
        fill_quant_mds(settled);
        dnnl_status_t rst = dense_desc_check(settled.src, settled.wei, settled.bias.ndims ? &settled.bias : nullptr, settled.dst);
        if (rst == dnnl_success) rst = dense_attr_check(settled);
        if (rst == dnnl_success) rst = select_impl(settled, 0);
        if (rst != dnnl_success) return rst;
        if (settled.scratch_bytes > primitive->scratch_cap && settled.engine->device >= 0) {
            cudaSetDevice(settled.engine->device);
            // earlier executions may still use the old buffer: they are in order on this stream
            if (primitive->scratch) {
                cudaStreamSynchronize(stream->stream);
                cudaFree(primitive->scratch);
                primitive->scratch = nullptr;
                primitive->scratch_cap = 0;
            }
            if (!cuda_ok(cudaMalloc(&primitive->scratch, settled.scratch_bytes), "cudaMalloc(scratchpad)"))
                return dnnl_out_of_memory;
            cudaMemsetAsync(primitive->scratch, 0, settled.scratch_bytes, stream->stream);
            primitive->scratch_cap = settled.scratch_bytes;
        }
    }
    if (primitive->pd.batched) {
        // a matmul per matrix of the batch, in order on the stream (they share the scratch)
        const dnnl_primitive_desc &bp = primitive->pd;
        dnnl_primitive_desc core;
        dnnl_status_t bst = batch_core(bp, core);
        if (bst != dnnl_success) return bst;
        core.impl = bp.impl; core.impl_name = bp.impl_name; core.scratch_bytes = bp.scratch_bytes;
        const int nd = bp.dst.ndims, nb = nd - 2;
        dnnl_dim_t count = 1;
        for (int d = 0; d < nb; ++d) count *= bp.dst.dims[d];
        if (bp.dst.has_zero_dim()) count = 0;
        for (dnnl_dim_t b = 0; b < count; ++b) {
            dnnl_dim_t idx[DNNL_MAX_NDIMS], rem = b;
            for (int d = nb - 1; d >= 0; --d) { idx[d] = rem % bp.dst.dims[d]; rem /= bp.dst.dims[d]; }
            auto off = [&](const dnnl_memory_desc &md) {
                dnnl_dim_t o = md.offset0;
                for (int d = 0; d < nb; ++d) o += (md.dims[d] == 1 ? 0 : idx[d]) * md.strides[d];
                return o;
            };
            core.src.offset0 = off(bp.src);
            core.wei.offset0 = off(bp.wei);
            core.dst.offset0 = off(bp.dst);
            if (bp.bias.ndims) core.bias.offset0 = off(bp.bias);
            for (size_t i = 0; i < bp.attr.post_ops.entries.size(); ++i)
                if (bp.attr.post_ops.entries[i].kind == dnnl_binary || bp.attr.post_ops.entries[i].kind == dnnl_prelu)
                    core.attr.post_ops.entries[i].src1.offset0 = off(bp.attr.post_ops.entries[i].src1);
            bst = execute_matmul_2d(primitive, core, stream, am, nargs, args);
            if (bst != dnnl_success) return bst;
        }
        return dnnl_success;
    }
    return execute_matmul_2d(primitive, primitive->pd.runtime_m ? settled : primitive->pd, stream, am, nargs, args);
}
