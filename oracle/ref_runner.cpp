// Drives the UNMODIFIED reference library (oracle/_ref/libdnnl_ref.so, built
// from the oneDNN checkout by oracle/Makefile.ref) through its public C++ API
// on a problem described by qmm_problem_t.  TEST INFRASTRUCTURE ONLY: it is
// used to (a) pin the C restatement in qmm_oracle.c to real reference output,
// (b) generate the fixtures in tests/golden/, (c) time the reference's CPU
// matmul as the benchmark's CPU baseline.  Nothing in the product links to it.
//
// Build (done by oracle/build_oracle.py):
//   g++ -std=c++17 -O2 -fPIC -shared ref_runner.cpp -I<ref>/include
//       -I_ref/include -L_ref -ldnnl_ref -Wl,-rpath,'$ORIGIN' -o _ref/libref_runner.so
#include <chrono>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "oneapi/dnnl/dnnl.hpp"
#include "qmm_oracle.h"

using namespace dnnl;
using dt = memory::data_type;
using dims = memory::dims;

namespace {

dt to_dt(int32_t c) { return static_cast<dt>(c); }

memory make_mem(const memory::desc &md, const engine &eng, const void *p) {
    return memory(md, eng, const_cast<void *>(p));
}

struct built_t {
    matmul prim;
    std::unordered_map<int, memory> args;
    std::string impl;
};

// quant parameter buffer descriptor: dense row-major over the masked dims,
// last two divided by the groups (what primitive_attr::set_scales documents)
memory::desc quant_md(const qmm_quant_t &q, int64_t d0, int64_t d1) {
    int64_t a = (q.mask & 1) ? d0 / q.g0 : 1;
    int64_t b = (q.mask & 2) ? d1 / q.g1 : 1;
    return memory::desc({a, b}, to_dt(q.dt), memory::format_tag::ab);
}

void add_quant(primitive_attr &attr, std::unordered_map<int, memory> &args,
        const engine &eng, const qmm_quant_t &q, int arg, int kind,
        int64_t d0, int64_t d1, int lead_dims /*grouped weights: 1*/,
        int64_t G) {
    if (!q.ptr) return;
    int mask = 0;
    if (q.mask & 1) mask |= 1 << (lead_dims + 0);
    if (q.mask & 2) mask |= 1 << (lead_dims + 1);
    if (lead_dims) mask |= 1;
    const bool grouped = q.g0 > 1 || q.g1 > 1;
    dims groups = grouped ? dims {q.g0, q.g1} : dims {};
    if (kind == 0)
        attr.set_scales(arg, mask, groups, to_dt(q.dt));
    else if (kind == 1)
        attr.set_zero_points(arg, mask, groups, to_dt(q.dt));
    else
        attr.set_precomputed_reductions(arg, mask, groups, to_dt(q.dt));
    memory::desc md = quant_md(q, d0, d1);
    if (lead_dims) {
        auto d = md.get_dims();
        md = memory::desc({G, d[0], d[1]}, to_dt(q.dt), memory::format_tag::abc);
    }
    const int base = kind == 0 ? DNNL_ARG_ATTR_SCALES
            : kind == 1        ? DNNL_ARG_ATTR_ZERO_POINTS
                               : DNNL_ARG_ATTR_PRECOMPUTED_REDUCTIONS;
    args.emplace(base | arg, make_mem(md, eng, q.ptr));
}

built_t build(const qmm_problem_t &p, const engine &eng, int pin_ref) {
    const bool grouped = p.group_count > 0;
    std::unordered_map<int, memory> args;
    primitive_attr attr;
    if (p.apply_to_int || p.fpmath_mode)
        attr.set_fpmath_mode(static_cast<fpmath_mode>(p.fpmath_mode), p.apply_to_int != 0);

    memory::desc src_md, wei_md, dst_md, bia_md;
    if (grouped) {
        src_md = memory::desc::grouped(
                {p.M, p.K}, to_dt(p.src_dt), 0, p.group_count);
        dst_md = memory::desc::grouped(
                {p.M, p.N}, to_dt(p.dst_dt), 0, p.group_count);
        wei_md = memory::desc({p.group_count, p.K, p.N}, to_dt(p.wei_dt),
                dims {p.wei_sg, p.wei_sk, p.wei_sn});
        if (p.bias)
            bia_md = memory::desc({p.group_count, p.N}, to_dt(p.bias_dt),
                    memory::format_tag::ab);
    } else {
        src_md = memory::desc(
                {p.M, p.K}, to_dt(p.src_dt), dims {p.src_sm, p.src_sk});
        wei_md = memory::desc(
                {p.K, p.N}, to_dt(p.wei_dt), dims {p.wei_sk, p.wei_sn});
        dst_md = memory::desc(
                {p.M, p.N}, to_dt(p.dst_dt), dims {p.dst_sm, p.dst_sn});
        if (p.bias)
            bia_md = memory::desc({p.bias_sm ? p.M : 1, p.bias_sn ? p.N : 1},
                    to_dt(p.bias_dt), memory::format_tag::ab);
    }

    add_quant(attr, args, eng, p.src_scale, DNNL_ARG_SRC, 0, p.M, p.K, 0, 0);
    add_quant(attr, args, eng, p.wei_scale, DNNL_ARG_WEIGHTS, 0, p.K, p.N,
            grouped ? 1 : 0, p.group_count);
    add_quant(attr, args, eng, p.dst_scale, DNNL_ARG_DST, 0, p.M, p.N, 0, 0);
    add_quant(attr, args, eng, p.src_zp, DNNL_ARG_SRC, 1, p.M, p.K, 0, 0);
    add_quant(attr, args, eng, p.wei_zp, DNNL_ARG_WEIGHTS, 1, p.K, p.N,
            grouped ? 1 : 0, p.group_count);
    add_quant(attr, args, eng, p.dst_zp, DNNL_ARG_DST, 1, p.M, p.N, 0, 0);
    add_quant(attr, args, eng, p.src_pr, DNNL_ARG_SRC, 2, p.M, p.K, 0, 0);

    post_ops po;
    for (int i = 0; i < p.n_po; ++i) {
        const qmm_postop_t &e = p.po[i];
        if (e.kind == QMM_PO_SUM) {
            po.append_sum(e.scale, e.zero_point, to_dt(p.sum_dt));
        } else if (e.kind == QMM_PO_ELTWISE) {
            po.append_eltwise(static_cast<algorithm>(e.alg), e.alpha, e.beta);
        } else if (e.kind == QMM_PO_PRELU) {
            memory::desc md({e.src1_sm ? p.M : 1, e.src1_sn ? p.N : 1},
                    memory::data_type::f32, memory::format_tag::ab);
            po.append_prelu((e.src1_sm ? 1 : 0) | (e.src1_sn ? 2 : 0));
            args.emplace(DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_WEIGHTS,
                    make_mem(md, eng, e.src1));
        } else {
            memory::desc md({e.src1_sm ? p.M : 1, e.src1_sn ? p.N : 1},
                    to_dt(e.src1_dt), memory::format_tag::ab);
            po.append_binary(static_cast<algorithm>(e.alg), md);
            args.emplace(DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_SRC_1,
                    make_mem(md, eng, e.src1));
        }
    }
    if (p.n_po) attr.set_post_ops(po);

    matmul::primitive_desc pd = p.bias
            ? matmul::primitive_desc(eng, src_md, wei_md, bia_md, dst_md, attr)
            : matmul::primitive_desc(eng, src_md, wei_md, dst_md, attr);
    if (pin_ref) {
        // walk the implementation list until a scalar reference one
        while (std::string(pd.impl_info_str()).rfind("ref", 0) != 0)
            if (!pd.next_impl()) throw error(dnnl_unimplemented, "no ref impl");
    }

    if (grouped) {
        void *sh[2] = {const_cast<void *>(p.src), const_cast<int32_t *>(p.offsets)};
        void *dh[2] = {p.dst, const_cast<int32_t *>(p.offsets)};
        args.emplace(DNNL_ARG_SRC,
                memory(src_md, eng, std::vector<void *>(sh, sh + 2)));
        args.emplace(DNNL_ARG_DST,
                memory(dst_md, eng, std::vector<void *>(dh, dh + 2)));
    } else {
        args.emplace(DNNL_ARG_SRC, make_mem(src_md, eng, p.src));
        args.emplace(DNNL_ARG_DST, make_mem(dst_md, eng, p.dst));
    }
    args.emplace(DNNL_ARG_WEIGHTS, make_mem(wei_md, eng, p.wei));
    if (p.bias) args.emplace(DNNL_ARG_BIAS, make_mem(bia_md, eng, p.bias));

    built_t b {matmul(pd), std::move(args), pd.impl_info_str()};
    return b;
}

} // namespace

extern "C" {

// Runs the problem on the reference CPU engine.
//   pin_ref != 0 : use the scalar ref* implementation (the parity oracle)
//   pin_ref == 0 : use the first implementation the library dispatches
// iters > 0 additionally times `iters` executions after one warm-up and
// stores the best wall time in *best_ms.  The implementation name is copied
// into impl_name.  Returns 0, or the dnnl status code of the failing call.
int ref_runner_run(const qmm_problem_t *p, int pin_ref, int iters,
        double *best_ms, char *impl_name, int impl_len) {
    try {
        engine eng(engine::kind::cpu, 0);
        stream s(eng);
        built_t b = build(*p, eng, pin_ref);
        if (impl_name && impl_len > 0) {
            std::strncpy(impl_name, b.impl.c_str(), impl_len - 1);
            impl_name[impl_len - 1] = 0;
        }
        b.prim.execute(s, b.args);
        s.wait();
        if (iters > 0 && best_ms) {
            double best = 1e30;
            for (int i = 0; i < iters; ++i) {
                auto t0 = std::chrono::steady_clock::now();
                b.prim.execute(s, b.args);
                s.wait();
                auto t1 = std::chrono::steady_clock::now();
                double ms = std::chrono::duration<double, std::milli>(t1 - t0)
                                    .count();
                if (ms < best) best = ms;
            }
            *best_ms = best;
        }
        return 0;
    } catch (const error &e) {
        if (impl_name && impl_len > 0) {
            std::strncpy(impl_name, e.message, impl_len - 1);
            impl_name[impl_len - 1] = 0;
        }
        return e.status ? (int)e.status : -1;
    }
}

// ---- problems with batch dims ----------------------------------------------
// A matmul of any rank, described by plain tensors (dims and element strides): the batched
// problems of the tests, whose matrices the 2D restatement computes one by one.  The reference
// decides the broadcast of size-1 batch dims, the layout of prelu weights and the meaning of
// masks over batch dims; this entry point lets the tests ask it.
#define QMM_ND_MAX 6
typedef struct {
    const void *ptr; // null: absent
    int32_t dt, ndims;
    int64_t dims[QMM_ND_MAX], strides[QMM_ND_MAX];
} qmm_nd_tensor_t;
typedef struct {
    const void *ptr;
    int32_t dt, mask, arg /* DNNL_ARG_SRC / WEIGHTS / DST */, kind /* 0 scales, 1 zero-points */;
    int64_t g0, g1;
} qmm_nd_quant_t;
typedef struct {
    int32_t kind /* QMM_PO_* */, alg, zero_point, mask /* prelu */;
    float alpha, beta, scale;
    qmm_nd_tensor_t src1; // binary operand; prelu: ptr only (f32, the layout the library defines)
} qmm_nd_postop_t;
typedef struct {
    qmm_nd_tensor_t src, wei, dst, bias;
    int32_t n_quant, n_po, apply_to_int, fpmath_mode;
    qmm_nd_quant_t quant[8];
    qmm_nd_postop_t po[8];
} qmm_nd_problem_t;

static memory::desc nd_md(const qmm_nd_tensor_t &t) {
    return memory::desc(dims(t.dims, t.dims + t.ndims), to_dt(t.dt), dims(t.strides, t.strides + t.ndims));
}

int ref_runner_run_nd(const qmm_nd_problem_t *p, int pin_ref, char *impl_name, int impl_len) {
    try {
        engine eng(engine::kind::cpu, 0);
        stream s(eng);
        std::unordered_map<int, memory> args;
        primitive_attr attr;
        if (p->apply_to_int || p->fpmath_mode)
            attr.set_fpmath_mode(static_cast<fpmath_mode>(p->fpmath_mode), p->apply_to_int != 0);
        const memory::desc src_md = nd_md(p->src), wei_md = nd_md(p->wei), dst_md = nd_md(p->dst);
        const int nd = p->dst.ndims;
        for (int i = 0; i < p->n_quant; ++i) {
            const qmm_nd_quant_t &q = p->quant[i];
            const qmm_nd_tensor_t &base = q.arg == DNNL_ARG_SRC ? p->src : q.arg == DNNL_ARG_WEIGHTS ? p->wei : p->dst;
            const bool grouped = q.g0 > 1 || q.g1 > 1;
            dims groups = grouped ? dims {q.g0, q.g1} : dims {};
            if (q.kind == 0) attr.set_scales(q.arg, q.mask, groups, to_dt(q.dt));
            else attr.set_zero_points(q.arg, q.mask, groups, to_dt(q.dt));
            dims qd(nd, 1);
            for (int d = 0; d < nd; ++d)
                if ((q.mask >> d) & 1) qd[d] = base.dims[d];
            qd[nd - 2] /= (q.mask >> (nd - 2)) & 1 ? q.g0 : 1;
            qd[nd - 1] /= (q.mask >> (nd - 1)) & 1 ? q.g1 : 1;
            dims qs(nd, 1);
            for (int d = nd - 2; d >= 0; --d) qs[d] = qs[d + 1] * qd[d + 1];
            args.emplace((q.kind == 0 ? DNNL_ARG_ATTR_SCALES : DNNL_ARG_ATTR_ZERO_POINTS) | q.arg,
                    make_mem(memory::desc(qd, to_dt(q.dt), qs), eng, q.ptr));
        }
        post_ops po;
        for (int i = 0; i < p->n_po; ++i) {
            const qmm_nd_postop_t &e = p->po[i];
            if (e.kind == QMM_PO_SUM) po.append_sum(e.scale, e.zero_point);
            else if (e.kind == QMM_PO_ELTWISE) po.append_eltwise(static_cast<algorithm>(e.alg), e.alpha, e.beta);
            else if (e.kind == QMM_PO_PRELU) po.append_prelu(e.mask);
            else po.append_binary(static_cast<algorithm>(e.alg), nd_md(e.src1));
        }
        if (p->n_po) attr.set_post_ops(po);
        matmul::primitive_desc pd = p->bias.ptr
                ? matmul::primitive_desc(eng, src_md, wei_md, nd_md(p->bias), dst_md, attr)
                : matmul::primitive_desc(eng, src_md, wei_md, dst_md, attr);
        if (pin_ref)
            while (std::string(pd.impl_info_str()).rfind("ref", 0) != 0)
                if (!pd.next_impl()) throw error(dnnl_unimplemented, "no ref impl");
        for (int i = 0; i < p->n_po; ++i) {
            const qmm_nd_postop_t &e = p->po[i];
            if (e.kind == QMM_PO_BINARY)
                args.emplace(DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_SRC_1, make_mem(nd_md(e.src1), eng, e.src1.ptr));
            else if (e.kind == QMM_PO_PRELU) {
                // the library states the weights' descriptor: dims masked, its own dense layout
                memory::desc wmd = pd.query_md(query::exec_arg_md, DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_WEIGHTS);
                if (wmd.get_ndims() == 0) { // not answered: ab, acb, acdb, acdeb (src/cpu/primitive_attr_postops.cpp:219-242)
                    dims wd(nd, 1);
                    for (int d = 0; d < nd; ++d)
                        if ((e.mask >> d) & 1) wd[d] = p->dst.dims[d];
                    static const memory::format_tag tags[] = {memory::format_tag::a, memory::format_tag::ab,
                            memory::format_tag::acb, memory::format_tag::acdb, memory::format_tag::acdeb};
                    if (nd > 5) throw error(dnnl_unimplemented, "prelu beyond five dims");
                    wmd = memory::desc(wd, dt::f32, tags[nd - 1]);
                }
                args.emplace(DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_WEIGHTS, make_mem(wmd, eng, e.src1.ptr));
            }
        }
        args.emplace(DNNL_ARG_SRC, make_mem(src_md, eng, p->src.ptr));
        args.emplace(DNNL_ARG_WEIGHTS, make_mem(wei_md, eng, p->wei.ptr));
        args.emplace(DNNL_ARG_DST, make_mem(dst_md, eng, p->dst.ptr));
        if (p->bias.ptr) args.emplace(DNNL_ARG_BIAS, make_mem(nd_md(p->bias), eng, p->bias.ptr));
        if (impl_name && impl_len > 0) {
            std::strncpy(impl_name, pd.impl_info_str(), impl_len - 1);
            impl_name[impl_len - 1] = 0;
        }
        matmul(pd).execute(s, args);
        s.wait();
        return 0;
    } catch (const error &e) {
        if (impl_name && impl_len > 0) {
            std::strncpy(impl_name, e.message, impl_len - 1);
            impl_name[impl_len - 1] = 0;
        }
        return e.status ? (int)e.status : -1;
    }
}

// Runs a reorder on the reference CPU engine (whatever implementation the
// library dispatches; the reorder primitive descriptor has no iterator).
int ref_runner_reorder(const qmm_reorder_t *r, char *impl_name, int impl_len) {
    try {
        engine eng(engine::kind::cpu, 0);
        stream s(eng);
        dims d(r->dims, r->dims + r->ndims);
        memory::desc src_md(d, to_dt(r->src_dt), dims(r->src_strides, r->src_strides + r->ndims));
        memory::desc dst_md(d, to_dt(r->dst_dt), dims(r->dst_strides, r->dst_strides + r->ndims));
        primitive_attr attr;
        std::unordered_map<int, memory> args;
        auto quant = [&](const qmm_rquant_t &q, int arg, bool zp) {
            if (!q.ptr) return;
            const bool grouped = q.g0 > 1 || q.g1 > 1;
            dims groups = grouped ? dims {q.g0, q.g1} : dims {};
            if (zp) attr.set_zero_points(arg, q.mask, groups, to_dt(q.dt));
            else attr.set_scales(arg, q.mask, groups, to_dt(q.dt));
            dims qd(r->ndims, 1);
            for (int i = 0; i < r->ndims; ++i)
                if ((q.mask >> i) & 1) qd[i] = r->dims[i];
            if (r->ndims >= 2) {
                qd[r->ndims - 1] /= ((q.mask >> (r->ndims - 1)) & 1) ? q.g1 : 1;
                qd[r->ndims - 2] /= ((q.mask >> (r->ndims - 2)) & 1) ? q.g0 : 1;
            }
            dims qs(r->ndims, 1);
            for (int i = r->ndims - 2; i >= 0; --i) qs[i] = qs[i + 1] * qd[i + 1];
            memory::desc md(qd, to_dt(q.dt), qs);
            args.emplace((zp ? DNNL_ARG_ATTR_ZERO_POINTS : DNNL_ARG_ATTR_SCALES) | arg, make_mem(md, eng, q.ptr));
        };
        quant(r->src_scale, DNNL_ARG_SRC, false);
        quant(r->dst_scale, DNNL_ARG_DST, false);
        quant(r->src_zp, DNNL_ARG_SRC, true);
        quant(r->dst_zp, DNNL_ARG_DST, true);
        if (r->beta != 0.f) {
            post_ops po;
            po.append_sum(r->beta);
            attr.set_post_ops(po);
        }
        reorder::primitive_desc pd(eng, src_md, eng, dst_md, attr);
        if (impl_name && impl_len > 0) {
            std::strncpy(impl_name, pd.impl_info_str(), impl_len - 1);
            impl_name[impl_len - 1] = 0;
        }
        args.emplace(DNNL_ARG_FROM, make_mem(src_md, eng, r->src));
        args.emplace(DNNL_ARG_TO, make_mem(dst_md, eng, r->dst));
        reorder(pd).execute(s, args);
        s.wait();
        return 0;
    } catch (const error &e) {
        if (impl_name && impl_len > 0) {
            std::strncpy(impl_name, e.message, impl_len - 1);
            impl_name[impl_len - 1] = 0;
        }
        return e.status ? (int)e.status : -1;
    }
}

} // extern "C"
