// A program written against the reference's unchanged dnnl.hpp that runs on the
// GPU: u8 x s8 -> s32 matmul with a src zero-point (bit-exact against a scalar
// loop on the host), and the same with per-column weight scales, a bias and a
// relu post-op into f32.  Prints "ok" lines; exit code 0 when everything matches.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "oneapi/dnnl/dnnl.hpp"

using namespace dnnl;
using dt = memory::data_type;
using tag = memory::format_tag;

template <typename T>
static void write_to(memory &m, const std::vector<T> &v) {
    void *p = m.map_data();
    std::memcpy(p, v.data(), v.size() * sizeof(T));
    m.unmap_data(p);
}
template <typename T>
static std::vector<T> read_from(memory &m, size_t n) {
    std::vector<T> v(n);
    void *p = m.map_data();
    std::memcpy(v.data(), p, n * sizeof(T));
    m.unmap_data(p);
    return v;
}

int main() {
    const memory::dim M = 100, K = 272, N = 176;
    engine eng(engine::kind::gpu, 0);
    stream strm(eng);
    std::mt19937 rng(7);
    std::vector<uint8_t> src(M * K);
    std::vector<int8_t> wei(K * N);
    std::vector<float> scales(N), bias(N);
    for (auto &x : src) x = (uint8_t)(rng() % 256);
    for (auto &x : wei) x = (int8_t)((int)(rng() % 255) - 127);
    for (auto &x : scales) x = 0.001f + 0.009f * (float)(rng() % 1000) / 1000.f;
    for (auto &x : bias) x = (float)((int)(rng() % 2001) - 1000) / 100.f;
    const int32_t zp = 128;

    memory::desc src_md({M, K}, dt::u8, tag::ab), wei_md({K, N}, dt::s8, tag::ab);
    memory src_m(src_md, eng), wei_m(wei_md, eng);
    write_to(src_m, src);
    write_to(wei_m, wei);
    memory zp_m(memory::desc({1}, dt::s32, tag::x), eng);
    write_to(zp_m, std::vector<int32_t> {zp});

    std::vector<int64_t> acc(M * N);
    for (memory::dim m = 0; m < M; ++m)
        for (memory::dim n = 0; n < N; ++n) {
            int64_t a = 0;
            for (memory::dim k = 0; k < K; ++k) a += ((int)src[m * K + k] - zp) * (int)wei[k * N + n];
            acc[m * N + n] = a;
        }

    int bad = 0;
    { // s32 dst, bit-exact
        memory::desc dst_md({M, N}, dt::s32, tag::ab);
        primitive_attr attr;
        attr.set_zero_points_mask(DNNL_ARG_SRC, 0);
        matmul::primitive_desc pd(eng, src_md, wei_md, dst_md, attr);
        memory dst_m(dst_md, eng);
        matmul(pd).execute(strm, {{DNNL_ARG_SRC, src_m}, {DNNL_ARG_WEIGHTS, wei_m}, {DNNL_ARG_DST, dst_m},
                                         {DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_SRC, zp_m}});
        strm.wait();
        auto got = read_from<int32_t>(dst_m, M * N);
        int wrong = 0;
        for (size_t i = 0; i < got.size(); ++i) wrong += got[i] != (int32_t)acc[i];
        std::printf("s32 %s %s (%d mismatches)\n", pd.impl_info_str(), wrong ? "FAILED" : "ok", wrong);
        bad += wrong;
    }
    { // f32 dst with per-column weight scales, bias and relu
        memory::desc dst_md({M, N}, dt::f32, tag::ab), bias_md({1, N}, dt::f32, tag::ab);
        primitive_attr attr;
        attr.set_zero_points_mask(DNNL_ARG_SRC, 0);
        attr.set_scales_mask(DNNL_ARG_WEIGHTS, 1 << 1);
        post_ops po;
        po.append_eltwise(algorithm::eltwise_relu, 0.f, 0.f);
        attr.set_post_ops(po);
        matmul::primitive_desc pd(eng, src_md, wei_md, bias_md, dst_md, attr);
        memory dst_m(dst_md, eng), bias_m(bias_md, eng), sc_m(memory::desc({N}, dt::f32, tag::x), eng);
        write_to(bias_m, bias);
        write_to(sc_m, scales);
        matmul(pd).execute(strm, {{DNNL_ARG_SRC, src_m}, {DNNL_ARG_WEIGHTS, wei_m}, {DNNL_ARG_BIAS, bias_m},
                                         {DNNL_ARG_DST, dst_m}, {DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_SRC, zp_m},
                                         {DNNL_ARG_ATTR_SCALES | DNNL_ARG_WEIGHTS, sc_m}});
        strm.wait();
        auto got = read_from<float>(dst_m, M * N);
        int wrong = 0;
        for (memory::dim m = 0; m < M; ++m)
            for (memory::dim n = 0; n < N; ++n) {
                float d = (float)acc[m * N + n]; // the reference's order: scale, then bias, then relu
                d *= scales[n];
                d += bias[n];
                d = d > 0.f ? d : 0.f;
                const float g = got[m * N + n];
                if (std::fabs(g - d) > 1e-5f * std::fabs(d) + 1e-30f) ++wrong;
            }
        std::printf("f32 %s %s (%d beyond 1e-5)\n", pd.impl_info_str(), wrong ? "FAILED" : "ok", wrong);
        bad += wrong;
    }
    { // dnnl::reorder: f32 weights -> s8 with one dst scale per column, then back to f32 column-major
        std::vector<float> wf(K * N);
        for (auto &x : wf) x = (float)((int)(rng() % 2001) - 1000) / 400.f;
        memory::desc f_md({K, N}, dt::f32, tag::ab), q_md({K, N}, dt::s8, tag::ab), t_md({K, N}, dt::f32, tag::ba);
        memory f_m(f_md, eng), q_m(q_md, eng), t_m(t_md, eng), sc_m(memory::desc({N}, dt::f32, tag::x), eng);
        write_to(f_m, wf);
        write_to(sc_m, scales);
        primitive_attr qattr, dattr;
        qattr.set_scales_mask(DNNL_ARG_DST, 1 << 1);
        dattr.set_scales_mask(DNNL_ARG_SRC, 1 << 1);
        reorder::primitive_desc qpd(eng, f_md, eng, q_md, qattr);
        reorder(qpd).execute(strm, {{DNNL_ARG_FROM, f_m}, {DNNL_ARG_TO, q_m}, {DNNL_ARG_ATTR_SCALES | DNNL_ARG_DST, sc_m}});
        reorder(reorder::primitive_desc(q_m, t_m, dattr))
                .execute(strm, {{DNNL_ARG_FROM, q_m}, {DNNL_ARG_TO, t_m}, {DNNL_ARG_ATTR_SCALES | DNNL_ARG_SRC, sc_m}});
        strm.wait();
        auto q = read_from<int8_t>(q_m, K * N);
        auto t = read_from<float>(t_m, K * N);
        int wrong = 0;
        for (memory::dim k = 0; k < K; ++k)
            for (memory::dim n = 0; n < N; ++n) {
                float d = wf[k * N + n] / scales[n];
                d = d < -128.f ? -128.f : (d > 127.f ? 127.f : d);
                const int8_t want = (int8_t)std::nearbyintf(d);
                wrong += q[k * N + n] != want;
                wrong += t[n * K + k] != scales[n] * (float)want;
            }
        std::printf("reorder %s %s (%d mismatches)\n", qpd.impl_info_str(), wrong ? "FAILED" : "ok", wrong);
        bad += wrong;
    }
    return bad ? 1 : 0;
}
