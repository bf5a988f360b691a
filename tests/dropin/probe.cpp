// A program written against the reference's unchanged dnnl.hpp: builds the
// primitive descriptors of the quantized matmul workloads on the CUDA engine
// and prints the implementation each one gets.  Nothing executes, so it also
// runs on a device-less engine (DNNL_B200_NO_DEVICE=1).
#include <iostream>
#include <vector>

#include "oneapi/dnnl/dnnl.hpp"

using namespace dnnl;
using dt = memory::data_type;
using tag = memory::format_tag;

int main() {
    if (engine::get_count(engine::kind::cpu) != 0) return 2; // there is no CPU engine in this library
    engine eng(engine::kind::gpu, 0);
    stream strm(eng);

    { // int8 with a src zero-point, s32 dst
        memory::desc src({256, 1024}, dt::u8, tag::ab), wei({1024, 1024}, dt::s8, tag::ab),
                dst({256, 1024}, dt::s32, tag::ab);
        primitive_attr attr;
        attr.set_zero_points_mask(DNNL_ARG_SRC, 0);
        matmul::primitive_desc pd(eng, src, wei, dst, attr);
        std::cout << "int8_zp " << pd.impl_info_str() << "\n";
    }
    { // fp8 prefill with per-tensor scales and a bf16 bias
        memory::desc src({512, 512}, dt::f8_e4m3, tag::ab), wei({512, 1024}, dt::f8_e4m3, tag::ab),
                bias({1, 1024}, dt::bf16, tag::ab), dst({512, 1024}, dt::bf16, tag::ab);
        primitive_attr attr;
        attr.set_scales_mask(DNNL_ARG_SRC, 0);
        attr.set_scales_mask(DNNL_ARG_WEIGHTS, 0);
        matmul::primitive_desc pd(eng, src, wei, bias, dst, attr);
        std::cout << "fp8 " << pd.impl_info_str() << "\n";
    }
    { // int4 weight decompression, grouped scales and zero-points
        memory::desc src({1, 1024}, dt::bf16, tag::ab), wei({1024, 512}, dt::s4, tag::ab),
                dst({1, 512}, dt::bf16, tag::ab);
        primitive_attr attr;
        attr.set_fpmath_mode(fpmath_mode::bf16, true);
        attr.set_scales(DNNL_ARG_WEIGHTS, 3, {128, 1}, dt::bf16);
        attr.set_zero_points(DNNL_ARG_WEIGHTS, 3, {128, 1}, dt::u4);
        matmul::primitive_desc pd(eng, src, wei, dst, attr);
        std::cout << "int4 " << pd.impl_info_str() << "\n";
        // the implementation list ends with the generic kernels
        std::string last = pd.impl_info_str();
        while (pd.next_impl()) last = pd.impl_info_str();
        std::cout << "int4_last " << last << "\n";
    }
    { // int8 with the post-op chain: gelu_tanh, residual add, requantization
        memory::desc src({64, 256}, dt::s8, tag::ab), wei({256, 128}, dt::s8, tag::ab),
                bias({1, 128}, dt::f32, tag::ab), dst({64, 128}, dt::s8, tag::ab), res({64, 128}, dt::f32, tag::ab);
        primitive_attr attr;
        attr.set_scales_mask(DNNL_ARG_SRC, 1 << 0);
        attr.set_scales_mask(DNNL_ARG_WEIGHTS, 1 << 1);
        attr.set_scales_mask(DNNL_ARG_DST, 0);
        attr.set_zero_points_mask(DNNL_ARG_DST, 0);
        post_ops po;
        po.append_eltwise(algorithm::eltwise_gelu_tanh, 0.f, 0.f);
        po.append_binary(algorithm::binary_add, res);
        attr.set_post_ops(po);
        matmul::primitive_desc pd(eng, src, wei, bias, dst, attr);
        std::cout << "int8_postops " << pd.impl_info_str() << "\n";
    }
    { // grouped (MoE): bf16 rows of 8 experts concatenated, s8 weights [G, K, N], one scale per (expert, column)
        const memory::dim G = 8, M = 512, K = 256, N = 384;
        memory::desc src = memory::desc::grouped({M, K}, dt::bf16, 0, G);
        memory::desc dst = memory::desc::grouped({M, N}, dt::bf16, 0, G);
        memory::desc wei({G, K, N}, dt::s8, tag::abc);
        primitive_attr attr;
        attr.set_fpmath_mode(fpmath_mode::bf16, true);
        attr.set_scales_mask(DNNL_ARG_WEIGHTS, (1 << 0) | (1 << 2));
        matmul::primitive_desc pd(eng, src, wei, dst, attr);
        std::cout << "grouped " << pd.impl_info_str() << "\n";
    }
    return 0;
}
