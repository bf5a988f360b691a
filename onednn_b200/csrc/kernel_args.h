// Plain-data description of one matmul execution, passed by value to the
// kernels.  Filled by the primitive at execute time from the primitive
// descriptor (shapes, attributes) and the execution arguments (pointers).
#pragma once
#include <stdint.h>

namespace qmm {

// dnnl_data_type_t values
enum : int {
    DT_UNDEF = 0, DT_F16 = 1, DT_BF16 = 2, DT_F32 = 3, DT_S32 = 4, DT_S8 = 5,
    DT_U8 = 6, DT_F8_E5M2 = 9, DT_F8_E4M3 = 10, DT_S4 = 11, DT_U4 = 12
};

enum : int { PO_SUM = 1, PO_ELTWISE = 2, PO_BINARY = 3, PO_PRELU = 4 };
// a prelu post-op reaches the kernels as a binary operation on its weights tensor: x >= 0 ? x : w * x
// (no dnnl_alg_kind_t has this value)
constexpr int ALG_PRELU = 0x1ffe0;

constexpr int MAX_POST_OPS = 32;

// One quantization parameter (scale, zero-point or precomputed reduction).
// The buffer is dense row-major over the masked dims of the 2D (M,K), (K,N)
// or (M,N) tensor it belongs to, the two dims divided by their group sizes.
struct QParam {
    const void *ptr; // nullptr: parameter absent
    int dt;
    int mask; // bit0: first dim of the 2D tensor, bit1: second dim
    int64_t g0, g1; // group sizes (>= 1)
    int64_t ld; // row pitch in elements
    int64_t gstride; // grouped matmul: elements between experts (weights)
    float host_value; // value of a host-side scalar (ptr == nullptr, on_host)
    int on_host;
};

struct PostOpArg {
    int kind;
    int alg;
    float alpha, beta, scale;
    int zero_point; // sum
    int src1_dt; // binary
    int per_group; // grouped matmul: src1 is [G,1], indexed by the expert
    const void *src1;
    int64_t sm, sn; // element strides of src1, 0 on a broadcast dim
};

// Replication of dst stores into the same place of other GPUs' buffers (a sharded matmul whose
// full result every rank wants): the kernel repeats each dst store at `delta[i]` bytes from the
// local address, and the last CTA to finish publishes `epoch` in flags[r][rank] of every rank r.
constexpr int MAX_PEERS = 16;
struct PeerReplication {
    int count; // peers stored to besides the local dst (0: off)
    int world, rank;
    unsigned epoch;
    unsigned *done; // local counter of finished CTAs, zero between launches
    long long delta[MAX_PEERS - 1];
    unsigned *flags[MAX_PEERS]; // flag array [world] of every rank, as mapped on this GPU
};

struct MatmulArgs {
    int64_t M, N, K;
    const void *src;
    int src_dt;
    int64_t src_sm, src_sk;
    const void *wei;
    int wei_dt;
    int64_t wei_sk, wei_sn, wei_sg;
    const void *bias;
    int bias_dt;
    int64_t bias_sm, bias_sn, bias_sg;
    void *dst;
    int dst_dt;
    int64_t dst_sm, dst_sn;
    QParam src_scale, wei_scale, dst_scale, src_zp, wei_zp, dst_zp, src_pr;
    int apply_to_int; // weights decompression (fpmath apply_to_int)
    int non_default_attr;
    int sum_dt;
    int n_po;
    PostOpArg po[MAX_POST_OPS];
    // grouped (2D x 3D) problems
    int group_count;
    const int32_t *offsets; // cumulative END row per group, device memory
    const int32_t *dst_offsets;
    // device status word: kernels record errors here instead of trapping
    int *status;
    PeerReplication peers;
};

} // namespace qmm
