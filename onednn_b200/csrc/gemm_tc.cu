// "cuda:tcgen05" GEMM for 8-bit operands: int8 (u8/s8 x u8/s8 -> s32
// accumulate) and fp8 (e4m3/e5m2 -> f32 accumulate).
//
// The kernel computes dst^T tiles: the WEIGHTS are the A operand of
// tcgen05.mma (128 dst columns = the 128 TMEM lanes) and the SRC rows are the
// B operand (BT_M dst rows = TMEM columns).  An epilogue thread therefore owns
// one dst column n and reads consecutive rows m from TMEM: the 32 lanes of a
// warp hold 32 adjacent columns, so every global access of the epilogue (dst
// stores, binary post-op operands) is coalesced without a shared-memory
// transpose, and per-column terms (weight scales, bias, zero-point
// compensation) live in registers for the whole tile.
//
// One persistent CTA per SM walks the tiles.  Roles:
//   warp 0     TMA producer: weights tile ([128 k x 128 n] for N-contiguous
//              `ab` weights, [128 n x 128 B of k] for `ba`) and src tile
//              [BT_M rows x 128 B of k] into a ring of 128B-swizzled stages
//   warp 1     issues tcgen05.mma (M=128, N=BT_M, K=32 per instruction) into
//              one of two TMEM accumulator buffers, commits to mbarriers
//   warps 2-9  epilogue (two warps per TMEM lane quarter, each half of the
//              rows): zero-point compensation, scales, bias, post-op chain,
//              dst scale / zero-point, saturating store; overlaps the next
//              tile's multiplication
// Epilogue arithmetic follows the reference (ref_matmul_int8.cpp:241-304,
// ref_matmul.cpp:218-332): integer sums are exact, so int8 results equal the
// reference's bit for bit; fp8 differs only by the f32 summation order.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>
#include <string>

#include "device_math.cuh"
#include "launch.h"
#include "objects.hpp"
// waits of this kernel are long (a tile's mainloop, a ring that is full): let the hardware hold the
// polling thread for up to this many nanoseconds per poll (measured: 3 % on the fp8 GEMM)
#define QMM_TRY_WAIT_HINT_NS 2000
#include "sm100_ptx.cuh"

namespace qmm {

namespace {

constexpr int BT_N = 128; // dst columns per tile = TMEM lanes = UMMA M
constexpr int BKB = 128; // bytes (= 8-bit elements) of K per stage: one swizzle row
constexpr int UMMA_K = 32; // K per tcgen05.mma for 8-bit operands
// Epilogue warps: 8 keep up with the MMAs when the epilogue is scale + bias + store; a post-op chain
// is latency-bound per element: 16 warps (at 96 registers) hide a third more of it than 8, and 24
// (at 72 registers) another 6 % (int8 post-op workload: 12 warps 150 us, 16: 133, 20: 132, 24: 124-127).
#ifndef QMM_CHAIN_EPI_WARPS
#define QMM_CHAIN_EPI_WARPS 24
#endif
#ifndef QMM_CHAIN_CR
#define QMM_CHAIN_CR 8
#endif
constexpr int epi_warps(bool chain) { return chain ? QMM_CHAIN_EPI_WARPS : 8; }
constexpr int num_threads(bool chain) { return 64 + 32 * epi_warps(chain); }

struct TcParams {
    int num_m_tiles, num_n_tiles, num_k_blocks;
    uint32_t idesc;
    int w_kmajor; // weights are `ba` (K contiguous)
#ifdef QMM_PROFILE
    int mainloop_only; // 1 no epilogue, 2 TMEM reads only, 3 everything but the stores, 4 binary operands read from one address (wrong results)
#endif
    int after_prekernel; // launched as the programmatic dependent of the column / row sum kernel before it
    const int32_t *colsum; // sum_k w[k][n]       (src zero-point compensation)
    const int32_t *rowsum; // sum_k s[m][k]       (weights zero-point compensation)
};

template <int BT_M, int STAGES>
struct SmemLayout {
    static constexpr int W_BYTES = BT_N * BKB;
    static constexpr int S_BYTES = BT_M * BKB;
    static constexpr int STAGE_BYTES = W_BYTES + S_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BAR_OFFSET + 256 + 1024; // barriers + alignment slack
};

// Per-column terms of the epilogue, in registers of the thread that owns the column.
struct ColTerms {
    float wei_scale; // 1 when absent
    float bias; // bias[n] when the bias is a row vector, else 0
    int zs_colsum; // src_zp * colsum[n] - K * src_zp * wei_zp[n]
    int wei_zp; // wei_zp[n]
    float dst_zp; // dst_zp[n] when per-N
};

template <bool INT>
__device__ __forceinline__ ColTerms load_col_terms(const MatmulArgs &a, const TcParams &tp, int64_t n) {
    ColTerms c;
    c.wei_scale = 1.f;
    c.bias = 0.f;
    c.zs_colsum = 0;
    c.wei_zp = 0;
    c.dst_zp = 0.f;
    if (n >= a.N) return c;
    if (a.dst_zp.ptr && a.dst_zp.mask > 0) c.dst_zp = (float)((const int *)a.dst_zp.ptr)[n];
    if (a.wei_scale.ptr) c.wei_scale = load_float(a.wei_scale.dt, a.wei_scale.ptr, (a.wei_scale.mask & 2) ? n : 0);
    else if (a.wei_scale.on_host) c.wei_scale = a.wei_scale.host_value;
    if (a.bias && a.bias_sm == 0) c.bias = load_float(a.bias_dt, a.bias, n * a.bias_sn);
    if (INT) {
        if (a.wei_zp.ptr) c.wei_zp = load_int(a.wei_zp.dt, a.wei_zp.ptr, (a.wei_zp.mask & 2) ? n : 0);
        if (a.src_zp.ptr) {
            const int zs = ((const int *)a.src_zp.ptr)[0];
            c.zs_colsum = zs * tp.colsum[n] - (int)a.K * zs * c.wei_zp;
        }
    }
    return c;
}

// Per-tensor terms of the epilogue, read once per thread.
struct TensorTerms {
    bool has_dst_scale, has_dst_zp, dst_zp_per_n, row_scale, row_sum, bias_by_row;
    float dst_scale, dst_rcp, dst_zp, src_scale;
};

template <bool INT>
__device__ __forceinline__ TensorTerms load_tensor_terms(const MatmulArgs &a, const TcParams &tp) {
    TensorTerms t;
    t.has_dst_scale = a.non_default_attr && (a.dst_scale.ptr || a.dst_scale.on_host);
    t.dst_scale = a.dst_scale.ptr ? load_float(a.dst_scale.dt, a.dst_scale.ptr, 0) : a.dst_scale.host_value;
    t.dst_rcp = __frcp_rn(t.dst_scale);
    // the floating-point reference path has no dst zero-point
    t.has_dst_zp = a.non_default_attr && INT && a.dst_zp.ptr;
    t.dst_zp_per_n = a.dst_zp.mask > 0;
    t.dst_zp = (t.has_dst_zp && !t.dst_zp_per_n) ? (float)((const int *)a.dst_zp.ptr)[0] : 0.f;
    t.row_scale = a.src_scale.ptr && (a.src_scale.mask & 1);
    t.src_scale = 1.f; // per-tensor src scale (1 when absent or per-row)
    if (a.src_scale.ptr && !t.row_scale) t.src_scale = load_float(a.src_scale.dt, a.src_scale.ptr, 0);
    else if (a.src_scale.on_host) t.src_scale = a.src_scale.host_value;
    t.row_sum = INT && tp.rowsum != nullptr;
    t.bias_by_row = a.bias && a.bias_sm != 0;
    return t;
}

// Typed store of one f32 value, saturating / rounding as the reference does
// (src/cpu/simple_q10n.hpp:41-81; src/common/bfloat16.cpp:22-47: f32
// subnormals flush to signed zero before the bf16 rounding).
template <int DST>
__device__ __forceinline__ uint32_t typed_bits(float v) {
    if constexpr (DST == DT_F32) {
        return __float_as_uint(v);
    } else if constexpr (DST == DT_BF16) {
        if (fabsf(v) < 1.17549435e-38f) v = copysignf(0.f, v);
        unsigned short b = __bfloat16_as_ushort(__float2bfloat16_rn(v));
        if (v != v) b = (unsigned short)((__float_as_uint(v) >> 16) | 0x40u); // NaN: payload kept, quiet bit set
        return b;
    } else if constexpr (DST == DT_F16) {
        return __half_as_ushort(__float2half_rn(v));
    } else if constexpr (DST == DT_S32) {
        v = fminf(fmaxf(v, -2147483648.f), 2147483520.f);
        return (uint32_t)__float2int_rn(v);
    } else if constexpr (DST == DT_S8) {
        return (uint32_t)(unsigned char)(signed char)__float2int_rn(fminf(fmaxf(v, -128.f), 127.f));
    } else {
        return (uint32_t)(unsigned char)__float2int_rn(fminf(fmaxf(v, 0.f), 255.f));
    }
}
template <int DST>
__device__ __forceinline__ void store_bits(void *p, uint32_t b) {
    if constexpr (DST == DT_F32 || DST == DT_S32) *(uint32_t *)p = b;
    else if constexpr (DST == DT_BF16 || DST == DT_F16) *(unsigned short *)p = (unsigned short)b;
    else *(unsigned char *)p = (unsigned char)b;
}
template <int DST>
__device__ __forceinline__ void store_typed(void *p, float v) {
    store_bits<DST>(p, typed_bits<DST>(v));
}
template <int DST>
struct dst_size {
    static constexpr int value = (DST == DT_F32 || DST == DT_S32) ? 4 : (DST == DT_BF16 || DST == DT_F16) ? 2 : 1;
};

// 32 consecutive dst rows of column n, accumulators in r[0..31].  Absent
// scales are 1 and an absent bias is 0, which leaves values unchanged.
// FULL: all R rows exist (m0 + R <= M): no clamped row indices, no predicated stores.
template <bool INT, bool CHAIN, int DST, int R, bool FULL = false>
__device__ __forceinline__ void epilogue_rows(const MatmulArgs &a, const TcParams &tp, const TensorTerms &t,
        const ColTerms &c, const uint32_t (&r)[R], int64_t m0, int64_t n) {
    if (n >= a.N) return;
    char *dptr = (char *)a.dst + (m0 * a.dst_sm + n * a.dst_sn) * dst_size<DST>::value;
    const int64_t dstep = a.dst_sm * dst_size<DST>::value;
    const int rows = FULL ? R : (int)min((int64_t)R, a.M - m0);
    // Phases of straight-line code over the R rows (uniform conditions are
    // tested once per phase, not per row), so the rows' dependency chains
    // interleave; only the stores are predicated on the M tail.
    float d[R];
    if constexpr (INT) {
        if (t.row_sum) {
#pragma unroll
            for (int j = 0; j < R; ++j)
                d[j] = (float)((int)r[j] - c.zs_colsum - c.wei_zp * __ldg(tp.rowsum + (FULL ? m0 + j : min(m0 + j, a.M - 1))));
        } else {
#pragma unroll
            for (int j = 0; j < R; ++j) d[j] = (float)((int)r[j] - c.zs_colsum);
        }
    } else {
#pragma unroll
        for (int j = 0; j < R; ++j) d[j] = __uint_as_float(r[j]);
    }
    if (t.row_scale) {
        if (FULL && a.src_scale.dt == DT_F32) {
            const float *ss = (const float *)a.src_scale.ptr + m0;
#pragma unroll
            for (int j = 0; j < R; ++j) d[j] = __fmul_rn(d[j], __ldg(ss + j));
        } else {
#pragma unroll
            for (int j = 0; j < R; ++j)
                d[j] = __fmul_rn(d[j], load_float(a.src_scale.dt, a.src_scale.ptr, FULL ? m0 + j : min(m0 + j, a.M - 1)));
        }
    } else {
#pragma unroll
        for (int j = 0; j < R; ++j) d[j] = __fmul_rn(d[j], t.src_scale);
    }
#pragma unroll
    for (int j = 0; j < R; ++j) d[j] = __fadd_rn(__fmul_rn(d[j], c.wei_scale), c.bias);
    if constexpr (CHAIN) {
        if (t.bias_by_row) {
#pragma unroll
            for (int j = 0; j < R; ++j)
                d[j] = __fadd_rn(d[j],
                        load_float(a.bias_dt, a.bias, (FULL ? m0 + j : min(m0 + j, a.M - 1)) * a.bias_sm + n * a.bias_sn));
        }
        apply_post_ops_rows<R, (DST == DT_S8 || DST == DT_U8), FULL>(a, d, m0, n);
    }
    if (t.has_dst_scale) { // the reference divides; the same quotient from a reciprocal taken once per thread
#pragma unroll
        for (int j = 0; j < R; ++j) d[j] = div_by_scale(d[j], t.dst_scale, t.dst_rcp);
    }
    if (t.has_dst_zp) {
        const float z = t.dst_zp_per_n ? c.dst_zp : t.dst_zp;
#pragma unroll
        for (int j = 0; j < R; ++j) d[j] = __fadd_rn(d[j], z);
    }
#ifdef QMM_PROFILE
    if (tp.mainloop_only == 3) { // everything but the stores
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < R; ++j) acc += d[j];
        if (acc == 123.456f) store_typed<DST>(dptr, acc);
        return;
    }
#endif
    // (kernels with a post-op chain have no replicated form: they are short of registers as it is)
    if (CHAIN || a.peers.count == 0) {
#pragma unroll
        for (int j = 0; j < R; ++j)
            if (FULL || j < rows) store_typed<DST>(dptr + j * dstep, d[j]);
    } else {
        // every rank's copy of dst: the value is converted once and stored count + 1 times (plain
        // stores through peer-mapped addresses; the kernel's last CTA publishes the flags)
        uint32_t b[R];
#pragma unroll
        for (int j = 0; j < R; ++j) b[j] = typed_bits<DST>(d[j]);
#pragma unroll
        for (int j = 0; j < R; ++j)
            if (FULL || j < rows) store_bits<DST>(dptr + j * dstep, b[j]);
        for (int q = 0; q < a.peers.count; ++q) {
            char *pp = dptr + a.peers.delta[q];
#pragma unroll
            for (int j = 0; j < R; ++j)
                if (FULL || j < rows) store_bits<DST>(pp + j * dstep, b[j]);
        }
    }
}

// DSTT: the dst data type when the kernel was instantiated for one (post-op chain kernels: a single
// copy of the chain's code in the instruction stream), -1 to choose at run time.
template <bool INT, bool CHAIN, int R, int DSTT = -1>
__device__ __forceinline__ void epilogue_rows_any(const MatmulArgs &a, const TcParams &tp, const TensorTerms &t,
        const ColTerms &c, const uint32_t (&r)[R], int64_t m0, int64_t n) {
    if constexpr (DSTT >= 0) {
        // whole pieces (all but the last rows of a ragged M) take the straight path
        if (m0 + R <= a.M) epilogue_rows<INT, CHAIN, DSTT, R, true>(a, tp, t, c, r, m0, n);
        else epilogue_rows<INT, CHAIN, DSTT, R, false>(a, tp, t, c, r, m0, n);
        return;
    }
    switch (a.dst_dt) {
        case DT_BF16: epilogue_rows<INT, CHAIN, DT_BF16, R>(a, tp, t, c, r, m0, n); break;
        case DT_F32: epilogue_rows<INT, CHAIN, DT_F32, R>(a, tp, t, c, r, m0, n); break;
        case DT_S8: epilogue_rows<INT, CHAIN, DT_S8, R>(a, tp, t, c, r, m0, n); break;
        case DT_S32: epilogue_rows<INT, CHAIN, DT_S32, R>(a, tp, t, c, r, m0, n); break;
        case DT_F16: epilogue_rows<INT, CHAIN, DT_F16, R>(a, tp, t, c, r, m0, n); break;
        default: epilogue_rows<INT, CHAIN, DT_U8, R>(a, tp, t, c, r, m0, n); break;
    }
}

template <int KIND, int BT_M, int STAGES, bool CHAIN, int DSTT = -1>
__global__ void __launch_bounds__(num_threads(CHAIN), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
        const __grid_constant__ MatmulArgs a, const __grid_constant__ TcParams tp) {
    using L = SmemLayout<BT_M, STAGES>;
    constexpr bool INT = KIND == 1;
    constexpr int ACC_STAGES = 2;
    constexpr uint32_t TMEM_COLS = ACC_STAGES * BT_M; // 256 or 512, a power of two
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *full_bar = (uint64_t *)(smem + L::BAR_OFFSET);
    uint64_t *empty_bar = full_bar + STAGES;
    uint64_t *tmem_full = empty_bar + STAGES;
    uint64_t *tmem_empty = tmem_full + ACC_STAGES;
    uint32_t *tmem_base_slot = (uint32_t *)(tmem_empty + ACC_STAGES);
    volatile int *abort_flag = (volatile int *)(tmem_base_slot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int num_tiles = tp.num_m_tiles * tp.num_n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            ptx::mbar_init(&tmem_full[s], 1);
            ptx::mbar_init(&tmem_empty[s], epi_warps(CHAIN)); // one arrival per epilogue warp
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmW);
        ptx::prefetch_tensormap(&tmS);
    }
    if (warp == 1) ptx::tmem_alloc(tmem_base_slot, TMEM_COLS);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    // Tile order: the m index runs fastest, so the CTAs working at any moment
    // share a few weight column blocks and sweep the whole src once per block.
    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
                const int m0 = (tile % tp.num_m_tiles) * BT_M;
                const int n0 = (tile / tp.num_m_tiles) * BT_N;
                for (int kb = 0; kb < tp.num_k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1)) { *abort_flag = 1; atomicExch(a.status, 5); break; }
                    uint8_t *sw = smem + s * L::STAGE_BYTES, *ss = sw + L::W_BYTES;
                    ptx::mbar_arrive_expect_tx(&full_bar[s], L::STAGE_BYTES);
                    if (tp.w_kmajor) ptx::tma_load_2d(sw, &tmW, &full_bar[s], kb * BKB, n0);
                    else ptx::tma_load_2d(sw, &tmW, &full_bar[s], n0, kb * BKB);
                    ptx::tma_load_2d(ss, &tmS, &full_bar[s], kb * BKB, m0);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, acc_it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x, ++acc_it) {
                const int as = acc_it % ACC_STAGES;
                const uint32_t aph = (acc_it / ACC_STAGES) & 1;
                if (!ptx::mbar_wait(&tmem_empty[as], aph ^ 1)) { *abort_flag = 1; atomicExch(a.status, 5); break; }
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + as * BT_M;
                bool failed = false;
                for (int kb = 0; kb < tp.num_k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!ptx::mbar_wait(&full_bar[s], ph)) { failed = true; break; }
                    ptx::tc_fence_after_sync();
                    const uint32_t sw = ptx::smem_u32(smem + s * L::STAGE_BYTES), ss = sw + L::W_BYTES;
                    // weights: MN-major when N-contiguous (one 128-byte row per k), K-major for `ba`; src
                    // rows: K-major.  One thread issues: descriptors are built once per stage and advanced
                    // by a constant in their start-address field (16-byte units).
                    const uint64_t wd0 = tp.w_kmajor ? ptx::smem_desc_sw128(sw, 0, 1024) : ptx::smem_desc_sw128(sw, 128 * BKB, 1024);
                    const uint64_t wstep = tp.w_kmajor ? (uint64_t)(UMMA_K >> 4) : (uint64_t)((UMMA_K * 128) >> 4);
                    const uint64_t sd0 = ptx::smem_desc_sw128(ss, 0, 1024);
#pragma unroll
                    for (int kk = 0; kk < BKB / UMMA_K; ++kk)
                        ptx::mma_ss<KIND>(tmem_d, wd0 + kk * wstep, sd0 + (uint64_t)(kk * (UMMA_K >> 4)), tp.idesc, (kb | kk) != 0);
                    ptx::tc_commit(&empty_bar[s]); // stage reusable once these MMAs have read it
                }
                if (failed) { *abort_flag = 1; atomicExch(a.status, 5); break; }
                ptx::tc_commit(&tmem_full[as]); // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------ epilogue warps
        const int lane_base = (warp % 4) * 32; // TMEM lanes (dst columns) of this warp
        constexpr int GROUPS = epi_warps(CHAIN) / 4; // warps that share a quarter of the lanes
        constexpr int ROWS_PER_WARP = BT_M / (CHAIN ? 1 : GROUPS);
        const int group = (warp - 2) / 4;
        // without a chain each warp takes a contiguous share of the tile's rows; with one, the warps
        // of a lane quarter take the tile's 8-row pieces in turn (any number of warps divides them)
        const int row_base = CHAIN ? 0 : group * ROWS_PER_WARP;
        const TensorTerms tt = load_tensor_terms<INT>(a, tp);
        // the zero-point sums come from the kernel launched before this one, which runs beside this
        // kernel's set-up and first mainloop: only the epilogue warps wait for it
        if (tp.after_prekernel) asm volatile("griddepcontrol.wait;" ::: "memory");
        uint32_t acc_it = 0;
        for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x, ++acc_it) {
            const int as = acc_it % ACC_STAGES;
            const uint32_t aph = (acc_it / ACC_STAGES) & 1;
            const int64_t m_tile = (int64_t)(tile % tp.num_m_tiles) * BT_M + row_base;
            const int64_t n = (int64_t)(tile / tp.num_m_tiles) * BT_N + lane_base + lane;
            const ColTerms ct = load_col_terms<INT>(a, tp, n); // in flight while waiting for the MMAs
            if constexpr (CHAIN) {
                // Operands of binary post-ops that have a value per dst element (a residual) are read once,
                // row by row, in the middle of the chain: a miss there stalls the whole piece.  While the
                // tile is being multiplied, ask L2 for this warp's part of them (its rows x its 32 columns).
                for (int i = 0; i < a.n_po; ++i) {
                    const PostOpArg &e = a.po[i];
                    if (e.kind != PO_BINARY || e.sm == 0 || e.sn != 1) continue;
                    const int esz = (e.src1_dt == DT_F32 || e.src1_dt == DT_S32) ? 4 : (e.src1_dt == DT_BF16 || e.src1_dt == DT_F16) ? 2 : 1;
                    const int64_t nq = (int64_t)(tile / tp.num_m_tiles) * BT_N + lane_base;
                    if (nq >= a.N) continue;
                    constexpr int CRP = QMM_CHAIN_CR, PIECES_P = BT_M / CRP;
                    for (int idx = lane; idx < (PIECES_P + GROUPS - 1) / GROUPS * CRP; idx += 32) {
                        const int piece = group + GROUPS * (idx / CRP);
                        const int64_t m = m_tile + piece * CRP + idx % CRP;
                        if (piece < PIECES_P && m < a.M)
                            asm volatile("prefetch.global.L2 [%0];" ::"l"((const char *)e.src1 + (m * e.sm + nq) * esz));
                    }
                }
            }
            if (!ptx::mbar_wait(&tmem_full[as], aph)) { *abort_flag = 1; atomicExch(a.status, 5); break; }
            ptx::tc_fence_after_sync();
#ifdef QMM_PROFILE
            if (tp.mainloop_only == 1) { // results are not stored
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&tmem_empty[as]);
                continue;
            }
#endif
            if constexpr (CHAIN) {
                // With a post-op chain the code of 32 unrolled rows exceeds the instruction cache, so the
                // rows go through a rolled loop of 8-row pieces (8 independent dependency chains each).
                constexpr int CR = QMM_CHAIN_CR; // rows per piece: 4 leave too few independent chains (152 us on the int8 post-op workload), 16 overflow the instruction cache (175 us), 8: 134 us
                constexpr int PIECES = BT_M / CR;
#pragma unroll 1
                for (int c = group; c < PIECES; c += GROUPS) {
                    uint32_t r[CR];
                    ptx::tmem_ld_32xn(tmem_base + ((uint32_t)lane_base << 16) + as * BT_M + c * CR, r);
                    const int64_t m0 = m_tile + c * CR;
                    ptx::tmem_ld_wait();
                    if (c + GROUPS >= PIECES) { // accumulator fully read: hand the buffer back
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&tmem_empty[as]);
                    }
#ifdef QMM_PROFILE
                    if (tp.mainloop_only == 2) continue; // TMEM reads only
#endif
                    if (m0 < a.M) epilogue_rows_any<INT, CHAIN, CR, DSTT>(a, tp, tt, ct, r, m0, n);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < ROWS_PER_WARP / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(tmem_base + ((uint32_t)lane_base << 16) + as * BT_M + row_base + c * 32, r);
                    ptx::tmem_ld_wait();
                    if (c == ROWS_PER_WARP / 32 - 1) { // accumulator fully read: hand the buffer back
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&tmem_empty[as]);
                    }
                    const int64_t m0 = m_tile + c * 32;
#ifdef QMM_PROFILE
                    if (tp.mainloop_only == 2) continue; // TMEM reads only
#endif
                    if (m0 < a.M) epilogue_rows_any<INT, CHAIN, 32>(a, tp, tt, ct, r, m0, n);
                }
            }
        }
    }

    // ---------------------------------------------------- teardown
    if (!CHAIN && a.peers.count) __threadfence_system(); // this thread's peer stores, before the CTA is counted
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (!CHAIN && a.peers.count && threadIdx.x == 0) {
        // the last CTA to get here tells every rank that this rank's block is complete
        if (atomicAdd(a.peers.done, 1u) == gridDim.x - 1) {
            __threadfence_system();
            for (int r = 0; r < a.peers.world; ++r) {
                volatile unsigned *f = a.peers.flags[r] + a.peers.rank;
                *f = a.peers.epoch;
            }
            *a.peers.done = 0u;
        }
    }
}

// ---- zero-point compensation terms (int8 path) ----------------------------
// colsum[n] += sum over a chunk of k of w[k][n] (colsum zeroed beforehand).
// A block covers 128 columns x `kchunk` rows with 8 warps: a lane owns four
// neighbouring columns, the warps take every 8th row, the block adds its
// warps' sums in shared memory and issues one atomic add per column (integer
// addition: the result does not depend on the order).  VEC: weights are
// N-contiguous bytes with a 4-byte aligned pitch, so a lane's four columns are
// one 32-bit load and dp4a adds each byte into its own sum.
template <bool VEC>
__global__ void __launch_bounds__(256) colsum_kernel(const __grid_constant__ MatmulArgs a, int32_t *colsum, int kchunk) {
    asm volatile("griddepcontrol.launch_dependents;"); // the GEMM may start; its epilogue warps wait for this grid
    __shared__ int part[8][128];
    const int lane = threadIdx.x & 31, kl = threadIdx.x >> 5;
    const int64_t n0 = (int64_t)blockIdx.x * 128 + lane * 4;
    const int64_t k0 = (int64_t)blockIdx.y * kchunk, k1 = min(a.K, k0 + kchunk);
    int s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    if (VEC) {
        if (n0 < a.N) {
            const char *col = (const char *)a.wei + n0;
            if (a.wei_dt == DT_S8) {
#pragma unroll 4
                for (int64_t k = k0 + kl; k < k1; k += 8) {
                    const int v = *(const int *)(col + k * a.wei_sk);
                    s0 = __dp4a(v, 0x00000001, s0);
                    s1 = __dp4a(v, 0x00000100, s1);
                    s2 = __dp4a(v, 0x00010000, s2);
                    s3 = __dp4a(v, 0x01000000, s3);
                }
            } else {
#pragma unroll 4
                for (int64_t k = k0 + kl; k < k1; k += 8) {
                    const unsigned v = *(const unsigned *)(col + k * a.wei_sk);
                    s0 += v & 0xffu;
                    s1 += (v >> 8) & 0xffu;
                    s2 += (v >> 16) & 0xffu;
                    s3 += v >> 24;
                }
            }
        }
    } else {
        for (int64_t k = k0 + kl; k < k1; k += 8) {
            if (n0 + 0 < a.N) s0 += load_int(a.wei_dt, a.wei, k * a.wei_sk + (n0 + 0) * a.wei_sn);
            if (n0 + 1 < a.N) s1 += load_int(a.wei_dt, a.wei, k * a.wei_sk + (n0 + 1) * a.wei_sn);
            if (n0 + 2 < a.N) s2 += load_int(a.wei_dt, a.wei, k * a.wei_sk + (n0 + 2) * a.wei_sn);
            if (n0 + 3 < a.N) s3 += load_int(a.wei_dt, a.wei, k * a.wei_sk + (n0 + 3) * a.wei_sn);
        }
    }
    part[kl][lane * 4 + 0] = s0;
    part[kl][lane * 4 + 1] = s1;
    part[kl][lane * 4 + 2] = s2;
    part[kl][lane * 4 + 3] = s3;
    __syncthreads();
    if (threadIdx.x < 128) {
        const int64_t n = (int64_t)blockIdx.x * 128 + threadIdx.x;
        int s = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += part[w][threadIdx.x];
        if (n < a.N) atomicAdd(colsum + n, s);
    }
}
// rowsum[m] = sum_k s[m][k]; one warp per row
__global__ void rowsum_kernel(const __grid_constant__ MatmulArgs a, int32_t *rowsum) {
    asm volatile("griddepcontrol.launch_dependents;");
    const int64_t m = (int64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (m >= a.M) return;
    int s = 0;
    for (int64_t k = threadIdx.x % 32; k < a.K; k += 32) s += load_int(a.src_dt, a.src, m * a.src_sm + k * a.src_sk);
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x % 32 == 0) rowsum[m] = s;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
        const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
        CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_tiled_fn get_encode() {
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
                && q == cudaDriverEntryPointSuccess)
            fn = (encode_tiled_fn)p;
    }
    return fn;
}

// 2D map over a byte matrix [rows, cols] with row pitch `pitch` bytes; box =
// [box_rows, 128 bytes], 128-byte swizzle, out-of-bounds reads give zeros.
bool make_map_2d(CUtensorMap *map, const void *base, uint64_t cols, uint64_t rows, uint64_t pitch, uint32_t box_rows) {
    encode_tiled_fn enc = get_encode();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            == CUDA_SUCCESS;
}

template <int KIND, int BT_M, int STAGES, bool CHAIN, int DSTT = -1>
int launch_cfg(const CUtensorMap &mw, const CUtensorMap &ms, const MatmulArgs &a, TcParams tp, int sm_count,
        cudaStream_t st) {
    using L = SmemLayout<BT_M, STAGES>;
    auto kern = gemm_tc_kernel<KIND, BT_M, STAGES, CHAIN, DSTT>;
    static std::atomic<unsigned long long> configured; // one per instantiation of this template
    if (!opt_in_dynamic_smem(kern, L::TOTAL, configured)) return 5;
    const int tiles = tp.num_m_tiles * tp.num_n_tiles;
    const int grid = tiles < sm_count ? tiles : sm_count;
    bool launched = false;
    if (tp.after_prekernel) { // programmatic dependent of the sum kernel launched just before
        cudaLaunchConfig_t cfg {};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3((unsigned)num_threads(CHAIN));
        cfg.dynamicSmemBytes = (size_t)L::TOTAL;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        launched = cudaLaunchKernelEx(&cfg, kern, mw, ms, a, tp) == cudaSuccess;
        if (!launched) (void)cudaGetLastError(); // the attribute was refused: an ordinary launch below
    }
    if (!launched) kern<<<grid, num_threads(CHAIN), L::TOTAL, st>>>(mw, ms, a, tp);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

} // namespace

size_t gemm_tc_scratch_bytes(int64_t M, int64_t N) { return (size_t)(M + N) * sizeof(int32_t) + 256; }

bool gemm_tc_pointers_ok(const MatmulArgs &a) {
    return ((uintptr_t)a.src % 16 == 0) && ((uintptr_t)a.wei % 16 == 0);
}

// `scratch`: gemm_tc_scratch_bytes(M, N) bytes of device memory, needed only
// when zero-points are present.
int launch_gemm_tc(const MatmulArgs &a_in, void *scratch, int sm_count, cudaStream_t st) {
#ifdef QMM_PROFILE
    MatmulArgs a = a_in;
    if (getenv("ONEDNN_CUDA_TC_MAINLOOP_ONLY") && atoi(getenv("ONEDNN_CUDA_TC_MAINLOOP_ONLY")) == 4)
        for (int i = 0; i < a.n_po; ++i) a.po[i].sm = a.po[i].sn = 0;
#else
    const MatmulArgs &a = a_in;
#endif
    if (a.M == 0 || a.N == 0) return 0;
    if (a.K == 0) return 3;
    const bool int_path = a.src_dt == DT_S8 || a.src_dt == DT_U8;
    const bool w_kmajor = a.wei_sk == 1 && a.wei_sn != 1;
    TcParams tp {};
    tp.num_n_tiles = (int)((a.N + BT_N - 1) / BT_N);
    tp.num_k_blocks = (int)((a.K + BKB - 1) / BKB);
    tp.w_kmajor = w_kmajor;
#ifdef QMM_PROFILE // a build with -DQMM_PROFILE reads the switch; the shipped library has no such code
    static const int mainloop_only = getenv("ONEDNN_CUDA_TC_MAINLOOP_ONLY") ? atoi(getenv("ONEDNN_CUDA_TC_MAINLOOP_ONLY")) : 0;
    tp.mainloop_only = mainloop_only;
#endif

    int32_t *colsum = (int32_t *)scratch;
    int32_t *rowsum = colsum ? colsum + ((a.N + 63) / 64) * 64 : nullptr;
    if (int_path && a.src_zp.ptr) {
        if (!scratch) return 5;
        // enough blocks to fill the GPU, at least 64 rows each
        const unsigned nb = (unsigned)((a.N + 127) / 128);
        int64_t chunks = (4 * (int64_t)(sm_count > 0 ? sm_count : 148) + nb - 1) / nb;
        chunks = chunks < 1 ? 1 : (chunks > (a.K + 63) / 64 ? (a.K + 63) / 64 : chunks);
        const int kchunk = (int)(((a.K + chunks - 1) / chunks + 7) / 8 * 8);
        const dim3 grid(nb, (unsigned)((a.K + kchunk - 1) / kchunk));
        if (cudaMemsetAsync(colsum, 0, (size_t)a.N * sizeof(int32_t), st) != cudaSuccess) return 5;
        const bool vec = a.wei_sn == 1 && a.wei_sk % 4 == 0 && (uintptr_t)a.wei % 4 == 0 && a.N % 4 == 0
                && (a.wei_dt == DT_S8 || a.wei_dt == DT_U8);
        if (vec) colsum_kernel<true><<<grid, 256, 0, st>>>(a, colsum, kchunk);
        else colsum_kernel<false><<<grid, 256, 0, st>>>(a, colsum, kchunk);
        count_launch();
        tp.colsum = colsum;
    }
    if (int_path && a.wei_zp.ptr) {
        if (!scratch) return 5;
        rowsum_kernel<<<(unsigned)((a.M + 3) / 4), 128, 0, st>>>(a, rowsum);
        count_launch();
        tp.rowsum = rowsum;
    }
    tp.after_prekernel = tp.colsum != nullptr || tp.rowsum != nullptr;

    // 256 dst rows per tile unless that leaves SMs without work
    const int64_t tiles256 = (int64_t)tp.num_n_tiles * ((a.M + 255) / 256);
    const bool tall = a.M > 128 && tiles256 >= sm_count / 2;
    const int BT_M = tall ? 256 : 128;
    tp.num_m_tiles = (int)((a.M + BT_M - 1) / BT_M);

    CUtensorMap mw, ms;
    if (!make_map_2d(&ms, a.src, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.src_sm, BT_M)) return 5;
    if (w_kmajor) {
        if (!make_map_2d(&mw, a.wei, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.wei_sn, BT_N)) return 5;
    } else {
        if (!make_map_2d(&mw, a.wei, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.wei_sk, BKB)) return 5;
    }
    // operand A = weights, operand B = src
    uint32_t wfmt, sfmt, cfmt;
    if (int_path) {
        wfmt = a.wei_dt == DT_S8 ? ptx::FMT_S8 : ptx::FMT_U8;
        sfmt = a.src_dt == DT_S8 ? ptx::FMT_S8 : ptx::FMT_U8;
        cfmt = ptx::CFMT_S32;
    } else {
        wfmt = a.wei_dt == DT_F8_E4M3 ? ptx::FMT_E4M3 : ptx::FMT_E5M2;
        sfmt = a.src_dt == DT_F8_E4M3 ? ptx::FMT_E4M3 : ptx::FMT_E5M2;
        cfmt = ptx::CFMT_F32;
    }
    tp.idesc = ptx::make_idesc(cfmt, wfmt, sfmt, !w_kmajor, false, BT_N, BT_M);
    const bool chain = a.n_po > 0 || (a.bias && a.bias_sm != 0); // a bias varying along M rides the generic tail
    if (chain && a.peers.count) return 3; // refused when the replication is registered; not reached
    // kernels with a post-op chain are instantiated per dst data type
#define QMM_TC_CHAIN(KIND, BTM, ST) \
    (a.dst_dt == DT_S8         ? launch_cfg<KIND, BTM, ST, true, DT_S8>(mw, ms, a, tp, sm_count, st) \
                    : a.dst_dt == DT_U8   ? launch_cfg<KIND, BTM, ST, true, DT_U8>(mw, ms, a, tp, sm_count, st) \
                    : a.dst_dt == DT_BF16 ? launch_cfg<KIND, BTM, ST, true, DT_BF16>(mw, ms, a, tp, sm_count, st) \
                    : a.dst_dt == DT_F16  ? launch_cfg<KIND, BTM, ST, true, DT_F16>(mw, ms, a, tp, sm_count, st) \
                    : a.dst_dt == DT_F32  ? launch_cfg<KIND, BTM, ST, true, DT_F32>(mw, ms, a, tp, sm_count, st) \
                                          : launch_cfg<KIND, BTM, ST, true, DT_S32>(mw, ms, a, tp, sm_count, st))
#define QMM_TC_LAUNCH(KIND) \
    (tall ? (chain ? QMM_TC_CHAIN(KIND, 256, 4) : launch_cfg<KIND, 256, 4, false>(mw, ms, a, tp, sm_count, st)) \
          : (chain ? QMM_TC_CHAIN(KIND, 128, 6) : launch_cfg<KIND, 128, 6, false>(mw, ms, a, tp, sm_count, st)))
    return int_path ? QMM_TC_LAUNCH(1) : QMM_TC_LAUNCH(0);
#undef QMM_TC_LAUNCH
#undef QMM_TC_CHAIN
}

// ---- allocation-free variant ----------------------------------------------
// Scratch of dnnl_cuda_interop_matmul_u8s8s32_zp_static: the column sums of
// the weights (zero-point compensation), preceded by a small header (the
// zero-point value and the kernel status word).  It is part of the library
// image: every GPU that loads the library holds these bytes until exit.
constexpr int64_t STATIC_MAX_N = 131072;
constexpr int STATIC_HEADER_WORDS = 64;
static __device__ __align__(256) int32_t g_static_scratch[STATIC_HEADER_WORDS + STATIC_MAX_N];

// hdr[0]: the src zero-point of the call in flight, read by the GEMM epilogue.
// hdr[1]: the kernels' status word.  It starts at zero when the library is
// loaded and is sticky: a call never clears it, so a bounded wait that expired
// in any earlier call stays visible until ..._static_status reads and resets it.
__global__ void static_scratch_header_kernel(int32_t *hdr, int32_t zero_point) { hdr[0] = zero_point; }
__global__ void static_scratch_status_reset_kernel(int32_t *hdr) { hdr[1] = 0; }

// Device address of the static scratch on the current device (looked up once
// per device; the table is filled under a mutex so that two host threads may
// make their first calls together).
constexpr int STATIC_MAX_DEVICES = 64;
struct StaticScratchSlot {
    int32_t *ptr = nullptr;
    int sm_count = 0;
};
bool static_scratch_of_current_device(StaticScratchSlot *out) {
    static StaticScratchSlot slots[STATIC_MAX_DEVICES];
    static std::mutex mu;
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return false;
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) {
        set_last_error("static scratch: device ordinal beyond 63");
        return false;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!slots[dev].ptr) { // set-up, once per device; not to be done under stream capture
        void *p = nullptr;
        // the array's NAME is a host-side stand-in here; kernels need its device address
        if (!cuda_ok(cudaGetSymbolAddress(&p, g_static_scratch), "cudaGetSymbolAddress")) return false;
        int sms = 0;
        if (!cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute"))
            return false;
        slots[dev].sm_count = sms;
        slots[dev].ptr = (int32_t *)p;
    }
    *out = slots[dev];
    return true;
}

} // namespace qmm

// Host side of the static scratch: the array's NAME is only a host-side
// stand-in here; kernels need its device address, looked up once per device
// (with that device current) by cudaGetSymbolAddress.  The call allocates
// nothing: it enqueues a memset of the column sums, three small kernels and
// the GEMM on the caller's stream.
extern "C" dnnl_status_t dnnl_cuda_interop_matmul_u8s8s32_zp_static(void *cuda_stream, int64_t M, int64_t N,
        int64_t K, const uint8_t *src, const int8_t *weights, int32_t src_zero_point, int32_t *dst) {
    using namespace qmm;
    if (M < 0 || N < 0 || K < 0 || ((M && K) && !src) || ((K && N) && !weights) || ((M && N) && !dst))
        return (dnnl_status_t)2; // invalid_arguments
    if (N > STATIC_MAX_N) {
        set_last_error("dnnl_cuda_interop_matmul_u8s8s32_zp_static: N exceeds the static scratch (131072 columns)");
        return (dnnl_status_t)2;
    }
    if (M == 0 || N == 0 || K == 0) return (dnnl_status_t)0; // nothing to compute, as the primitive does
    if (K % 16 || N % 16 || (uintptr_t)src % 16 || (uintptr_t)weights % 16 || M >= (1LL << 31)
            || K >= (1LL << 31)) {
        set_last_error("dnnl_cuda_interop_matmul_u8s8s32_zp_static: K and N must be multiples of 16 and the "
                       "src / weights pointers 16-byte aligned");
        return (dnnl_status_t)3; // unimplemented
    }
    StaticScratchSlot slot;
    if (!static_scratch_of_current_device(&slot)) return (dnnl_status_t)5;
    int32_t *hdr = slot.ptr;
    cudaStream_t st = (cudaStream_t)cuda_stream;
    static_scratch_header_kernel<<<1, 1, 0, st>>>(hdr, src_zero_point);
    count_launch();

    MatmulArgs a {};
    a.M = M; a.N = N; a.K = K;
    a.src = src; a.src_dt = DT_U8; a.src_sm = K; a.src_sk = 1;
    a.wei = weights; a.wei_dt = DT_S8; a.wei_sk = N; a.wei_sn = 1;
    a.dst = dst; a.dst_dt = DT_S32; a.dst_sm = N; a.dst_sn = 1;
    for (QParam *q : {&a.src_scale, &a.wei_scale, &a.dst_scale, &a.src_zp, &a.wei_zp, &a.dst_zp, &a.src_pr})
        q->g0 = q->g1 = 1;
    a.src_zp.ptr = hdr; // word 0 of the header
    a.src_zp.dt = DT_S32;
    a.non_default_attr = 1;
    a.sum_dt = DT_S32;
    a.status = hdr + 1;
    const int rc = launch_gemm_tc(a, hdr + STATIC_HEADER_WORDS, slot.sm_count, st);
    if (rc == 5) set_last_error(std::string("kernel launch: ") + cudaGetErrorString(cudaGetLastError()));
    return (dnnl_status_t)rc;
}

// Reads the sticky status word of the static entry point on the current
// device: waits for the work already enqueued on `cuda_stream`, copies the word
// to *status (0 = every call since the last query completed; 5 = a bounded
// wait inside a kernel expired and its dst is incomplete) and resets it.
// Allocates nothing; synchronises the stream, so it is not for use while the
// stream is being captured.
extern "C" dnnl_status_t dnnl_cuda_interop_matmul_u8s8s32_zp_static_status(void *cuda_stream, int *status) {
    using namespace qmm;
    if (!status) return (dnnl_status_t)2;
    StaticScratchSlot slot;
    if (!static_scratch_of_current_device(&slot)) return (dnnl_status_t)5;
    cudaStream_t st = (cudaStream_t)cuda_stream;
    int32_t word = 0;
    if (!cuda_ok(cudaMemcpyAsync(&word, slot.ptr + 1, sizeof(word), cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync"))
        return (dnnl_status_t)5;
    if (!cuda_ok(cudaStreamSynchronize(st), "cudaStreamSynchronize")) return (dnnl_status_t)5;
    *status = word;
    if (word != 0) {
        static_scratch_status_reset_kernel<<<1, 1, 0, st>>>(slot.ptr);
        count_launch();
        if (!cuda_ok(cudaGetLastError(), "status reset")) return (dnnl_status_t)5;
    }
    return (dnnl_status_t)0;
}
