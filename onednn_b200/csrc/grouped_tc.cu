// "cuda:tcgen05:grouped": grouped (MoE) weight-decompression matmul on the
// 5th-generation tensor cores: for every expert e with src rows [b_e, e_e),
//   dst[rows, :] = (src[rows, :] (bf16) x float(W_e[K, N] (s8))) * scale[e, :]
// with f32 accumulation in tensor memory.  The scale multiplies the finished
// sum, as the reference's grouped implementation does
// (src/cpu/matmul/ref_grouped_gemm.cpp:312-339); results differ from it only
// by f32 summation order.  A second instantiation of the kernel adds, in the
// epilogue, the bias, the eltwise / binary post-op chain and weight
// zero-points: sum_k s (w - z) = sum_k s w - z sum_k s, with the src row sums
// from a small pre-kernel.
//
// The tensor cores take 16-bit operands from shared memory, so the int8
// weights are widened on the way: TMA brings a raw [64 k x 128 n] s8 tile,
// converter warps rewrite it as bf16 (exact: 8 significant bits) in the
// MN-major 128B-swizzled layout the MMA reads, and `tcgen05.mma kind::f16`
// multiplies it with the src rows (K-major, straight from TMA).  As in the
// 8-bit GEMM the kernel computes dst^T: weights are the A operand (128 dst
// columns = TMEM lanes), src rows the B operand, so an epilogue lane owns one
// dst column, keeps its scale in a register and stores coalesced rows.
//
// Tiles are (expert, 128 columns, up to 256 rows of that expert); the MMA's N
// extent is the tile's row count rounded up to 16, so small experts cost
// little tensor time.  Tile order: expert, column block, row block fastest,
// so CTAs running together share weight tiles through L2.  A small planning
// kernel turns the offsets (cumulative END rows, validated like
// ref_grouped_gemm.cpp:164-213) into per-expert tile ranges on the device:
// no host synchronisation.  One persistent CTA per SM: warp 0 streams the raw
// weight tiles (ring of 8: they come from HBM), the last warp the src rows
// (ring of 4: they come from L2), warps 2-9 convert into a ring of 2 bf16
// tiles, warp 1 issues the MMAs, the next four warps run the epilogue; two
// TMEM accumulator buffers.  Every mbarrier wait is bounded.
#include <cuda.h>

#include "device_math.cuh"
#include "launch.h"
#include "sm100_ptx.cuh"

namespace qmm {

namespace {

constexpr int GT_N = 128; // dst columns per tile = TMEM lanes = UMMA M
constexpr int GT_M = 256; // most src rows per tile = UMMA N
constexpr int GK = 64; // k per stage: one 128-byte swizzle row of bf16 src
// Three rings, one per kind of tile, because their needs differ: the raw weights come from HBM
// (deep ring of small tiles to cover its latency), the src rows from L2, and the bf16 copy is
// produced and consumed on the SM (two slots: one being written, one being multiplied).
constexpr int RAW_STAGES = 8, A_STAGES = 2, B_STAGES = 4;
constexpr int RAW_BYTES = GK * GT_N; // s8 weights as loaded
constexpr int A_BYTES = GK * GT_N * 2; // the same tile as bf16: two 64-column blocks of [64 k][128 B]
constexpr int B_BYTES = GT_M * GK * 2; // src rows, K-major
constexpr int CONV_WARPS = 8, EPI_WARPS = 4;
constexpr int G_THREADS = 32 * (3 + CONV_WARPS + EPI_WARPS);
constexpr int ACC_STAGES = 2;
constexpr int A_OFFSET = 0, B_OFFSET = A_STAGES * A_BYTES, RAW_OFFSET = B_OFFSET + B_STAGES * B_BYTES;
constexpr int G_BAR_OFFSET = RAW_OFFSET + RAW_STAGES * RAW_BYTES;
constexpr int G_SMEM_BYTES = G_BAR_OFFSET + 512 + 1024;

// plan[0] = {total tiles, groups, 0, 0}; plan[1 + g] = {first src row, first dst row, rows, first tile}
struct Tile {
    int g, n0, m0, rows, src_row, dst_row;
};
__device__ __forceinline__ Tile decode_tile(const int4 *plan, int groups, int num_n_tiles, int t) {
    int lo = 0, hi = groups; // last group whose first tile is <= t, skipping empty groups behind it
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(&plan[1 + mid]).w <= t) lo = mid; else hi = mid;
    }
    const int4 e = __ldg(&plan[1 + lo]);
    const int r = t - e.w;
    const int mt = (e.z + GT_M - 1) / GT_M;
    Tile tl;
    tl.g = lo;
    tl.n0 = (r / mt) * GT_N;
    tl.m0 = (r % mt) * GT_M;
    tl.rows = min(GT_M, e.z - tl.m0);
    tl.src_row = e.x + tl.m0;
    tl.dst_row = e.y + tl.m0;
    return tl;
}

__global__ void grouped_plan_kernel(const __grid_constant__ MatmulArgs a, int4 *plan, int num_n_tiles) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    if (a.group_count == 0) { // a dense problem: one group that owns every row
        plan[1] = make_int4(0, 0, (int)a.M, 0);
        plan[0] = make_int4((int)((a.M + GT_M - 1) / GT_M) * num_n_tiles, 1, 0, 0);
        return;
    }
    bool bad = false;
    int tiles = 0;
    for (int g = 0; g < a.group_count; ++g) {
        const int64_t b = g == 0 ? 0 : a.offsets[g - 1], e = a.offsets[g];
        const int64_t db = g == 0 ? 0 : a.dst_offsets[g - 1], de = a.dst_offsets[g];
        if (b < 0 || e > a.M || e < b || db < 0 || de > a.M || de < db || de - db != e - b) bad = true;
        const int rows = bad ? 0 : (int)(e - b);
        plan[1 + g] = make_int4((int)b, (int)db, rows, tiles);
        tiles += ((rows + GT_M - 1) / GT_M) * num_n_tiles;
    }
    if (bad) {
        atomicExch(a.status, 2); // invalid_arguments, reported when the stream is waited on
        tiles = 0;
    }
    plan[0] = make_int4(tiles, a.group_count, 0, 0);
}

// four s8 -> four bf16 without a conversion instruction: with xx = x & 0x7f the bf16 0x43xx is
// 128 + (x & 127), with xx = x & 0x80 it is 128 or 256; their difference is x, exactly
__device__ __forceinline__ uint32_t prmt_(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ void s8x4_to_bf16x4(uint32_t w, uint32_t &o0, uint32_t &o1) {
    const uint32_t p0 = prmt_(w, 0x43434343u, 0x4140); // [x0, 0x43, x1, 0x43]
    const uint32_t p1 = prmt_(w, 0x43434343u, 0x4342); // [x2, 0x43, x3, 0x43]
    o0 = bf16x2_sub(p0 & 0xff7fff7fu, p0 & 0xff80ff80u);
    o1 = bf16x2_sub(p1 & 0xff7fff7fu, p1 & 0xff80ff80u);
}

// Sum over k of every src row (bf16), one warp per row: the factor of a weight zero-point,
// sum_k s (w - z) = sum_k s w - z sum_k s.
__global__ void grouped_rowsum_kernel(const __grid_constant__ MatmulArgs a, float *rowsum) {
    const int64_t m = (int64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (m >= a.M) return;
    const unsigned short *row = (const unsigned short *)a.src + m * a.src_sm;
    float s = 0.f;
    for (int64_t k = threadIdx.x % 32; k < a.K; k += 32) s += bf16_bits_to_f32(row[k]);
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x % 32 == 0) rowsum[m] = s;
}

template <bool EPI_CHAIN>
__global__ void __launch_bounds__(G_THREADS, 1)
grouped_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
        const __grid_constant__ MatmulArgs a, const int4 *plan, const float *rowsum, int num_n_tiles,
        int num_k_blocks) {
    constexpr uint32_t TMEM_COLS = ACC_STAGES * GT_M;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *raw_full = (uint64_t *)(smem + G_BAR_OFFSET); // raw weight tile has landed
    uint64_t *raw_empty = raw_full + RAW_STAGES; // the converters have read it
    uint64_t *b_full = raw_empty + RAW_STAGES; // src rows have landed
    uint64_t *b_empty = b_full + B_STAGES; // the MMAs have read them
    uint64_t *a_full = b_empty + B_STAGES; // the weights are rewritten as bf16
    uint64_t *a_empty = a_full + A_STAGES; // the MMAs have read them
    uint64_t *tmem_full = a_empty + A_STAGES;
    uint64_t *tmem_empty = tmem_full + ACC_STAGES;
    uint32_t *tmem_base_slot = (uint32_t *)(tmem_empty + ACC_STAGES);
    volatile int *abort_flag = (volatile int *)(tmem_base_slot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < RAW_STAGES; ++s) {
            ptx::mbar_init(&raw_full[s], 1);
            ptx::mbar_init(&raw_empty[s], CONV_WARPS);
        }
        for (int s = 0; s < B_STAGES; ++s) {
            ptx::mbar_init(&b_full[s], 1);
            ptx::mbar_init(&b_empty[s], 1);
        }
        for (int s = 0; s < A_STAGES; ++s) {
            ptx::mbar_init(&a_full[s], CONV_WARPS);
            ptx::mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            ptx::mbar_init(&tmem_full[s], 1);
            ptx::mbar_init(&tmem_empty[s], EPI_WARPS);
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
    const int4 head = __ldg(&plan[0]);
    const int num_tiles = head.x, groups = head.y;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer of the raw weight tiles
        if (lane == 0) {
            uint32_t it = 0;
            for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
                const Tile tl = decode_tile(plan, groups, num_n_tiles, t);
                for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
                    const int s = it % RAW_STAGES;
                    const uint32_t ph = (it / RAW_STAGES) & 1;
                    if (!ptx::mbar_wait(&raw_empty[s], ph ^ 1)) { *abort_flag = 1; atomicExch(a.status, 5); break; }
                    ptx::mbar_arrive_expect_tx(&raw_full[s], RAW_BYTES);
                    ptx::tma_load_3d(smem + RAW_OFFSET + s * RAW_BYTES, &tmW, &raw_full[s], tl.n0, kb * GK, tl.g);
                }
            }
        }
    } else if (warp == 2 + CONV_WARPS + EPI_WARPS) {
        // ------------------------------------------------ TMA producer of the src rows
        if (lane == 0) {
            uint32_t it = 0;
            for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
                const Tile tl = decode_tile(plan, groups, num_n_tiles, t);
                const int nbox = (tl.rows + 63) / 64; // src boxes of 64 rows
                for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
                    const int s = it % B_STAGES;
                    const uint32_t ph = (it / B_STAGES) & 1;
                    if (!ptx::mbar_wait(&b_empty[s], ph ^ 1)) { *abort_flag = 1; atomicExch(a.status, 5); break; }
                    uint8_t *bt = smem + B_OFFSET + s * B_BYTES;
                    ptx::mbar_arrive_expect_tx(&b_full[s], nbox * 64 * GK * 2);
                    for (int j = 0; j < nbox; ++j)
                        ptx::tma_load_2d(bt + j * 64 * GK * 2, &tmS, &b_full[s], kb * GK, tl.src_row + 64 * j);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, acc_it = 0;
            for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x, ++acc_it) {
                const Tile tl = decode_tile(plan, groups, num_n_tiles, t);
                const uint32_t n_mma = (uint32_t)max(16, (tl.rows + 15) & ~15);
                const uint32_t idesc
                        = ptx::make_idesc(ptx::CFMT_F32, ptx::FMT_BF16, ptx::FMT_BF16, true, false, GT_N, n_mma);
                const int as = acc_it % ACC_STAGES;
                const uint32_t aph = (acc_it / ACC_STAGES) & 1;
                if (!ptx::mbar_wait(&tmem_empty[as], aph ^ 1)) { *abort_flag = 1; atomicExch(a.status, 5); break; }
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + as * GT_M;
                bool failed = false;
                for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
                    const int sa_i = it % A_STAGES, sb_i = it % B_STAGES;
                    if (!ptx::mbar_wait(&a_full[sa_i], (it / A_STAGES) & 1)
                            || !ptx::mbar_wait(&b_full[sb_i], (it / B_STAGES) & 1)) {
                        failed = true;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t sa = ptx::smem_u32(smem + A_OFFSET + sa_i * A_BYTES);
                    const uint32_t sb = ptx::smem_u32(smem + B_OFFSET + sb_i * B_BYTES);
                    // weights MN-major: 16 k-rows of 128 bytes per MMA, 64-column blocks 8 KB apart; src rows
                    // K-major: 32 bytes of the row per MMA.  The issuing thread is one instruction stream
                    // (about five cycles per dependent instruction), so the descriptors are built once per
                    // stage and advanced by constants in their start-address field (16-byte units).
                    const uint64_t wd0 = ptx::smem_desc_sw128(sa, GK * 128, 1024);
                    const uint64_t sd0 = ptx::smem_desc_sw128(sb, 0, 1024);
#pragma unroll
                    for (int kk = 0; kk < GK / 16; ++kk)
                        ptx::mma_ss<2>(tmem_d, wd0 + (uint64_t)(kk * ((16 * 128) >> 4)), sd0 + (uint64_t)(kk * (32 >> 4)), idesc,
                                (kb | kk) != 0);
                    // both tiles are reusable once these MMAs have read them
                    ptx::tc_commit(&a_empty[sa_i]);
                    ptx::tc_commit(&b_empty[sb_i]);
                }
                if (failed) { *abort_flag = 1; atomicExch(a.status, 5); break; }
                ptx::tc_commit(&tmem_full[as]); // accumulator complete
            }
        }
    } else if (warp < 2 + CONV_WARPS) {
        // ------------------------------------------------ converters: s8 tile -> bf16 MMA operand
        const int ct = threadIdx.x - 64; // 0 .. 32 CONV_WARPS - 1
        const int c = ct & 7; // 16-byte chunk of the raw row: columns 16c .. 16c+15
        const int blk = c >> 2, q = 2 * (c & 3); // 64-column block and 16-byte chunk pair of the bf16 row
        // A 16-byte store is served a quarter-warp (8 lanes, here one k-row) at a time: the lanes of
        // block 0 store their even chunk first and those of block 1 their odd one, so that the eight
        // stores of a quarter-warp fall on eight different 16-byte bank groups.
        const int q_first = q + blk, q_second = q + 1 - blk;
        uint32_t it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok && !*abort_flag; t += gridDim.x) {
            for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
                const int sr = it % RAW_STAGES, sa_i = it % A_STAGES;
                // the raw tile has landed, and the MMAs have finished with the bf16 slot to overwrite
                if (!__all_sync(0xffffffffu,
                            ptx::mbar_wait(&raw_full[sr], (it / RAW_STAGES) & 1)
                                    && ptx::mbar_wait(&a_empty[sa_i], ((it / A_STAGES) & 1) ^ 1))) {
                    ok = false;
                    break;
                }
                const uint8_t *raw = smem + RAW_OFFSET + sr * RAW_BYTES;
                uint8_t *at = smem + A_OFFSET + sa_i * A_BYTES + blk * (GK * 128);
#pragma unroll
                for (int i = 0; i < 16 / CONV_WARPS; ++i) {
                    const int r = (ct >> 3) + 4 * CONV_WARPS * i; // k-row
                    const uint4 w = *reinterpret_cast<const uint4 *>(raw + r * 128 + c * 16);
                    uint4 lo, hi;
                    s8x4_to_bf16x4(w.x, lo.x, lo.y);
                    s8x4_to_bf16x4(w.y, lo.z, lo.w);
                    s8x4_to_bf16x4(w.z, hi.x, hi.y);
                    s8x4_to_bf16x4(w.w, hi.z, hi.w);
                    uint8_t *row = at + r * 128;
                    *reinterpret_cast<uint4 *>(row + ((q_first ^ (r & 7)) << 4)) = blk ? hi : lo;
                    *reinterpret_cast<uint4 *>(row + ((q_second ^ (r & 7)) << 4)) = blk ? lo : hi;
                }
                ptx::fence_proxy_async(); // the MMA reads these bytes through the async proxy
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&a_full[sa_i]);
                    ptx::mbar_arrive(&raw_empty[sr]);
                }
            }
        }
        if (!ok) { *abort_flag = 1; atomicExch(a.status, 5); }
    } else {
        // ------------------------------------------------ epilogue warps
        const int lane_base = (warp % 4) * 32; // TMEM lanes (dst columns) this warp may read
        uint32_t acc_it = 0;
        for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x, ++acc_it) {
            const Tile tl = decode_tile(plan, groups, num_n_tiles, t);
            const int as = acc_it % ACC_STAGES;
            const uint32_t aph = (acc_it / ACC_STAGES) & 1;
            const int64_t n = tl.n0 + lane_base + lane;
            float scale = 1.f;
            if (a.wei_scale.ptr && n < a.N)
                scale = load_float(a.wei_scale.dt, a.wei_scale.ptr,
                        (int64_t)tl.g * a.wei_scale.gstride + ((a.wei_scale.mask & 2) ? n : 0));
            float zp = 0.f; // weight zero-point of this column (chain epilogue only)
            if (EPI_CHAIN && a.wei_zp.ptr && n < a.N)
                zp = (float)load_int(a.wei_zp.dt, a.wei_zp.ptr,
                        (int64_t)tl.g * a.wei_zp.gstride + ((a.wei_zp.mask & 2) ? n : 0));
            if (!ptx::mbar_wait(&tmem_full[as], aph)) { *abort_flag = 1; atomicExch(a.status, 5); break; }
            ptx::tc_fence_after_sync();
            const int chunks = (tl.rows + 31) / 32;
#pragma unroll 1
            for (int cidx = 0; cidx < chunks; ++cidx) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(tmem_base + ((uint32_t)lane_base << 16) + as * GT_M + cidx * 32, r);
                ptx::tmem_ld_wait();
                if (cidx == chunks - 1) { // accumulator fully read: hand the buffer back
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&tmem_empty[as]);
                }
                if (n < a.N) {
                    const int m_hi = min(32, tl.rows - cidx * 32);
                    const int64_t row0 = (int64_t)tl.dst_row + cidx * 32;
                    if constexpr (EPI_CHAIN) {
                        // bias (one row per expert, or the dense problem's own broadcast) and the post-op
                        // chain, in the reference's order: scale, bias, post-ops, store
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (j >= m_hi) continue;
                            const int64_t m = row0 + j;
                            float acc = __uint_as_float(r[j]);
                            if (a.wei_zp.ptr) acc = fmaf(-zp, __ldg(rowsum + tl.src_row + cidx * 32 + j), acc);
                            float d = __fmul_rn(acc, scale);
                            if (a.bias)
                                d = __fadd_rn(d,
                                        load_float(a.bias_dt, a.bias,
                                                a.group_count > 0 ? (int64_t)tl.g * a.bias_sg + n
                                                                  : m * a.bias_sm + n * a.bias_sn));
                            d = apply_post_ops(a, d, 0.f, m, n, tl.g);
                            store_float(a.dst_dt, d, a.dst, m * a.dst_sm + n);
                        }
                    } else if (a.dst_dt == DT_BF16) {
                        unsigned short *d = (unsigned short *)a.dst + row0 * a.dst_sm + n;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < m_hi) d[(int64_t)j * a.dst_sm] = f32_to_bf16_bits(__uint_as_float(r[j]) * scale);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < m_hi)
                                store_float(a.dst_dt, __uint_as_float(r[j]) * scale, a.dst, (row0 + j) * a.dst_sm + n);
                    }
                }
            }
        }
    }

    // ---------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
        const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
        CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_tiled_fn grouped_get_encode() {
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess
                && q == cudaDriverEntryPointSuccess)
            fn = (encode_tiled_fn)ptr;
    }
    return fn;
}

} // namespace

// plan records, then (256-byte aligned) one f32 row sum per src row
static size_t plan_bytes(int groups) { return ((size_t)(1 + groups) * sizeof(int4) + 255) / 256 * 256; }
size_t grouped_tc_scratch_bytes(int groups, int64_t M) { return plan_bytes(groups) + (size_t)M * sizeof(float); }

bool grouped_tc_pointers_ok(const MatmulArgs &a) {
    return (uintptr_t)a.wei % 16 == 0 && (uintptr_t)a.src % 16 == 0 && (uintptr_t)a.dst % 2 == 0;
}

// bf16 src [M, K] (rows of all experts concatenated), s8 weights [G, K, N] with N contiguous, per-(expert, column)
// weight scales, bf16 / f16 / f32 dst.  `scratch`: grouped_tc_scratch_bytes(group_count) bytes.
int launch_grouped_tc(const MatmulArgs &a, void *scratch, int sm_count, cudaStream_t st) {
    if (a.M == 0 || a.N == 0) return 0;
    encode_tiled_fn enc = grouped_get_encode();
    if (!enc || !scratch) return 5;
    CUtensorMap tw, ts;
    { // weights as bytes [G][K][N]: raw tile of 64 k x 128 n; a dense [K][N] matrix is one group
        const int64_t groups = a.group_count > 0 ? a.group_count : 1;
        const int64_t group_pitch = a.group_count > 0 ? a.wei_sg : a.K * a.wei_sk;
        cuuint64_t dims[3] = {(cuuint64_t)a.N, (cuuint64_t)a.K, (cuuint64_t)groups};
        cuuint64_t strides[2] = {(cuuint64_t)a.wei_sk, (cuuint64_t)group_pitch};
        cuuint32_t box[3] = {GT_N, GK, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        if (enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(a.wei), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                != CUDA_SUCCESS)
            return 5;
    }
    { // src as 16-bit words [M][K]: boxes of 64 rows x 64 k, 128B swizzle
        cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
        cuuint64_t strides[1] = {(cuuint64_t)(a.src_sm * 2)};
        cuuint32_t box[2] = {GK, 64};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(a.src), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                != CUDA_SUCCESS)
            return 5;
    }
    const int num_n_tiles = (int)((a.N + GT_N - 1) / GT_N);
    const int num_k_blocks = (int)((a.K + GK - 1) / GK);
    int4 *plan = (int4 *)scratch;
    grouped_plan_kernel<<<1, 32, 0, st>>>(a, plan, num_n_tiles);
    count_launch();
    float *rowsum = (float *)((char *)scratch + plan_bytes(a.group_count > 0 ? a.group_count : 1));
    if (a.wei_zp.ptr) {
        grouped_rowsum_kernel<<<(unsigned)((a.M + 7) / 8), 256, 0, st>>>(a, rowsum);
        count_launch();
    }
    // epilogue with zero-points / bias / post-ops: its own instantiation
    const bool chain = a.bias != nullptr || a.n_po > 0 || a.wei_zp.ptr != nullptr;
    auto kern = chain ? grouped_tc_kernel<true> : grouped_tc_kernel<false>;
    static std::atomic<unsigned long long> configured[2];
    if (!opt_in_dynamic_smem(kern, G_SMEM_BYTES, configured[chain])) return 5;
    kern<<<sm_count > 0 ? sm_count : 148, G_THREADS, G_SMEM_BYTES, st>>>(tw, ts, a, plan, rowsum, num_n_tiles, num_k_blocks);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

} // namespace qmm
