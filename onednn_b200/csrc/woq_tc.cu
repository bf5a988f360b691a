// "cuda:tcgen05:woq4": int4 weight-decompression matmul for few rows (decode,
// M <= 32) on the 5th-generation tensor cores, with the decompressed weights
// passed to the MMA through TENSOR MEMORY instead of shared memory:
//   dst[M,N] = src[M,K] (bf16/f16) x dequant(weights[K,N] s4/u4 `ab`),
// scales per column or per (K-group, column), optional zero-points (fpmath
// apply_to_int; reference arithmetic: src/cpu/matmul/ref_matmul.cpp:193-233).
//
// The problem is bound by the HBM stream of the packed weights (half a byte
// each).  tcgen05.mma takes its A operand from tensor memory, so the weights
// never exist as 16-bit values in shared memory (which would cost 4 bytes of
// shared-memory traffic per weight):
//   * TMA streams raw nibble tiles (128-byte swizzled boxes) and the matching
//     src columns into a ring of stages;
//   * converter warps read 8 (or 4) bytes per k-row and lane and rebuild
//     operand registers with one PRMT per two k-rows and one LOP3 per two
//     weights: a nibble u becomes the bf16 128+u (f16: the subnormal u*2^-24),
//     exactly; the four registers of a lane are the 16 x 16 operand fragment
//     that `tcgen05.st.16x128b.x2` writes into the A slot (TMEM lane = dst
//     column, two k per 32-bit column);
//   * one thread issues `tcgen05.mma.kind::f16` (A from TMEM, B = the src rows
//     from shared memory, K-major), D = dst^T in TMEM (lane = dst column,
//     column = src row), plus one MMA against a constant all-ones A tile whose
//     result is S[m] = sum_k src[m][k] of the quantization group;
//   * at the end of every K-group the epilogue warps read the group sums and
//     fold them into f32 totals in registers:
//        tot += scale * (acc - (offset + zero_point) * S),
//     which removes the 128 (+8 for s4) offset of the rebuilt nibbles and the
//     zero-point after the exact integer-weighted sum; results differ from
//     the reference's only by f32 summation order.
// Work decomposition is stream-K over (column tile, stage) units, one CTA per
// SM with equal byte counts; CTAs that share a column tile add their partial
// sums through a scratchpad in CTA order (deterministic), the last arriver
// runs the epilogue (bias, post-ops, store).  Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>

#include "device_math.cuh"
#include "launch.h"
#include "sm100_ptx.cuh"

namespace qmm {

namespace {

constexpr int CONV_WARPS = 8, EPI_WARPS = 4;
constexpr int WT_THREADS = 32 * (CONV_WARPS + EPI_WARPS + 2); // + TMA producer + MMA issuer
constexpr int W_STAGE_BYTES = 16384; // raw nibbles per stage
constexpr int A_SLOTS = 8; // operand slots in tensor memory, one k16 step each

// MR: src rows the epilogue reads (8, 16, 32); NBLK: 128-lane MMA blocks per column tile.
template <int MR, int NBLK>
struct WtCfg {
    static constexpr int MP = MR < 16 ? 16 : MR; // MMA N extent (a multiple of 16)
    static constexpr int NB = 128 * NBLK; // dst columns per tile
    static constexpr int ROW_BYTES = NB / 2; // packed bytes per k-row of a tile: 256 or 128
    static constexpr int KS = W_STAGE_BYTES / ROW_BYTES; // k-rows per stage: 64 or 128
    static constexpr int SPS = KS / 16; // k16 steps per stage
    static constexpr int W_BOXES = ROW_BYTES / 128; // TMA boxes [KS rows x 128 B] per stage
    static constexpr int S_BOXES = KS / 64; // src boxes [MP rows x 64 k] per stage
    static constexpr int S_BYTES = S_BOXES * MP * 128;
    static constexpr int STAGE_BYTES = W_STAGE_BYTES + ((S_BYTES + 1023) / 1024) * 1024;
    static constexpr int STAGES = NBLK == 4 ? 8 : 6;
    static constexpr int OUT_PITCH = NB + 8; // floats per row of the output tile in shared memory
    static constexpr int OUT_BYTES = MR * OUT_PITCH * 4;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES + OUT_BYTES;
    static constexpr int SMEM_BYTES = BAR_OFFSET + 512 + 1024;
    // tensor memory columns
    static constexpr int ACC_COLS = (NBLK + 1) * MP; // per buffer: NBLK result blocks + the S block
    static constexpr int A_COL0 = 2 * ACC_COLS;
    static constexpr int A_SLOT_COLS = 8 * NBLK;
    static constexpr int ONES_COL = A_COL0 + A_SLOTS * A_SLOT_COLS;
    static_assert(ONES_COL + 8 <= 512, "tensor memory");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};

struct WtParams {
    int M;
    int ksteps; // ceil(K / 16)
    int kstages; // ceil(K / KS)
    int group_steps; // k16 steps per quantization group (ksteps when not grouped along K)
    int ntiles; // column tiles
    int per; // (tile, stage) units per CTA
    int max_slots; // partial-sum slots per column tile
    int sgn4; // weights are s4 (else u4)
    int zp_mode; // 0 none, 1 per (group, column), 2 per tensor
    uint32_t idesc;
    float *partial; // [ntiles][max_slots][M * NB]
    int *counters; // [ntiles]
#ifdef QMM_PROFILE
    int ablate; // 1 no MMAs, 2 converters idle, 4 epilogue idle, 8 no S block, 16 unpack without stores (wrong results)
#endif
};
#ifdef QMM_PROFILE
#define WT_ABLATE(bit) (p.ablate & (bit))
#else
#define WT_ABLATE(bit) false
#endif

__device__ __forceinline__ uint32_t nib2(uint32_t x, uint32_t magic) { // (x & 0x000F000F) ^ magic
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000F000F, %2, 0x6a;" : "=r"(r) : "r"(x), "r"(magic));
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// 16 TMEM lanes x 8 columns: thread (g = lane / 4, t = lane % 4) supplies r0 = (lane g, column t),
// r1 = (lane g + 8, column t), r2 = (lane g, column 4 + t), r3 = (lane g + 8, column 4 + t)
__device__ __forceinline__ void tmem_st_16x128b_x2(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r0), "r"(r1),
                 "r"(r2), "r"(r3)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(v)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts_f16(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, bool acc) {
    const uint32_t en = acc ? 1u : 0u;
    asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
            "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(en)
            : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[N]) {
    if constexpr (N == 8) {
        ptx::tmem_ld_32x8(taddr, r);
    } else if constexpr (N == 16) {
        asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr)
                : "memory");
    } else {
        ptx::tmem_ld_32x32(taddr, r);
    }
}
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory"); }

// One segment of a CTA's range: stages [sb, se) of column tile `tile`.
struct Segment {
    int tile, sb, se;
};
__device__ __forceinline__ Segment segment_at(int64_t L, int64_t L1, int kstages) {
    Segment s;
    s.tile = (int)(L / kstages);
    s.sb = (int)(L - (int64_t)s.tile * kstages);
    const int64_t e = s.sb + (L1 - L);
    s.se = e < kstages ? (int)e : kstages;
    return s;
}

template <int MR, int NBLK, bool F16>
__global__ void __launch_bounds__(WT_THREADS, 1)
woq_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
        const __grid_constant__ MatmulArgs a, const __grid_constant__ WtParams p) {
    using C = WtCfg<MR, NBLK>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float *out_tile = (float *)(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t *full = (uint64_t *)(smem + C::BAR_OFFSET);
    uint64_t *empty = full + C::STAGES;
    uint64_t *a_full = empty + C::STAGES;
    uint64_t *a_empty = a_full + A_SLOTS;
    uint64_t *acc_full = a_empty + A_SLOTS;
    uint64_t *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = (uint32_t *)(acc_empty + 2);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    int *last_flag = (int *)(tmem_slot + 2);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < A_SLOTS; ++s) {
            ptx::mbar_init(&a_full[s], 4); // the four converter warps of one k16 step
            ptx::mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&acc_full[s], 1);
            ptx::mbar_init(&acc_empty[s], EPI_WARPS);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmW);
        ptx::prefetch_tensormap(&tmS);
    }
    if (warp == CONV_WARPS + EPI_WARPS + 1) ptx::tmem_alloc(tmem_slot, 512);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (warp < 4) { // the all-ones operand tile (its MMA yields the sum of the src values of a group)
        tmem_st_32x8(tmem_base + ((uint32_t)(32 * warp) << 16) + C::ONES_COL, F16 ? 0x3C003C00u : 0x3F803F80u);
        tmem_st_wait();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();

    const int64_t total = (int64_t)p.ntiles * p.kstages;
    const int64_t L0 = (int64_t)blockIdx.x * p.per;
    const int64_t L1 = L0 + p.per < total ? L0 + p.per : total;

    if (warp == CONV_WARPS + EPI_WARPS) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            for (int64_t L = L0; L < L1 && !*abort_flag;) {
                const Segment sg = segment_at(L, L1, p.kstages);
                const int xbyte = sg.tile * C::ROW_BYTES;
                for (int st = sg.sb; st < sg.se; ++st, ++it) {
                    const int s = it % C::STAGES;
                    if (!ptx::mbar_wait(&empty[s], ((it / C::STAGES) & 1) ^ 1)) { *abort_flag = 1; atomicExch(a.status, 5); break; }
                    uint8_t *sw = smem + s * C::STAGE_BYTES, *ss = sw + W_STAGE_BYTES;
                    ptx::mbar_arrive_expect_tx(&full[s], W_STAGE_BYTES + C::S_BYTES);
#pragma unroll
                    for (int b = 0; b < C::W_BOXES; ++b)
                        ptx::tma_load_2d(sw + b * (C::KS * 128), &tmW, &full[s], xbyte + b * 128, st * C::KS);
#pragma unroll
                    for (int b = 0; b < C::S_BOXES; ++b)
                        ptx::tma_load_2d(ss + b * (C::MP * 128), &tmS, &full[s], st * C::KS + b * 64, 0);
                }
                L += sg.se - sg.sb;
            }
        }
    } else if (warp == CONV_WARPS + EPI_WARPS + 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, ks = 0, gc = 0;
            bool failed = false;
            for (int64_t L = L0; L < L1 && !failed && !*abort_flag;) {
                const Segment sg = segment_at(L, L1, p.kstages);
                const int kend = min(sg.se * C::SPS, p.ksteps);
                int kpos = sg.sb * C::SPS;
                int gend = min(kend, (kpos / p.group_steps + 1) * p.group_steps); // end of the current group piece
                bool fresh = true; // the next MMA starts a group piece
                for (int st = sg.sb; st < sg.se && !failed; ++st, ++it) {
                    const int s = it % C::STAGES;
                    if (!ptx::mbar_wait(&full[s], (it / C::STAGES) & 1)) { failed = true; break; }
                    const uint32_t ss = ptx::smem_u32(smem + s * C::STAGE_BYTES + W_STAGE_BYTES);
                    const int nst = min(C::SPS, kend - st * C::SPS);
                    for (int q = 0; q < nst; ++q, ++ks, ++kpos) {
                        const uint32_t buf = gc & 1;
                        if (fresh && !ptx::mbar_wait(&acc_empty[buf], ((gc >> 1) & 1) ^ 1)) { failed = true; break; }
                        const int slot = ks % A_SLOTS;
                        if (!ptx::mbar_wait(&a_full[slot], (ks / A_SLOTS) & 1)) { failed = true; break; }
                        ptx::tc_fence_after_sync();
                        const uint64_t bd = ptx::smem_desc_sw128(ss + (q >> 2) * (C::MP * 128) + (q & 3) * 32, 0, 1024);
                        const uint32_t acc = tmem_base + buf * C::ACC_COLS;
                        const uint32_t asl = tmem_base + C::A_COL0 + slot * C::A_SLOT_COLS;
                        if (!WT_ABLATE(1)) {
#pragma unroll
                            for (int j = 0; j < NBLK; ++j) mma_ts_f16(acc + j * C::MP, asl + 8 * j, bd, p.idesc, !fresh);
                            if (!WT_ABLATE(8)) mma_ts_f16(acc + NBLK * C::MP, tmem_base + C::ONES_COL, bd, p.idesc, !fresh);
                        }
                        fresh = false;
                        ptx::tc_commit(&a_empty[slot]);
                        if (kpos + 1 == gend) { // group piece complete
                            ptx::tc_commit(&acc_full[buf]);
                            ++gc;
                            fresh = true;
                            gend = min(kend, gend + p.group_steps);
                        }
                    }
                    ptx::tc_commit(&empty[s]); // the stage's src tile has been read; the converters are through it too
                }
                L += sg.se - sg.sb;
            }
            if (failed) { *abort_flag = 1; atomicExch(a.status, 5); }
        }
    } else if (warp < CONV_WARPS) {
        // ------------------------------------------------ converters
        // Warp (q = warp % 4, r = warp / 4): TMEM lanes 32q..32q+31 of every block, k16 steps of parity r.
        // Its slice of a tile's k-row is the 16*NBLK bytes at 16*NBLK*q; lane (g, tig) owns 2*NBLK of them
        // (4*NBLK columns) and, per step, the k-rows 2tig, 2tig+1, 2tig+8, 2tig+9: exactly the registers
        // of the 16x128b.x2 store, byte t = 2j + h going to block j, lanes 32q + 16h + g (low nibble) and +8.
        const int q = warp & 3, r = warp >> 2;
        const int g = lane >> 2, tig = lane & 3;
        constexpr int BL = 2 * NBLK; // bytes per lane and k-row
        const int off = q * (16 * NBLK) + g * BL; // byte offset in the tile's k-row
        const uint32_t box_off = (uint32_t)(off >> 7) * (C::KS * 128);
        const uint32_t chunk = (off & 127) >> 4, within = off & 15;
        // 128B swizzle: 16-byte chunk index XOR (row & 7); rows 2tig (+8) and 2tig+1 (+8)
        const uint32_t lds0 = box_off + (2 * tig) * 128 + ((chunk ^ (uint32_t)(2 * tig)) << 4) + within;
        const uint32_t lds1 = box_off + (2 * tig + 1) * 128 + ((chunk ^ (uint32_t)(2 * tig + 1)) << 4) + within;
        const uint32_t magic = F16 ? (p.sgn4 ? 0x00080008u : 0u) : (p.sgn4 ? 0x43084308u : 0x43004300u);
        uint32_t it = 0, ks = 0;
        bool ok = true;
        for (int64_t L = L0; L < L1 && ok && !*abort_flag;) {
            const Segment sg = segment_at(L, L1, p.kstages);
            const int kend = min(sg.se * C::SPS, p.ksteps);
            for (int st = sg.sb; st < sg.se && ok; ++st, ++it) {
                const int s = it % C::STAGES;
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(&full[s], (it / C::STAGES) & 1))) { ok = false; break; }
                const uint8_t *sw = smem + s * C::STAGE_BYTES;
                const int nst = min(C::SPS, kend - st * C::SPS);
                for (int qs = 0; qs < nst; ++qs, ++ks) {
                    if ((qs & 1) != r) continue;
                    const int slot = ks % A_SLOTS;
                    if (WT_ABLATE(2)) {
                        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&a_empty[slot], ((ks / A_SLOTS) & 1) ^ 1))) { ok = false; break; }
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&a_full[slot]);
                        continue;
                    }
                    uint32_t R[4][BL / 4];
                    const uint8_t *b0 = sw + qs * 2048;
                    if constexpr (NBLK == 4) {
                        const uint2 v0 = *reinterpret_cast<const uint2 *>(b0 + lds0);
                        const uint2 v1 = *reinterpret_cast<const uint2 *>(b0 + lds1);
                        const uint2 v2 = *reinterpret_cast<const uint2 *>(b0 + lds0 + 1024);
                        const uint2 v3 = *reinterpret_cast<const uint2 *>(b0 + lds1 + 1024);
                        R[0][0] = v0.x; R[0][1] = v0.y; R[1][0] = v1.x; R[1][1] = v1.y;
                        R[2][0] = v2.x; R[2][1] = v2.y; R[3][0] = v3.x; R[3][1] = v3.y;
                    } else {
                        R[0][0] = *reinterpret_cast<const uint32_t *>(b0 + lds0);
                        R[1][0] = *reinterpret_cast<const uint32_t *>(b0 + lds1);
                        R[2][0] = *reinterpret_cast<const uint32_t *>(b0 + lds0 + 1024);
                        R[3][0] = *reinterpret_cast<const uint32_t *>(b0 + lds1 + 1024);
                    }
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait(&a_empty[slot], ((ks / A_SLOTS) & 1) ^ 1))) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    const uint32_t asl = tmem_base + ((uint32_t)(32 * q) << 16) + C::A_COL0 + slot * C::A_SLOT_COLS;
#pragma unroll
                    for (int t = 0; t < BL; ++t) {
                        // byte t of the four rows: low nibble = column 2t, high nibble = column 2t + 1
                        const uint32_t sel = ((4 + (t & 3)) << 12) | ((4 + (t & 3)) << 8) | ((t & 3) << 4) | (t & 3);
                        const uint32_t x01 = prmt(R[0][t >> 2], R[1][t >> 2], sel);
                        const uint32_t x23 = prmt(R[2][t >> 2], R[3][t >> 2], sel);
                        if (WT_ABLATE(16)) {
                            if ((nib2(x01, magic) ^ nib2(x01 >> 4, magic) ^ nib2(x23, magic) ^ nib2(x23 >> 4, magic)) == 0x12345u)
                                tmem_st_16x128b_x2(asl, x01, x23, x01, x23);
                            continue;
                        }
                        tmem_st_16x128b_x2(asl + ((uint32_t)(16 * (t & 1)) << 16) + 8 * (t >> 1), nib2(x01, magic),
                                nib2(x01 >> 4, magic), nib2(x23, magic), nib2(x23 >> 4, magic));
                    }
                    tmem_st_wait();
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&a_full[slot]);
                }
            }
            L += sg.se - sg.sb;
        }
        if (!ok) { *abort_flag = 1; atomicExch(a.status, 5); }
    } else {
        // ------------------------------------------------ epilogue warps
        // Warp q owns TMEM lanes 32q..32q+31; lane l = 16h + 8hi + g holds, for block j, the dst column
        // tile_n0 + 32*NBLK*q + 4*NBLK*g + 4j + 2h + hi.
        const int q = warp & 3;
        const int eh = lane >> 4, ehi = (lane >> 3) & 1, eg = lane & 7;
        const int col_in_tile = 32 * NBLK * q + 4 * NBLK * eg + 2 * eh + ehi;
        const int tid = threadIdx.x - CONV_WARPS * 32; // 0 .. 127
        const float off = (F16 ? 0.f : 128.f) + (p.sgn4 ? 8.f : 0.f);
        const float acc_scale = F16 ? 16777216.f : 1.f; // the f16 nibbles are u * 2^-24
        const float zt = p.zp_mode == 2 ? (float)load_int(a.wei_zp.dt, a.wei_zp.ptr, 0) : 0.f;
        float tot[NBLK][MR];
#pragma unroll
        for (int j = 0; j < NBLK; ++j)
#pragma unroll
            for (int m = 0; m < MR; ++m) tot[j][m] = 0.f;
        uint32_t gc = 0;
        // The four warps meet at named barriers, so none of them may leave the loops early: after an
        // expired wait (or once another role has given up) a warp skips its waits and tensor-memory
        // reads but still walks through every barrier; the status word tells the host that dst is invalid.
        bool ok = true;
        for (int64_t L = L0; L < L1;) {
            const Segment sg = segment_at(L, L1, p.kstages);
            const int64_t n_base = (int64_t)sg.tile * C::NB + col_in_tile;
            const int kend = min(sg.se * C::SPS, p.ksteps);
            int kpos = sg.sb * C::SPS;
            if (*abort_flag) ok = false;
            while (kpos < kend && ok) {
                const int gi = kpos / p.group_steps;
                const int gend = min(kend, (gi + 1) * p.group_steps);
                // parameters of this group for the lane's NBLK columns (in flight while waiting)
                float sc[NBLK], oz[NBLK];
#pragma unroll
                for (int j = 0; j < NBLK; ++j) {
                    const int64_t n = n_base + 4 * j;
                    sc[j] = 0.f;
                    oz[j] = 0.f;
                    if (n < a.N) {
                        sc[j] = load_float(a.wei_scale.dt, a.wei_scale.ptr,
                                        ((a.wei_scale.mask & 1) ? (int64_t)gi * a.wei_scale.ld : 0) + n)
                                * acc_scale;
                        float z = zt;
                        if (p.zp_mode == 1) z = (float)load_int(a.wei_zp.dt, a.wei_zp.ptr, (int64_t)gi * a.wei_zp.ld + n);
                        oz[j] = (off + z) / acc_scale;
                    }
                }
                const uint32_t buf = gc & 1;
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(&acc_full[buf], (gc >> 1) & 1))) { ok = false; break; } // leaves the group loop only
                ptx::tc_fence_after_sync();
                if (WT_ABLATE(4)) {
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
                    ++gc;
                    kpos = gend;
                    continue;
                }
                const uint32_t acc = tmem_base + ((uint32_t)(32 * q) << 16) + buf * C::ACC_COLS;
                uint32_t S[MR];
                tmem_ld_cols<MR>(acc + NBLK * C::MP, S);
#pragma unroll
                for (int j = 0; j < NBLK; ++j) {
                    uint32_t v[MR];
                    tmem_ld_cols<MR>(acc + j * C::MP, v);
                    ptx::tmem_ld_wait();
                    if (j == NBLK - 1) { // the buffer has been read: hand it back
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
                    }
#pragma unroll
                    for (int m = 0; m < MR; ++m)
                        tot[j][m] = fmaf(sc[j], fmaf(-oz[j], __uint_as_float(S[m]), __uint_as_float(v[m])), tot[j][m]);
                }
                ++gc;
                kpos = gend;
            }
            // ---- end of the segment: totals -> shared-memory tile [m][column] -> reduction across the
            // CTAs that share the column tile -> bias, post-ops, store
#pragma unroll
            for (int j = 0; j < NBLK; ++j)
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    if (m < p.M) out_tile[m * C::OUT_PITCH + col_in_tile + 4 * j] = tot[j][m];
                    tot[j][m] = 0.f;
                }
            epi_barrier();
            const int first = (int)(((int64_t)sg.tile * p.kstages) / p.per);
            const int last = (int)((((int64_t)sg.tile + 1) * p.kstages - 1) / p.per);
            const int nelem = p.M * C::NB;
            bool finalize = true;
            float *base = p.partial + ((int64_t)sg.tile * p.max_slots) * nelem;
            if (last > first) {
                const int count = last - first + 1, slot = (int)blockIdx.x - first;
                for (int i = tid; i < nelem; i += EPI_WARPS * 32)
                    base[(int64_t)slot * nelem + i] = out_tile[(i / C::NB) * C::OUT_PITCH + (i % C::NB)];
                __threadfence();
                epi_barrier();
                if (tid == 0) *last_flag = atomicAdd(&p.counters[sg.tile], 1) == count - 1;
                epi_barrier();
                finalize = *last_flag != 0;
                if (finalize) {
                    __threadfence();
                    if (tid == 0) p.counters[sg.tile] = 0; // ready for the next launch
                }
            }
            if (finalize) {
                float ssc = 1.f;
                if (a.src_scale.ptr) ssc = load_float(a.src_scale.dt, a.src_scale.ptr, 0);
                else if (a.src_scale.on_host) ssc = a.src_scale.host_value;
                const int count = last - first + 1;
                for (int i = tid; i < nelem; i += EPI_WARPS * 32) {
                    const int m = i / C::NB, c = i % C::NB;
                    const int64_t n = (int64_t)sg.tile * C::NB + c;
                    float v;
                    if (last > first) {
                        v = 0.f;
                        for (int sl = 0; sl < count; ++sl) v += __ldcg(base + (int64_t)sl * nelem + i);
                    } else {
                        v = out_tile[m * C::OUT_PITCH + c];
                    }
                    if (n < a.N) {
                        float d = v * ssc;
                        if (a.bias) d = __fadd_rn(d, load_float(a.bias_dt, a.bias, m * a.bias_sm + n * a.bias_sn));
                        finish_store(a, d, m, n, false);
                    }
                }
            }
            epi_barrier(); // the tile and the flag are reused by the next segment
            L += sg.se - sg.sb;
        }
        if (!ok) { *abort_flag = 1; atomicExch(a.status, 5); }
    }

    // ---------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == CONV_WARPS + EPI_WARPS + 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
        const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
        CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_tiled_fn wt_get_encode() {
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

// The cut of the (column tile, stage) space: `per` units per CTA, at most
// `max_slots` CTAs on one column tile.
struct WtPlan {
    int nblk, mr, ntiles, kstages, per, grid, max_slots;
};
WtPlan wt_plan(int64_t M, int64_t N, int64_t K, int sm_count) {
    WtPlan pl;
    pl.mr = M <= 8 ? 8 : (M <= 16 ? 16 : 32);
    pl.nblk = pl.mr == 32 ? 2 : 4;
    const int nb = 128 * pl.nblk, ks = W_STAGE_BYTES / (nb / 2);
    pl.ntiles = (int)((N + nb - 1) / nb);
    pl.kstages = (int)((K + ks - 1) / ks);
    const int64_t total = (int64_t)pl.ntiles * pl.kstages;
    if (sm_count < 1) sm_count = 148;
    int64_t per = (total + sm_count - 1) / sm_count;
    if (per < 4) per = 4; // a CTA is worth its launch
    pl.per = (int)per;
    pl.grid = (int)((total + per - 1) / per);
    pl.max_slots = (int)((pl.kstages + per - 1) / per) + 1;
    return pl;
}

template <int MR, int NBLK, bool F16>
int wt_launch(const CUtensorMap &tw, const CUtensorMap &ts, const MatmulArgs &a, const WtParams &p, int grid,
        cudaStream_t st) {
    using C = WtCfg<MR, NBLK>;
    auto kern = woq_tc_kernel<MR, NBLK, F16>;
    static std::atomic<unsigned long long> configured;
    if (!opt_in_dynamic_smem(kern, C::SMEM_BYTES, configured)) return 5;
    kern<<<grid, WT_THREADS, C::SMEM_BYTES, st>>>(tw, ts, a, p);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

} // namespace

size_t woq_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int sm_count) {
    const WtPlan pl = wt_plan(M, N, K, sm_count);
    return ((size_t)pl.ntiles * sizeof(int) + 255) / 256 * 256
            + (size_t)pl.ntiles * pl.max_slots * (size_t)M * (128 * pl.nblk) * sizeof(float);
}

bool woq_tc_pointers_ok(const MatmulArgs &a) {
    return (uintptr_t)a.wei % 16 == 0 && (uintptr_t)a.src % 16 == 0;
}

// `scratch`: woq_tc_scratch_bytes(...) bytes whose counters (the first
// ceil(N / tile) ints) are zero before the first launch; the kernel leaves
// them zero.
int launch_woq_tc(const MatmulArgs &a, void *scratch, int sm_count, cudaStream_t st) {
    if (a.M == 0 || a.N == 0) return 0;
    encode_tiled_fn enc = wt_get_encode();
    if (!enc || !scratch) return 5;
    const WtPlan pl = wt_plan(a.M, a.N, a.K, sm_count);
    const int nb = 128 * pl.nblk, ks = W_STAGE_BYTES / (nb / 2), mp = pl.mr < 16 ? 16 : pl.mr;
    CUtensorMap tw, ts;
    {
        cuuint64_t dims[2] = {(cuuint64_t)(a.N / 2), (cuuint64_t)a.K};
        cuuint64_t strides[1] = {(cuuint64_t)(a.wei_sk / 2)};
        cuuint32_t box[2] = {128, (cuuint32_t)ks};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(a.wei), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                != CUDA_SUCCESS)
            return 5;
    }
    {
        // src rows as 16-bit words; rows beyond M and k beyond K read as zeros
        cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
        cuuint64_t strides[1] = {(cuuint64_t)((a.M > 1 ? a.src_sm : a.K) * 2)};
        cuuint32_t box[2] = {64, (cuuint32_t)mp};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(a.src), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                != CUDA_SUCCESS)
            return 5;
    }
    WtParams p {};
    p.M = (int)a.M;
    p.ksteps = (int)((a.K + 15) / 16);
    p.kstages = pl.kstages;
    const int64_t group = (a.wei_scale.ptr && (a.wei_scale.mask & 1)) ? a.wei_scale.g0
            : (a.wei_zp.ptr && (a.wei_zp.mask & 1))                    ? a.wei_zp.g0
                                                                       : a.K;
    p.group_steps = (int)(group / 16);
    if (p.group_steps < 1 || p.group_steps > p.ksteps) p.group_steps = p.ksteps;
    p.ntiles = pl.ntiles;
    p.per = pl.per;
    p.max_slots = pl.max_slots;
    p.sgn4 = a.wei_dt == DT_S4;
    p.zp_mode = !a.wei_zp.ptr ? 0 : (a.wei_zp.mask ? 1 : 2);
    const bool f16 = a.src_dt == DT_F16;
    const uint32_t fmt = f16 ? ptx::FMT_F16 : ptx::FMT_BF16;
    p.idesc = ptx::make_idesc(ptx::CFMT_F32, fmt, fmt, false, false, 128, mp);
    p.counters = (int *)scratch;
    p.partial = (float *)((char *)scratch + ((size_t)pl.ntiles * sizeof(int) + 255) / 256 * 256);
#ifdef QMM_PROFILE // a build with -DQMM_PROFILE reads the switch; the shipped library has no such code
    p.ablate = getenv("ONEDNN_CUDA_WOQ_ABLATE") ? atoi(getenv("ONEDNN_CUDA_WOQ_ABLATE")) : 0;
#endif
#define QMM_WT(MR, NBLK) (f16 ? wt_launch<MR, NBLK, true>(tw, ts, a, p, pl.grid, st) : wt_launch<MR, NBLK, false>(tw, ts, a, p, pl.grid, st))
    if (pl.mr == 8) return QMM_WT(8, 4);
    if (pl.mr == 16) return QMM_WT(16, 4);
    return QMM_WT(32, 2);
#undef QMM_WT
}

} // namespace qmm
