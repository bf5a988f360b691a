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
//     column = src row);
//   * at the end of every K-group the epilogue warps read the group sums and
//     fold them into f32 totals in registers:
//        tot += scale * (acc - (offset + zero_point) * S),   S[m] = sum_k src[m][k] of the group
//     which removes the 128 (+8 for s4) offset of the rebuilt nibbles and the
//     zero-point after the exact integer-weighted sum; results differ from the
//     reference's only by f32 summation order.  S comes from a small pre-kernel
//     (sums per k16 step); those sums, the scales and the zero-points of a
//     stage's groups travel by TMA in the same ring stage as the src tile, so
//     the epilogue never waits for a global load of its own (under this
//     kernel's load a load takes microseconds).
// The hand-offs are per stage, not per k-step: a converter warp fills its part
// of an operand stage in tensor memory (three of them, so that conversion,
// multiplication and the release of a stage overlap), arrives once, and frees
// the shared-memory stage with a plain arrive; the issuing thread's
// tcgen05.commit frees the operand stage and adds the last arrival to the
// shared-memory stage (its src tile).
// Work decomposition is stream-K over (column tile, stage) units, one CTA per
// SM with equal byte counts; CTAs that share a column tile add their partial
// sums through a scratchpad in CTA order (deterministic), the last arriver
// runs the epilogue (bias, post-ops, store).  Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>
#include <string>

#include "device_math.cuh"
#include "launch.h"
#include "objects.hpp"
#include "sm100_ptx.cuh"

namespace qmm {

namespace {

// A warp issues a tcgen05.mma about every 40 to 65 cycles, whatever its size; issuing warps add up,
// and the MMAs of this kernel are small (N = 16 or 32), so every 128-column block of a tile has an
// issuer warp of its own where the registers allow it (WtCfg::MMA_WARPS).
constexpr int CONV_WARPS = 8, EPI_WARPS = 4;
// A thread issues a stage of TMA copies in a few hundred cycles (a wait, an expect-tx and about 70
// cycles per copy), which is the time a stage may take: the weights and the rest (src tile, sums,
// scales, zero-points) have a producer thread each, in different warps.
constexpr int PRODUCER_WARP = CONV_WARPS + EPI_WARPS, PARAM_WARP = PRODUCER_WARP + 1, MMA_WARP0 = PARAM_WARP + 1;
constexpr int W_STAGE_BYTES = 16384; // raw nibbles per stage
constexpr int A_STAGES = 3; // operand stages in tensor memory, one shared-memory stage (128 columns) each

// MR: src rows the epilogue reads (8, 16, 32); NBLK: 128-lane MMA blocks per column tile.
template <int MR, int NBLK>
struct WtCfg {
    static constexpr int MP = MR < 16 ? 16 : MR; // MMA N extent (a multiple of 16)
    // Issuing warps: one per 128-column block where the epilogue's registers allow it.  Sixteen warps
    // may use 128 registers each; one more warp puts five on a scheduler, whose quarter of the
    // register file then gives 96 - enough for the 8-row epilogue only.
    static constexpr int MMA_WARPS = MR == 8 ? NBLK : 2;
    static constexpr int THREADS = 32 * (CONV_WARPS + EPI_WARPS + 2 + MMA_WARPS);
    static constexpr int NB = 128 * NBLK; // dst columns per tile
    static constexpr int ROW_BYTES = NB / 2; // packed bytes per k-row of a tile: 256 or 128
    static constexpr int KS = W_STAGE_BYTES / ROW_BYTES; // k-rows per stage: 64 or 128
    static constexpr int SPS = KS / 16; // k16 steps per stage
    static constexpr int W_BOXES = ROW_BYTES / 128; // TMA boxes [KS rows x 128 B] per stage
    static constexpr int S_BOXES = KS / 64; // src boxes [MP rows x 64 k] per stage
    static constexpr int S_BYTES = S_BOXES * MP * 128;
    // Two rings.  The weight stages are free again as soon as the converters have read them into
    // registers, so that ring's round trip is TMA latency plus a shared-memory read.  The other ring
    // carries, per stage, the src tile and the stage's parameters (step sums, scale and zero-point
    // rows of its groups); its stages are small, are freed by the MMAs and the epilogue, and their size
    // and number depend on the data types and the group size (WtParams).
    static constexpr int STAGES = NBLK == 4 ? 8 : 6; // weight stages
    static constexpr int S_STAGES_MAX = 16;
    static constexpr int SUMS_BYTES = SPS * MR * 4;
    static constexpr int OUT_OFFSET = STAGES * W_STAGE_BYTES;
    static constexpr int OUT_PITCH = NB + 8; // floats per row of the output tile in shared memory
    static constexpr int OUT_BYTES = MR * OUT_PITCH * 4;
    static constexpr int SSUM_BYTES = EPI_WARPS * 32 * 4; // per epilogue warp: S[m] of the current group
    static constexpr int BAR_OFFSET = OUT_OFFSET + OUT_BYTES + SSUM_BYTES;
    static constexpr int S_RING_OFFSET = ((BAR_OFFSET + 512 + 1023) / 1024) * 1024;
    static constexpr int SMEM_LIMIT = 227 * 1024 - 1024; // minus the alignment slack of the dynamic array
    // tensor memory columns: two accumulator buffers, then the operand stages
    static constexpr int ACC_COLS = NBLK * MP; // per buffer: NBLK result blocks
    static constexpr int A_COL0 = 2 * ACC_COLS;
    // an operand stage: [block][k16 step][8 columns of two k each]
    static constexpr int A_STAGE_COLS = NBLK * SPS * 8;
    static_assert(A_COL0 + A_STAGES * A_STAGE_COLS <= 512, "tensor memory");
    static_assert(S_RING_OFFSET + 6 * (S_BYTES + 1024) <= SMEM_LIMIT, "shared memory");
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
    int fast_store; // plain epilogue: no post-ops / dst scale, 16-bit or f32 dst rows that take 4-column vectors
    uint32_t idesc;
    float *partial; // [ntiles][max_slots][M * NB]
    int *counters; // [ntiles]
    const float *step_sums; // [ksteps][MR]: sum of the 16 src values of row m in k16 step k (pre-kernel)
    // the src / parameter ring: stage = src tile | step sums | scale rows | zero-point rows
    int s_stages, s_stage_bytes;
    int off_sums, off_sc, off_zp; // byte offsets inside a stage
    int sc_box_bytes, zp_box_bytes; // what one TMA copy of the rows brings
    int sc_row_bytes, zp_row_bytes; // pitch of a row of NB columns in shared memory
#ifdef QMM_PROFILE
    int ablate; // 1 no MMAs, 2 converters idle, 4 epilogue idle, 8 no S block, 16 unpack without stores (wrong results)
    unsigned long long *trace; // [role][256] globaltimer stamps of CTA 0 (role 0 producer, 1 MMA, 2 converter 0, 3 epilogue)
#endif
};
#ifdef QMM_PROFILE
#define WT_ABLATE(bit) (p.ablate & (bit))
#define WT_TRACE(role, idx) do { if (p.trace && blockIdx.x == 0 && (idx) < 256) p.trace[(role) * 256 + (idx)] = (unsigned long long)clock64(); } while (0)
#else
#define WT_ABLATE(bit) false
#define WT_TRACE(role, idx) do { } while (0)
#endif

__device__ __forceinline__ uint32_t nib2(uint32_t x, uint32_t magic) { // (x & 0x000F000F) ^ magic
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000F000F, %2, 0x6a;" : "=r"(r) : "r"(x), "r"(magic));
    return r;
}
__device__ __forceinline__ uint32_t nib2_hi(uint32_t x, uint32_t magic) { // (x & 0x00F000F0) ^ magic
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x00F000F0, %2, 0x6a;" : "=r"(r) : "r"(x), "r"(magic));
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// 16 TMEM lanes x 8 columns per k16 step: thread (g = lane / 4, t = lane % 4) supplies r0 = (lane g, column t),
// r1 = (lane g + 8, column t), r2 = (lane g, column 4 + t), r3 = (lane g + 8, column 4 + t);
// S consecutive k16 steps (8 columns each): 16 lanes x 8S columns in one instruction
template <int S>
__device__ __forceinline__ void tmem_st_16x128b_steps(uint32_t taddr, const uint32_t (&r)[4 * S]) {
    if constexpr (S == 4) {
        asm volatile(
                "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
                "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
                "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                : "memory");
    } else {
        static_assert(S == 8, "4 or 8 k16 steps per stage");
        asm volatile(
                "tcgen05.st.sync.aligned.16x128b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
                "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
                "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
                "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
                "r"(r[31])
                : "memory");
    }
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem], issued by the lane(s) with `issue` set
__device__ __forceinline__ void mma_ts_f16(bool issue, uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, bool acc) {
    const uint32_t en = acc ? 1u : 0u;
    asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
            "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
            "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(en), "r"((uint32_t)issue)
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
// The general store (post-ops, dst scale, any dst type) is rare and large: kept out of line so that
// the hot loops of the five roles stay close together in the instruction cache.
__device__ __noinline__ void finish_store_cold(const MatmulArgs &a, float d, int64_t m, int64_t n) {
    finish_store(a, d, m, n, false);
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
__global__ void __launch_bounds__((WtCfg<MR, NBLK>::THREADS), 1)
woq_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
        const __grid_constant__ CUtensorMap tmSums, const __grid_constant__ CUtensorMap tmSc,
        const __grid_constant__ CUtensorMap tmZp, const __grid_constant__ MatmulArgs a, const __grid_constant__ WtParams p) {
    using C = WtCfg<MR, NBLK>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float *out_tile = (float *)(smem + C::OUT_OFFSET);
    float *ssum_all = (float *)(smem + C::OUT_OFFSET + C::OUT_BYTES);
    uint64_t *full = (uint64_t *)(smem + C::BAR_OFFSET); // weight stages
    uint64_t *empty = full + C::STAGES;
    uint64_t *s_full = empty + C::STAGES; // src stages
    uint64_t *s_empty = s_full + C::S_STAGES_MAX;
    uint64_t *a_full = s_empty + C::S_STAGES_MAX;
    uint64_t *a_empty = a_full + A_STAGES;
    uint64_t *acc_full = a_empty + A_STAGES;
    uint64_t *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = (uint32_t *)(acc_empty + 2);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    int *last_flag = (int *)(tmem_slot + 2);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], CONV_WARPS / 2); // the stage's four converter warps
        }
        for (int s = 0; s < p.s_stages; ++s) {
            ptx::mbar_init(&s_full[s], 1);
            ptx::mbar_init(&s_empty[s], C::MMA_WARPS + EPI_WARPS); // the src tile and the parameters have been read
        }
        for (int s = 0; s < A_STAGES; ++s) {
            ptx::mbar_init(&a_full[s], CONV_WARPS / 2);
            ptx::mbar_init(&a_empty[s], C::MMA_WARPS);
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&acc_full[s], C::MMA_WARPS);
            ptx::mbar_init(&acc_empty[s], EPI_WARPS);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmW);
        ptx::prefetch_tensormap(&tmS);
        ptx::prefetch_tensormap(&tmSums);
        ptx::prefetch_tensormap(&tmSc);
        if (p.zp_mode == 1) ptx::prefetch_tensormap(&tmZp);
    }
    if (warp == MMA_WARP0) ptx::tmem_alloc(tmem_slot, 512);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t total = (int64_t)p.ntiles * p.kstages;
    const int64_t L0 = (int64_t)blockIdx.x * p.per;
    const int64_t L1 = L0 + p.per < total ? L0 + p.per : total;

    if (warp == PRODUCER_WARP) {
        // ------------------------------------------------ TMA producer
        // (the whole warp walks the loop, one elected thread issues: see elect_one)
        {
            const bool issue = lane == 0;
            uint32_t it = 0;
            int s = 0;
            uint32_t ph = 1; // parity of the empty barrier's previous phase: a fresh barrier passes
            bool ok = true;
            for (int64_t L = L0; L < L1 && ok && !*abort_flag;) {
                const Segment sg = segment_at(L, L1, p.kstages);
                const int xbyte = sg.tile * C::ROW_BYTES;
                for (int st = sg.sb; st < sg.se; ++st, ++it) {
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait(&empty[s], ph))) { ok = false; break; }
                    uint8_t *sw = smem + s * W_STAGE_BYTES;
                    if (ptx::elect_one()) {
                        ptx::mbar_arrive_expect_tx(&full[s], W_STAGE_BYTES);
#pragma unroll
                        for (int b = 0; b < C::W_BOXES; ++b)
                            ptx::tma_load_2d(sw + b * (C::KS * 128), &tmW, &full[s], xbyte + b * 128, st * C::KS);
                    }
                    __syncwarp();
                    if (issue) WT_TRACE(0, it);
                    if (++s == C::STAGES) { s = 0; ph ^= 1; }
                }
                L += sg.se - sg.sb;
            }
            if (!ok && issue) { *abort_flag = 1; atomicExch(a.status, 5); }
        }
    } else if (warp == PARAM_WARP) {
        // ------------------------------------------------ second producer: src tile, step sums and,
        // where a group piece can begin in the stage, the scale / zero-point rows of the stage's groups
        {
            const bool issue = lane == 0;
            int s = 0;
            uint32_t ph = 1;
            [[maybe_unused]] uint32_t pit = 0;
            const uint32_t base_tx = C::S_BYTES + C::SUMS_BYTES;
            const uint32_t par_tx = p.sc_box_bytes + (p.zp_mode == 1 ? p.zp_box_bytes : 0);
            // the step sums come from the pre-kernel, of which this kernel is the programmatic dependent
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            for (int64_t L = L0; L < L1 && ok && !*abort_flag;) {
                const Segment sg = segment_at(L, L1, p.kstages);
                const int xpair = sg.tile * (C::NB / 2); // parameter maps count pairs of columns
                int first = sg.sb * C::SPS;
                int gi0 = first / p.group_steps, r = first - gi0 * p.group_steps; // group of the stage's first step, steps into it
                for (int st = sg.sb; st < sg.se; ++st) {
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait(&s_empty[s], ph))) { ok = false; break; }
                    uint8_t *ss = smem + C::S_RING_OFFSET + s * p.s_stage_bytes;
                    const bool params = st == sg.sb || r == 0 || p.group_steps - r < C::SPS;
                    if (ptx::elect_one()) {
                        ptx::mbar_arrive_expect_tx(&s_full[s], base_tx + (params ? par_tx : 0u));
#pragma unroll
                        for (int b = 0; b < C::S_BOXES; ++b)
                            ptx::tma_load_2d(ss + b * (C::MP * 128), &tmS, &s_full[s], st * C::KS + b * 64, 0);
                        ptx::tma_load_2d(ss + p.off_sums, &tmSums, &s_full[s], 0, first);
                        if (params) {
                            ptx::tma_load_2d(ss + p.off_sc, &tmSc, &s_full[s], xpair, gi0);
                            if (p.zp_mode == 1) ptx::tma_load_2d(ss + p.off_zp, &tmZp, &s_full[s], xpair, gi0);
                        }
                    }
                    __syncwarp();
                    if (issue) WT_TRACE(12, pit);
                    ++pit;
                    first += C::SPS;
                    r += C::SPS;
                    while (r >= p.group_steps) { r -= p.group_steps; ++gi0; }
                    if (++s == p.s_stages) { s = 0; ph ^= 1; }
                }
                L += sg.se - sg.sb;
            }
            if (!ok && issue) { *abort_flag = 1; atomicExch(a.status, 5); }
        }
    } else if (warp >= MMA_WARP0) {
        // ------------------------------------------------ MMA issuers: warp i takes the column blocks
        // [i * NBLK / MMA_WARPS, (i + 1) * NBLK / MMA_WARPS) of every k16 step; all walk the same barriers
        constexpr int JB = NBLK / C::MMA_WARPS;
        const int j0 = (warp - MMA_WARP0) * JB;
        // (the whole warp walks the loop, one elected thread issues)
        {
            const bool issue = lane == 0;
            uint32_t it = 0, gc = 0;
            int s = 0, as = 0;
            uint32_t aph = 0; // parity of the operand-stage barriers
            bool failed = false;
            for (int64_t L = L0; L < L1 && !failed && !*abort_flag;) {
                const Segment sg = segment_at(L, L1, p.kstages);
                const int kend = min(sg.se * C::SPS, p.ksteps);
                int kpos = sg.sb * C::SPS;
                int gend = min(kend, (kpos / p.group_steps + 1) * p.group_steps); // end of the current group piece
                bool fresh = true; // the next MMA starts a group piece
                for (int st = sg.sb; st < sg.se && !failed; ++st, ++it) {
                    // (the converters have seen the stage's src tile arrive before they arrive here)
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait(&a_full[as], aph))) { failed = true; break; }
                    if (j0 == 0 && issue) WT_TRACE(5, it);
                    ptx::tc_fence_after_sync();
                    const uint32_t ss = ptx::smem_u32(smem + C::S_RING_OFFSET + s * p.s_stage_bytes);
                    const uint32_t ast = tmem_base + C::A_COL0 + as * C::A_STAGE_COLS;
                    const int nst = min(C::SPS, kend - st * C::SPS);
                    bool committed = false; // the straight-line path commits inside its elected branch
                    // The common stage - whole, inside one group piece - is straight-line code:
                    // descriptor and tensor-memory addresses are a base plus compile-time offsets.
                    if (nst == C::SPS && kpos + C::SPS <= gend && !WT_ABLATE(1)) {
                        const uint32_t buf = gc & 1;
                        if (fresh) {
                            if (!__all_sync(0xffffffffu, ptx::mbar_wait(&acc_empty[buf], ((gc >> 1) & 1) ^ 1))) { failed = true; break; }
                            ptx::tc_fence_after_sync();
                        }
                        if (j0 == 0 && issue) WT_TRACE(6, it);
                        const uint32_t accb = tmem_base + buf * C::ACC_COLS + j0 * C::MP;
                        const uint32_t astb = ast + j0 * (8 * C::SPS);
                        const uint64_t bd0 = ptx::smem_desc_sw128(ss, 0, 1024);
                        kpos += C::SPS;
                        const bool piece_done = kpos == gend;
                        if (ptx::elect_one()) { // one elected thread issues (see elect_one)
#pragma unroll
                            for (int q = 0; q < C::SPS; ++q) {
                                // the start-address field counts 16-byte units: later steps add a constant to it
                                const uint64_t bd = bd0 + (uint64_t)(((q >> 2) * (C::MP * 128) + (q & 3) * 32) >> 4);
#pragma unroll
                                for (int j = 0; j < JB; ++j)
                                    mma_ts_f16(true, accb + j * C::MP, astb + j * (8 * C::SPS) + 8 * q, bd, p.idesc, q > 0 || !fresh);
                            }
                            if (piece_done) ptx::tc_commit(&acc_full[buf]); // group piece complete
                            ptx::tc_commit(&a_empty[as]); // the operand stage may be rewritten once these MMAs have read it
                            ptx::tc_commit(&s_empty[s]); // ... and the stage's src tile has been read
                        }
                        __syncwarp();
                        fresh = false;
                        if (piece_done) {
                            ++gc;
                            fresh = true;
                            gend = min(kend, gend + p.group_steps);
                        }
                        committed = true;
                    } else {
                        for (int q = 0; q < nst; ++q, ++kpos) {
                            const uint32_t buf = gc & 1;
                            if (fresh) {
                                if (!__all_sync(0xffffffffu, ptx::mbar_wait(&acc_empty[buf], ((gc >> 1) & 1) ^ 1))) { failed = true; break; }
                                ptx::tc_fence_after_sync();
                            }
                            const uint64_t bd = ptx::smem_desc_sw128(ss + (q >> 2) * (C::MP * 128) + (q & 3) * 32, 0, 1024);
                            const uint32_t acc = tmem_base + buf * C::ACC_COLS;
                            if (!WT_ABLATE(1)) {
#pragma unroll
                                for (int j = 0; j < JB; ++j)
                                    mma_ts_f16(issue, acc + (j0 + j) * C::MP, ast + (j0 + j) * (8 * C::SPS) + 8 * q, bd, p.idesc, !fresh);
                            }
                            fresh = false;
                            if (kpos + 1 == gend) { // group piece complete
                                ptx::tc_commit_if(issue, &acc_full[buf]);
                                ++gc;
                                fresh = true;
                                gend = min(kend, gend + p.group_steps);
                            }
                        }
                    }
                    if (failed) break;
                    if (!committed) {
                        ptx::tc_commit_if(issue, &a_empty[as]); // the operand stage may be rewritten once these MMAs have read it
                        ptx::tc_commit_if(issue, &s_empty[s]); // ... and the stage's src tile has been read
                    }
                    if (j0 == 0 && issue) WT_TRACE(1, it);
                    if (++s == p.s_stages) s = 0;
                    if (++as == A_STAGES) { as = 0; aph ^= 1; }
                }
                L += sg.se - sg.sb;
            }
            if (failed && issue) { *abort_flag = 1; atomicExch(a.status, 5); }
        }
    } else if (warp < CONV_WARPS) {
        // ------------------------------------------------ converters
        // Warp (q = warp % 4, r = warp / 4): TMEM lanes 32q..32q+31 of every block, the stages of parity r
        // (two stages of a lane quarter are in flight at a time).  Its slice of a tile's k-row is the
        // 16*NBLK bytes at 16*NBLK*q; lane (g, tig) owns 2*NBLK of them (4*NBLK columns) and, per k16
        // step, the k-rows 2tig, 2tig+1, 2tig+8, 2tig+9: the registers of a 16x128b store, byte t = 2j + h
        // going to block j, lanes 32q + 16h + g (low nibble) and +8.  A tcgen05.st costs the same few
        // cycles of the SM's store pipe whatever its size, so one store carries all the k16 steps of a
        // stage for its 16 lanes (x8 or x16: four 32-bit columns per repetition, two repetitions per step).
        const int q = warp & 3, r = warp >> 2;
        const int g = lane >> 2, tig = lane & 3;
        constexpr int BL = 2 * NBLK; // bytes per lane and k-row
        const int off = q * (16 * NBLK) + g * BL; // byte offset in the tile's k-row
        const uint32_t box_off = (uint32_t)(off >> 7) * (C::KS * 128);
        const uint32_t chunk = (off & 127) >> 4, within = off & 15;
        // 128B swizzle: 16-byte chunk index XOR (row & 7); rows 2tig (+8) and 2tig+1 (+8)
        const uint32_t lds0 = box_off + (2 * tig) * 128 + ((chunk ^ (uint32_t)(2 * tig)) << 4) + within;
        const uint32_t lds1 = box_off + (2 * tig + 1) * 128 + ((chunk ^ (uint32_t)(2 * tig + 1)) << 4) + within;
        // bf16 src: a nibble u becomes the bf16 128 + u (shifted down to the mantissa's low bits first).
        // f16 src: a low nibble is the subnormal u * 2^-24 where it stands and a high nibble u * 2^-20,
        // no shift; the epilogue's per-column factor undoes the power of two.  (The operand must have
        // the src's format: an MMA with an f16 A and a bf16 B is an illegal instruction.)
        // s4: the sign bit flipped, u = w + 8.
        const uint32_t magic = F16 ? (p.sgn4 ? 0x00080008u : 0u) : (p.sgn4 ? 0x43084308u : 0x43004300u);
        const uint32_t magic_hi = p.sgn4 ? 0x00800080u : 0u;
        uint32_t it = 0;
        int s = 0, as = 0, rs = 0;
        uint32_t ph = 0, aph = 1, rph = 0;
        bool ok = true;
        for (int64_t L = L0; L < L1 && ok && !*abort_flag;) {
            const Segment sg = segment_at(L, L1, p.kstages);
            const int kend = min(sg.se * C::SPS, p.ksteps);
            for (int st = sg.sb; st < sg.se && ok; ++st, ++it) {
                if ((int)(it & 1) == r) {
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&full[s], ph))) { ok = false; break; }
                    const uint8_t *sw = smem + s * W_STAGE_BYTES;
                    const int nst = min(C::SPS, kend - st * C::SPS);
                    if (warp == 0 && lane == 0) WT_TRACE(2, it);
                    const uint32_t ast = tmem_base + ((uint32_t)(32 * q) << 16) + C::A_COL0 + as * C::A_STAGE_COLS;
                    if (!WT_ABLATE(2)) {
                        // the stage's raw bytes of this lane: [step][row 2tig, 2tig+1, 2tig+8, 2tig+9]; steps beyond
                        // K (the last stage of a ragged K) read the zeros TMA filled in
                        uint32_t R[C::SPS][4][BL / 4];
#pragma unroll
                        for (int qs = 0; qs < C::SPS; ++qs) {
                            const uint8_t *b0 = sw + qs * 2048;
                            if constexpr (NBLK == 4) {
                                const uint2 v0 = *reinterpret_cast<const uint2 *>(b0 + lds0);
                                const uint2 v1 = *reinterpret_cast<const uint2 *>(b0 + lds1);
                                const uint2 v2 = *reinterpret_cast<const uint2 *>(b0 + lds0 + 1024);
                                const uint2 v3 = *reinterpret_cast<const uint2 *>(b0 + lds1 + 1024);
                                R[qs][0][0] = v0.x; R[qs][0][1] = v0.y; R[qs][1][0] = v1.x; R[qs][1][1] = v1.y;
                                R[qs][2][0] = v2.x; R[qs][2][1] = v2.y; R[qs][3][0] = v3.x; R[qs][3][1] = v3.y;
                            } else {
                                R[qs][0][0] = *reinterpret_cast<const uint32_t *>(b0 + lds0);
                                R[qs][1][0] = *reinterpret_cast<const uint32_t *>(b0 + lds1);
                                R[qs][2][0] = *reinterpret_cast<const uint32_t *>(b0 + lds0 + 1024);
                                R[qs][3][0] = *reinterpret_cast<const uint32_t *>(b0 + lds1 + 1024);
                            }
                        }
                        // the stage's bytes are in registers: the producer may refill it
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&empty[s]);
                        if (!__all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&a_empty[as], aph))) { ok = false; break; }
                        ptx::tc_fence_after_sync();
                        if (warp == 0 && lane == 0) WT_TRACE(7, it);
#pragma unroll
                        for (int t = 0; t < BL; ++t) {
                            // byte t of every row: low nibble = column 2t, high nibble = column 2t + 1
                            const uint32_t sel = ((4 + (t & 3)) << 12) | ((4 + (t & 3)) << 8) | ((t & 3) << 4) | (t & 3);
                            uint32_t o[4 * C::SPS];
#pragma unroll
                            for (int qs = 0; qs < C::SPS; ++qs) {
                                const uint32_t x01 = prmt(R[qs][0][t >> 2], R[qs][1][t >> 2], sel);
                                const uint32_t x23 = prmt(R[qs][2][t >> 2], R[qs][3][t >> 2], sel);
                                o[4 * qs + 0] = nib2(x01, magic);
                                o[4 * qs + 1] = F16 ? nib2_hi(x01, magic_hi) : nib2(x01 >> 4, magic);
                                o[4 * qs + 2] = nib2(x23, magic);
                                o[4 * qs + 3] = F16 ? nib2_hi(x23, magic_hi) : nib2(x23 >> 4, magic);
                            }
                            // block j = t / 2 holds its SPS steps in consecutive columns; lanes 16 (t & 1) ...
                            tmem_st_16x128b_steps<C::SPS>(ast + ((uint32_t)(16 * (t & 1)) << 16) + (t >> 1) * (8 * C::SPS), o);
                        }
                        tmem_st_wait();
                    } else {
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&empty[s]);
                        if (!__all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&a_empty[as], aph))) { ok = false; break; }
                    }
                    // the MMA warps wait for the operand stage only: the stage's src tile must be there too
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&s_full[rs], rph))) { ok = false; break; }
                    ptx::tc_fence_before_sync();
                    __syncwarp(); // every lane's stores to tensor memory are done
                    if (lane == 0) ptx::mbar_arrive(&a_full[as]);
                    if (warp == 0 && lane == 0) WT_TRACE(8, it);
                }
                if (++s == C::STAGES) { s = 0; ph ^= 1; }
                if (++as == A_STAGES) { as = 0; aph ^= 1; }
                if (++rs == p.s_stages) { rs = 0; rph ^= 1; }
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
        float *ssum = ssum_all + q * 32;
        const float off = (F16 ? 0.f : 128.f) + (p.sgn4 ? 8.f : 0.f);
        // the f16 operand's nibbles are u * 2^-24 (low nibble) or u * 2^-20 (high nibble: this lane's column is odd)
        const float acc_scale = F16 ? (ehi ? 1048576.f : 16777216.f) : 1.f;
        const float zt = p.zp_mode == 2 ? (float)load_int(a.wei_zp.dt, a.wei_zp.ptr, 0) : 0.f;
        float tot[NBLK][MR];
#pragma unroll
        for (int j = 0; j < NBLK; ++j)
#pragma unroll
            for (int m = 0; m < MR; ++m) tot[j][m] = 0.f;
        uint32_t gc = 0;
        // The scales, zero-points and src sums of a piece come from the ring stage in which the piece
        // begins (TMA put them there with the src tile); sums of later stages are added as they arrive.
        // (one warp-uniform branch on the type, then NBLK loads)
        auto read_scales = [&](const uint8_t *rows, int row, float (&out)[NBLK]) {
            const uint8_t *e = rows + row * p.sc_row_bytes;
            if (a.wei_scale.dt == DT_BF16) {
#pragma unroll
                for (int j = 0; j < NBLK; ++j)
                    out[j] = __uint_as_float((uint32_t) reinterpret_cast<const unsigned short *>(e)[col_in_tile + 4 * j] << 16);
            } else if (a.wei_scale.dt == DT_F32) {
#pragma unroll
                for (int j = 0; j < NBLK; ++j) out[j] = reinterpret_cast<const float *>(e)[col_in_tile + 4 * j];
            } else {
#pragma unroll
                for (int j = 0; j < NBLK; ++j) out[j] = __half2float(reinterpret_cast<const __half *>(e)[col_in_tile + 4 * j]);
            }
        };
        auto read_zps = [&](const uint8_t *rows, int row, float (&out)[NBLK]) {
            const uint8_t *e = rows + row * p.zp_row_bytes;
            const int dt = a.wei_zp.dt;
            if (dt == DT_U4 || dt == DT_S4) { // tiles start at even columns: the nibble is the column's parity
                const uint32_t sh = (col_in_tile & 1) * 4, flip = dt == DT_S4 ? 8u : 0u;
#pragma unroll
                for (int j = 0; j < NBLK; ++j) {
                    const uint32_t v = (e[(col_in_tile + 4 * j) >> 1] >> sh) & 15u;
                    out[j] = (float)((int)(v ^ flip) - (int)flip);
                }
            } else if (dt == DT_U8) {
#pragma unroll
                for (int j = 0; j < NBLK; ++j) out[j] = (float)e[col_in_tile + 4 * j];
            } else if (dt == DT_S8) {
#pragma unroll
                for (int j = 0; j < NBLK; ++j) out[j] = (float)reinterpret_cast<const signed char *>(e)[col_in_tile + 4 * j];
            } else {
#pragma unroll
                for (int j = 0; j < NBLK; ++j) out[j] = (float)reinterpret_cast<const int *>(e)[col_in_tile + 4 * j];
            }
        };
        const float inv_acc_scale = 1.f / acc_scale; // a power of two
        // The four warps meet at named barriers, so none of them may leave the loops early: after an
        // expired wait (or once another role has given up) a warp skips its waits and tensor-memory
        // reads but still walks through every barrier; the status word tells the host that dst is invalid.
        bool ok = true;
        int rs = 0; // ring stage
        uint32_t rph = 0;
        [[maybe_unused]] uint32_t eit = 0;
        for (int64_t L = L0; L < L1;) {
            const Segment sg = segment_at(L, L1, p.kstages);
            const int kend = min(sg.se * C::SPS, p.ksteps);
            int kpos = sg.sb * C::SPS;
            if (*abort_flag) ok = false;
            float sc[NBLK], oz[NBLK], sm = 0.f;
            int gi = kpos / p.group_steps; // group of kpos
            int gend = kpos; // end of the open piece
            bool open = false;
            for (int st = sg.sb; st < sg.se && ok; ++st) {
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&s_full[rs], rph))) { ok = false; break; }
                if (tid == 0) WT_TRACE(9, eit);
                ++eit;
                const uint8_t *stage = smem + C::S_RING_OFFSET + rs * p.s_stage_bytes;
                const float *sums = reinterpret_cast<const float *>(stage + p.off_sums);
                const int first = st * C::SPS, k1 = min(kend, first + C::SPS);
                const int gi0 = gi; // kpos == first here: the group of the stage's first step
                bool released = false;
                while (kpos < k1 && ok) {
                    if (!open) { // a piece begins: its factors are in this stage
                        gend = min(kend, (gi + 1) * p.group_steps);
                        read_scales(stage + p.off_sc, gi - gi0, sc); // columns beyond N: zeros
                        if (p.zp_mode == 1) {
                            read_zps(stage + p.off_zp, gi - gi0, oz);
                        } else {
#pragma unroll
                            for (int j = 0; j < NBLK; ++j) oz[j] = zt;
                        }
#pragma unroll
                        for (int j = 0; j < NBLK; ++j) {
                            sc[j] *= acc_scale;
                            oz[j] = (off + oz[j]) * inv_acc_scale;
                        }
                        sm = 0.f;
                        open = true;
                    }
                    const int upto = min(gend, k1);
                    if (lane < MR) {
#pragma unroll
                        for (int i = 0; i < C::SPS; ++i)
                            if (first + i >= kpos && first + i < upto) sm += sums[i * MR + lane];
                    }
                    kpos = upto;
                    if (kpos < gend) break; // the piece goes on in the next stage
                    open = false;
                    if (gend == (gi + 1) * p.group_steps) ++gi; // (else: the segment ends inside the group)
                    ssum[lane] = sm; // S[m] of the piece
                    __syncwarp();
                    if (kpos == k1) { // nothing more to read in this stage: hand it back before folding
                        if (lane == 0) ptx::mbar_arrive(&s_empty[rs]);
                        released = true;
                    }
                    const uint32_t buf = gc & 1;
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&acc_full[buf], (gc >> 1) & 1))) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    if (tid == 0) WT_TRACE(10, eit - 1);
                    if (WT_ABLATE(4)) {
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
                    } else {
                        const uint32_t acc = tmem_base + ((uint32_t)(32 * q) << 16) + buf * C::ACC_COLS;
                        constexpr int MH = MR > 16 ? 16 : MR; // accumulator columns read at a time
#pragma unroll
                        for (int j = 0; j < NBLK; ++j) {
#pragma unroll
                            for (int h = 0; h < MR / MH; ++h) {
                                uint32_t v[MH];
                                tmem_ld_cols<MH>(acc + j * C::MP + h * MH, v);
                                ptx::tmem_ld_wait();
                                if (j == NBLK - 1 && h == MR / MH - 1) { // the buffer has been read: hand it back
                                    ptx::tc_fence_before_sync();
                                    __syncwarp();
                                    if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
                                }
#pragma unroll
                                for (int m = 0; m < MH; ++m)
                                    tot[j][h * MH + m] = fmaf(sc[j], fmaf(-oz[j], ssum[h * MH + m], __uint_as_float(v[m])), tot[j][h * MH + m]);
                            }
                        }
                    }
                    __syncwarp(); // ssum is rewritten for the next piece
                    if (tid == 0) WT_TRACE(11, eit - 1);
                    ++gc;
                }
                if (!ok) break;
                if (!released) {
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&s_empty[rs]);
                }
                if (++rs == p.s_stages) { rs = 0; rph ^= 1; }
            }
            // ---- end of the segment: totals -> shared-memory tile [m][column] -> reduction across the
            // CTAs that share the column tile -> bias, post-ops, store
            if (tid == 0) WT_TRACE(3, 2 * (gc & 63));
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
            constexpr int NB4 = C::NB / 4; // float4 groups per row: 128 or 64
            const int nvec = p.M * NB4;
            const int nelem = p.M * C::NB;
            const int count = last - first + 1;
            bool finalize = true;
            float4 *base = reinterpret_cast<float4 *>(p.partial + ((int64_t)sg.tile * p.max_slots) * nelem);
            if (count > 1) {
                const int slot = (int)blockIdx.x - first;
                for (int i = tid; i < nvec; i += EPI_WARPS * 32)
                    base[(int64_t)slot * nvec + i] = *reinterpret_cast<const float4 *>(out_tile + (i / NB4) * C::OUT_PITCH + (i % NB4) * 4);
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
                for (int i = tid; i < nvec; i += EPI_WARPS * 32) {
                    const int m = i / NB4, c = (i % NB4) * 4;
                    const int64_t n = (int64_t)sg.tile * C::NB + c;
                    float4 v;
                    if (count > 1) { // the slots in CTA order: the same sum whichever CTA arrives last
                        v = __ldcg(base + i);
                        float4 w1 = make_float4(0.f, 0.f, 0.f, 0.f), w2 = w1, w3 = w1;
                        if (count > 1) w1 = __ldcg(base + (int64_t)nvec + i);
                        if (count > 2) w2 = __ldcg(base + 2 * (int64_t)nvec + i);
                        if (count > 3) w3 = __ldcg(base + 3 * (int64_t)nvec + i);
                        v.x += w1.x; v.y += w1.y; v.z += w1.z; v.w += w1.w;
                        if (count > 2) { v.x += w2.x; v.y += w2.y; v.z += w2.z; v.w += w2.w; }
                        if (count > 3) { v.x += w3.x; v.y += w3.y; v.z += w3.z; v.w += w3.w; }
                        for (int sl = 4; sl < count; ++sl) {
                            const float4 w = __ldcg(base + (int64_t)sl * nvec + i);
                            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
                        }
                    } else {
                        v = *reinterpret_cast<const float4 *>(out_tile + m * C::OUT_PITCH + c);
                    }
                    float d[4] = {v.x * ssc, v.y * ssc, v.z * ssc, v.w * ssc};
                    if (p.fast_store && n + 3 < a.N) {
                        if (a.bias) {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                d[e] = __fadd_rn(d[e], load_float(a.bias_dt, a.bias, m * a.bias_sm + (n + e) * a.bias_sn));
                        }
                        const int64_t o = (int64_t)m * a.dst_sm + n;
                        if (a.dst_dt == DT_F32) {
                            *reinterpret_cast<float4 *>((float *)a.dst + o) = make_float4(d[0], d[1], d[2], d[3]);
                        } else if (a.dst_dt == DT_BF16) {
                            uint2 pk;
                            pk.x = (uint32_t)f32_to_bf16_bits(d[0]) | ((uint32_t)f32_to_bf16_bits(d[1]) << 16);
                            pk.y = (uint32_t)f32_to_bf16_bits(d[2]) | ((uint32_t)f32_to_bf16_bits(d[3]) << 16);
                            *reinterpret_cast<uint2 *>((unsigned short *)a.dst + o) = pk;
                        } else {
                            uint2 pk;
                            pk.x = (uint32_t)__half_as_ushort(__float2half_rn(d[0])) | ((uint32_t)__half_as_ushort(__float2half_rn(d[1])) << 16);
                            pk.y = (uint32_t)__half_as_ushort(__float2half_rn(d[2])) | ((uint32_t)__half_as_ushort(__float2half_rn(d[3])) << 16);
                            *reinterpret_cast<uint2 *>((unsigned short *)a.dst + o) = pk;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (n + e >= a.N) continue;
                            float de = d[e];
                            if (a.bias) de = __fadd_rn(de, load_float(a.bias_dt, a.bias, m * a.bias_sm + (n + e) * a.bias_sn));
                            finish_store_cold(a, de, m, n + e);
                        }
                    }
                }
            }
            epi_barrier(); // the tile and the flag are reused by the next segment
            if (tid == 0) WT_TRACE(3, 2 * (gc & 63) + 1);
            L += sg.se - sg.sb;
        }
        if (!ok) { *abort_flag = 1; atomicExch(a.status, 5); }
    }

    // ---------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP0) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}

// sums[k][m] = sum of src[m][16k .. 16k+15] (bf16 / f16), zero for m >= M: the S terms of the
// zero-point / offset correction at k16-step granularity; one thread per (k, m).
template <int MR, bool F16>
__global__ void woq_step_sums_kernel(const __grid_constant__ MatmulArgs a, float *sums, int ksteps) {
    // the main kernel is launched as this one's programmatic dependent: it may start now and set
    // itself up; the one warp of it that reads these sums waits for this grid first
    asm volatile("griddepcontrol.launch_dependents;");
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ksteps * MR) return;
    const int k = i / MR, m = i % MR;
    float s = 0.f;
    if (m < a.M) {
        const uint4 *ptr = reinterpret_cast<const uint4 *>((const char *)a.src + ((int64_t)m * a.src_sm + (int64_t)k * 16) * 2);
        const uint4 v0 = __ldg(ptr), v1 = __ldg(ptr + 1);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (F16) {
                const __half2 h = *reinterpret_cast<const __half2 *>(&w[e]);
                s += __low2float(h) + __high2float(h);
            } else {
                s += __uint_as_float(w[e] << 16) + __uint_as_float(w[e] & 0xffff0000u);
            }
        }
    }
    sums[i] = s;
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

struct WtMaps {
    CUtensorMap w, s, sums, sc, zp;
};

// Parameter rows as TMA sees them: elements of two columns each (1, 2, 4 or 8 bytes), so that a
// tile's 256 or 128 pairs fit the 256-element limit of a box; rows beyond the last group and
// columns beyond N read as zeros.
bool wt_encode_rows(encode_tiled_fn enc, CUtensorMap *tm, const void *ptr, int bits, int64_t ncols, int64_t nrows,
        int64_t ld, int nb, int box_rows) {
    const int pair_bytes = 2 * bits / 8;
    const CUtensorMapDataType dt = pair_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
            : pair_bytes == 2                     ? CU_TENSOR_MAP_DATA_TYPE_UINT16
            : pair_bytes == 4                     ? CU_TENSOR_MAP_DATA_TYPE_UINT32
                                                  : CU_TENSOR_MAP_DATA_TYPE_UINT64;
    int64_t pitch = ld * bits / 8;
    if (nrows <= 1) pitch = (ncols * bits / 8 + 15) / 16 * 16; // unused, but checked
    cuuint64_t dims[2] = {(cuuint64_t)(ncols / 2), (cuuint64_t)nrows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch};
    cuuint32_t box[2] = {(cuuint32_t)(nb / 2), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(tm, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            == CUDA_SUCCESS;
}

int wt_bits(int dt) {
    switch (dt) {
        case DT_F32: case DT_S32: return 32;
        case DT_BF16: case DT_F16: return 16;
        case DT_S8: case DT_U8: return 8;
        default: return 4;
    }
}

// Rows of a parameter that one stage can need: the groups its k16 steps touch.
int wt_rows_per_stage(int group_steps, int sps) {
    if (group_steps % sps == 0) return 1;
    if (sps % group_steps == 0) return sps / group_steps;
    return (sps + group_steps - 2) / group_steps + 1;
}

// The src / parameter ring takes the shared memory the fixed parts leave: sizes and offsets of a stage
// and the number of stages.  False when fewer than four stages fit (small groups with wide parameter
// types): such problems are left to the next implementation when the descriptor is created.
template <int MR, int NBLK>
bool wt_ring_layout(int group_steps, int sc_bits, int zp_bits, WtParams &p) {
    using C = WtCfg<MR, NBLK>;
    const int rb = wt_rows_per_stage(group_steps, C::SPS);
    auto up128 = [](int v) { return (v + 127) / 128 * 128; };
    p.sc_row_bytes = C::NB * sc_bits / 8;
    p.zp_row_bytes = C::NB * zp_bits / 8;
    p.sc_box_bytes = rb * p.sc_row_bytes;
    p.zp_box_bytes = rb * p.zp_row_bytes;
    p.off_sums = C::S_BYTES;
    p.off_sc = p.off_sums + up128(C::SUMS_BYTES);
    p.off_zp = p.off_sc + up128(p.sc_box_bytes);
    p.s_stage_bytes = (p.off_zp + up128(p.zp_box_bytes) + 1023) / 1024 * 1024;
    p.s_stages = (C::SMEM_LIMIT - C::S_RING_OFFSET) / p.s_stage_bytes;
    if (p.s_stages > C::S_STAGES_MAX) p.s_stages = C::S_STAGES_MAX;
    return p.s_stages >= 4 && rb <= 256;
}

template <int MR, int NBLK, bool F16>
int wt_launch(encode_tiled_fn enc, WtMaps &tm, const MatmulArgs &a, WtParams &p, int grid, cudaStream_t st) {
    using C = WtCfg<MR, NBLK>;
    auto kern = woq_tc_kernel<MR, NBLK, F16>;
    const int ngroups = (p.ksteps + p.group_steps - 1) / p.group_steps;
    const int sc_bits = wt_bits(a.wei_scale.dt), zp_bits = p.zp_mode == 1 ? wt_bits(a.wei_zp.dt) : 0;
    const int rb = wt_rows_per_stage(p.group_steps, C::SPS);
    if (!wt_ring_layout<MR, NBLK>(p.group_steps, sc_bits, zp_bits, p)) {
        set_last_error("cuda:tcgen05:woq4: the parameter rows of a stage do not fit in shared memory");
        return 5;
    }
    const int smem_bytes = C::S_RING_OFFSET + p.s_stages * p.s_stage_bytes + 1024;
    {
        cuuint64_t dims[2] = {(cuuint64_t)MR, (cuuint64_t)p.ksteps};
        cuuint64_t strides[1] = {(cuuint64_t)(MR * 4)};
        cuuint32_t box[2] = {(cuuint32_t)MR, (cuuint32_t)C::SPS};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&tm.sums, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(p.step_sums), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                != CUDA_SUCCESS)
            return 5;
    }
    if (!wt_encode_rows(enc, &tm.sc, a.wei_scale.ptr, sc_bits, a.N, (a.wei_scale.mask & 1) ? ngroups : 1, a.wei_scale.ld, C::NB, rb))
        return 5;
    tm.zp = tm.sc;
    if (p.zp_mode == 1 && !wt_encode_rows(enc, &tm.zp, a.wei_zp.ptr, zp_bits, a.N, ngroups, a.wei_zp.ld, C::NB, rb)) return 5;
    static std::atomic<unsigned long long> configured;
    if (!opt_in_dynamic_smem(kern, 227 * 1024, configured)) return 5;
    const int nsum = p.ksteps * MR;
    woq_step_sums_kernel<MR, F16><<<(nsum + 255) / 256, 256, 0, st>>>(a, const_cast<float *>(p.step_sums), p.ksteps);
    {
        // programmatic dependent launch: the kernel's set-up (barriers, tensor memory, descriptor
        // prefetch) and its weight stream overlap the pre-kernel
        cudaLaunchConfig_t cfg {};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3((unsigned)C::THREADS);
        cfg.dynamicSmemBytes = (size_t)smem_bytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, kern, tm.w, tm.s, tm.sums, tm.sc, tm.zp, a, p) != cudaSuccess) {
            (void)cudaGetLastError(); // the attribute was refused: an ordinary launch (the waits in the kernels are no-ops then)
            kern<<<grid, C::THREADS, smem_bytes, st>>>(tm.w, tm.s, tm.sums, tm.sc, tm.zp, a, p);
        }
    }
    count_launch(2);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error(std::string("cuda:tcgen05:woq4 launch: ") + cudaGetErrorString(e));
        return 5;
    }
    return 0;
}

} // namespace

// counters | src step sums [ceil(K/16)][MR] | split-K partial sums
static size_t wt_sums_offset(const WtPlan &pl) { return ((size_t)pl.ntiles * sizeof(int) + 255) / 256 * 256; }
static size_t wt_partial_offset(const WtPlan &pl, int64_t K) {
    return wt_sums_offset(pl) + (((size_t)((K + 15) / 16) * pl.mr * sizeof(float)) + 255) / 256 * 256;
}
size_t woq_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int sm_count) {
    const WtPlan pl = wt_plan(M, N, K, sm_count);
    return wt_partial_offset(pl, K) + (size_t)pl.ntiles * pl.max_slots * (size_t)M * (128 * pl.nblk) * sizeof(float);
}

// Whether the kernel's shared-memory plan holds the problem: `group` = K-group of the weight
// parameters (K when there is none), scale / zero-point data types as DT_* (zp_dt < 0: no per-group
// zero-points).
bool woq_tc_fits(int64_t M, int64_t K, int64_t group, int scale_dt, int zp_dt) {
    WtParams p {};
    const int ksteps = (int)((K + 15) / 16);
    int gs = (int)(group / 16);
    if (gs < 1 || gs > ksteps) gs = ksteps;
    const int sc_bits = wt_bits(scale_dt), zp_bits = zp_dt < 0 ? 0 : wt_bits(zp_dt);
    if (M <= 8) return wt_ring_layout<8, 4>(gs, sc_bits, zp_bits, p);
    if (M <= 16) return wt_ring_layout<16, 4>(gs, sc_bits, zp_bits, p);
    return wt_ring_layout<32, 2>(gs, sc_bits, zp_bits, p);
}

bool woq_tc_pointers_ok(const MatmulArgs &a) {
    return (uintptr_t)a.wei % 16 == 0 && (uintptr_t)a.src % 16 == 0 && (uintptr_t)a.wei_scale.ptr % 16 == 0
            && (uintptr_t)a.wei_zp.ptr % 16 == 0;
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
    WtMaps tm;
    CUtensorMap &tw = tm.w, &ts = tm.s;
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
    {
        const int es = a.dst_dt == DT_F32 ? 4 : 2;
        p.fast_store = a.n_po == 0 && !a.dst_scale.ptr && !a.dst_scale.on_host
                && (a.dst_dt == DT_F32 || a.dst_dt == DT_BF16 || a.dst_dt == DT_F16) && a.dst_sn == 1
                && (a.dst_sm * es) % (4 * es) == 0 && (uintptr_t)a.dst % (4 * es) == 0;
    }
    const bool f16 = a.src_dt == DT_F16;
    const uint32_t fmt = f16 ? ptx::FMT_F16 : ptx::FMT_BF16;
    p.idesc = ptx::make_idesc(ptx::CFMT_F32, fmt, fmt, false, false, 128, mp);
    p.counters = (int *)scratch;
    p.step_sums = (const float *)((char *)scratch + wt_sums_offset(pl));
    p.partial = (float *)((char *)scratch + wt_partial_offset(pl, a.K));
#ifdef QMM_PROFILE // a build with -DQMM_PROFILE reads the switch; the shipped library has no such code
    p.ablate = getenv("ONEDNN_CUDA_WOQ_ABLATE") ? atoi(getenv("ONEDNN_CUDA_WOQ_ABLATE")) : 0;
    p.trace = getenv("ONEDNN_CUDA_WOQ_TRACE") ? (unsigned long long *)strtoull(getenv("ONEDNN_CUDA_WOQ_TRACE"), nullptr, 16) : nullptr;
#endif
#define QMM_WT(MR, NBLK) (f16 ? wt_launch<MR, NBLK, true>(enc, tm, a, p, pl.grid, st) : wt_launch<MR, NBLK, false>(enc, tm, a, p, pl.grid, st))
    if (pl.mr == 8) return QMM_WT(8, 4);
    if (pl.mr == 16) return QMM_WT(16, 4);
    return QMM_WT(32, 2);
#undef QMM_WT
}

} // namespace qmm
