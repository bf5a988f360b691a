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
// tcgen05.mma takes its A operand from TENSOR MEMORY, so the widened weights
// never pass through shared memory: TMA brings a raw [64 k x 128 n] s8 tile
// (128B-swizzled rows), converter warps read four k-rows of four columns per
// lane and k16 step, pair the k-rows with one PRMT, widen them to bf16 (exact:
// 8 significant bits) and write the stage's operand - 128 TMEM lanes x 32
// columns, the fragment layout of `tcgen05.st.16x128b` - with two stores per
// warp; `tcgen05.mma kind::f16` multiplies it with the src rows (K-major,
// straight from TMA).  Shared memory carries the raw bytes once in, once out,
// and the src rows; the bf16 copy (2 bytes per weight written and read again)
// is gone from it.  As in the 8-bit GEMM the kernel computes dst^T: weights
// are the A operand (128 dst columns = TMEM lanes), src rows the B operand, so
// an epilogue lane owns one dst column, keeps its scale in a register and
// stores coalesced rows.  Which column a TMEM lane holds is a permutation
// inside each group of 32 (lane 16h + 8i + g <-> column 4g + 2h + i), chosen
// so that a converter lane's four bytes go to the lanes its stores can reach.
//
// Tiles are (expert, 128 columns, up to 192 rows of that expert): two
// accumulator buffers of 192 columns and four operand slots of 32 fill the 512
// columns of tensor memory.  The MMA's N extent is the tile's row count
// rounded up to 16, so small experts cost little tensor time.  Tile order:
// expert, column block, row block fastest, so CTAs running together share
// weight tiles through L2.  A small planning kernel turns the offsets
// (cumulative END rows, validated like ref_grouped_gemm.cpp:164-213) into
// per-expert tile ranges on the device: no host synchronisation.  One
// persistent CTA per SM: warp 0 streams the raw weight tiles (ring of 8: they
// come from HBM), the last warp the src rows (ring of 6), warps 2-9 convert
// (two per lane quarter, alternating stages), warp 1 and the last three warps
// issue the MMAs (stage by stage, in turn), four warps run the epilogue.  The issuing loops are warp-uniform code whose
// tcgen05 / TMA instructions sit in a branch taken by one elected thread.  Every mbarrier wait is bounded.
#include <cuda.h>

#include "device_math.cuh"
#include "launch.h"
// waits of this kernel are long (a tile's mainloop, a ring that is full): let the hardware hold the
// polling thread for up to this many nanoseconds per poll (measured: 3 % on the fp8 GEMM)
#define QMM_TRY_WAIT_HINT_NS 2000
#include "sm100_ptx.cuh"

namespace qmm {

namespace {

constexpr int GT_N = 128; // dst columns per tile = TMEM lanes = UMMA M
constexpr int GT_M = 192; // most src rows per tile = UMMA N
constexpr int GK = 64; // k per stage: one 128-byte swizzle row of bf16 src
// Two shared-memory rings and one in tensor memory: the raw weights come from HBM (deep ring of small
// tiles to cover its latency), the src rows from L2, and the widened operand is produced and consumed
// on the SM (four slots of 32 columns beside the two accumulators).
constexpr int RAW_STAGES = 8, A_SLOTS = 4, B_STAGES = 6;
constexpr int RAW_BYTES = GK * GT_N; // s8 weights as loaded
constexpr int B_BYTES = GT_M * GK * 2; // src rows, K-major
constexpr int CONV_WARPS = 8, EPI_WARPS = 4;
constexpr int MMA_WARPS = 4; // issuers: stage s belongs to issuer s % MMA_WARPS
constexpr int G_THREADS = 32 * (3 + CONV_WARPS + EPI_WARPS + MMA_WARPS - 1);
constexpr int MMA_WARP1 = 3 + CONV_WARPS + EPI_WARPS; // the issuers after the first are the last warps
constexpr int ACC_STAGES = 2;
constexpr int A_SLOT_COLS = GK / 2; // two k per 32-bit column
constexpr int A_COL0 = ACC_STAGES * GT_M;
static_assert(A_COL0 + A_SLOTS * A_SLOT_COLS <= 512, "tensor memory");
constexpr int B_OFFSET = 0, RAW_OFFSET = B_OFFSET + B_STAGES * B_BYTES;
constexpr int G_BAR_OFFSET = RAW_OFFSET + RAW_STAGES * RAW_BYTES;
constexpr int PLAN_CACHE_GROUPS = 511; // records kept in shared memory (8 KB); more groups: read from global memory
constexpr int G_PLAN_OFFSET = G_BAR_OFFSET + 512;
constexpr int G_SMEM_BYTES = G_PLAN_OFFSET + (PLAN_CACHE_GROUPS + 1) * 16 + 1024;
static_assert(G_SMEM_BYTES <= 227 * 1024, "shared memory");

#ifdef QMM_PROFILE // builds with -DQMM_PROFILE stamp the SM clock of CTA 0 per role and stage; the shipped library has no such code
__device__ unsigned long long *g_grouped_trace = nullptr;
#define GT_TRACE(role, idx) do { if (g_grouped_trace && blockIdx.x == 0 && (idx) < 256) g_grouped_trace[(role) * 256 + (idx)] = (unsigned long long)clock64(); } while (0)
#else
#define GT_TRACE(role, idx) do { } while (0)
#endif

// plan[0] = {total tiles, groups, 0, 0}; plan[1 + g] = {first src row, first dst row, rows, first tile}
struct Tile {
    int g, n0, m0, rows, src_row, dst_row;
};
// (`plan` is the kernel's copy of the records in shared memory when they fit: every role looks a tile
// up when it begins it, and six dependent loads from global memory there cost microseconds per tile)
__device__ __forceinline__ Tile decode_tile(const int4 *plan, int groups, int num_n_tiles, int t) {
    int lo = 0, hi = groups; // last group whose first tile is <= t, skipping empty groups behind it
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (plan[1 + mid].w <= t) lo = mid; else hi = mid;
    }
    const int4 e = plan[1 + lo];
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
    asm volatile("griddepcontrol.launch_dependents;"); // the main kernel may set itself up meanwhile; it waits before it reads the plan
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

// 16 TMEM lanes x 32 columns (the four k16 steps of a stage): thread (g = lane / 4, t = lane % 4)
// supplies, for step s, r[4s] = (lane g, column 8s + t), r[4s + 1] = (lane g + 8, column 8s + t),
// r[4s + 2] = (lane g, column 8s + 4 + t), r[4s + 3] = (lane g + 8, column 8s + 4 + t)
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
            "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
            "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
            "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
            : "memory");
}
__device__ __forceinline__ void tmem_st_wait_() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]; executed by one (elected) thread
__device__ __forceinline__ void mma_ts_bf16(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, bool acc) {
    asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
            "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"((uint32_t)acc)
            : "memory");
}
// the dst column (inside its group of 32) that TMEM lane l holds
__device__ __forceinline__ int lane_column(int l) { return 4 * (l & 7) + 2 * (l >> 4) + ((l >> 3) & 1); }

// Sum over k of every src row (bf16), one warp per row: the factor of a weight zero-point,
// sum_k s (w - z) = sum_k s w - z sum_k s.
__global__ void grouped_rowsum_kernel(const __grid_constant__ MatmulArgs a, float *rowsum) {
    asm volatile("griddepcontrol.launch_dependents;");
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
        const __grid_constant__ CUtensorMap tmS2, const __grid_constant__ CUtensorMap tmS3,
        const __grid_constant__ MatmulArgs a, const int4 *plan_global, const float *rowsum, int num_n_tiles,
        int num_k_blocks) {
    constexpr uint32_t TMEM_COLS = 512;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *raw_full = (uint64_t *)(smem + G_BAR_OFFSET); // raw weight tile has landed
    uint64_t *raw_empty = raw_full + RAW_STAGES; // the converters have read it
    uint64_t *b_full = raw_empty + RAW_STAGES; // src rows have landed
    uint64_t *b_empty = b_full + B_STAGES; // the MMAs have read them
    uint64_t *a_full = b_empty + B_STAGES; // the stage's operand is in tensor memory
    uint64_t *a_empty = a_full + A_SLOTS; // the MMAs have read it
    uint64_t *tmem_full = a_empty + A_SLOTS;
    uint64_t *tmem_empty = tmem_full + ACC_STAGES;
    // stages whose MMAs are in the pipe (written by the two issuers in turn, read by the other)
    volatile uint32_t *stages_issued = (volatile uint32_t *)(tmem_empty + ACC_STAGES);
    uint32_t *tmem_base_slot = (uint32_t *)(tmem_empty + ACC_STAGES + 1);
    volatile int *abort_flag = (volatile int *)(tmem_base_slot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < RAW_STAGES; ++s) {
            ptx::mbar_init(&raw_full[s], 1);
            ptx::mbar_init(&raw_empty[s], CONV_WARPS / 2); // the stage's four converter warps
        }
        for (int s = 0; s < B_STAGES; ++s) {
            ptx::mbar_init(&b_full[s], 1);
            ptx::mbar_init(&b_empty[s], 1);
        }
        for (int s = 0; s < A_SLOTS; ++s) {
            ptx::mbar_init(&a_full[s], CONV_WARPS / 2);
            ptx::mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            ptx::mbar_init(&tmem_full[s], MMA_WARPS);
            ptx::mbar_init(&tmem_empty[s], EPI_WARPS);
        }
        *stages_issued = 0u;
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmW);
        ptx::prefetch_tensormap(&tmS);
        ptx::prefetch_tensormap(&tmS2);
        ptx::prefetch_tensormap(&tmS3);
    }
    if (warp == 1) ptx::tmem_alloc(tmem_base_slot, TMEM_COLS);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;
    // launched as the programmatic dependent of the planning (or row-sum) kernel: everything above ran
    // beside it; the plan and the row sums are read from here on
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int4 head = __ldg(&plan_global[0]);
    const int num_tiles = head.x, groups = head.y;
    const int4 *plan = plan_global;
    if (groups <= PLAN_CACHE_GROUPS) {
        int4 *cache = reinterpret_cast<int4 *>(smem + G_PLAN_OFFSET);
        for (int i = threadIdx.x; i <= groups; i += blockDim.x) cache[i] = __ldg(&plan_global[i]);
        __syncthreads();
        plan = cache;
    }

    if (warp == 0) {
        // ------------------------------------------------ TMA producer of the raw weight tiles
        // (the whole warp walks the loop, one elected thread issues: the addresses stay warp-uniform values)
        const bool issue = lane == 0;
        int s = 0;
        uint32_t ph = 1; // parity of the empty barrier's previous phase: a fresh barrier passes
        [[maybe_unused]] uint32_t pit = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok && !*abort_flag; t += gridDim.x) {
            const Tile tl = decode_tile(plan, groups, num_n_tiles, t);
            for (int kb = 0; kb < num_k_blocks; ++kb) {
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(&raw_empty[s], ph))) { ok = false; break; }
                if (ptx::elect_one()) {
                    ptx::mbar_arrive_expect_tx(&raw_full[s], RAW_BYTES);
                    ptx::tma_load_3d(smem + RAW_OFFSET + s * RAW_BYTES, &tmW, &raw_full[s], tl.n0, kb * GK, tl.g);
                }
                __syncwarp();
                if (issue) GT_TRACE(0, pit);
                ++pit;
                if (++s == RAW_STAGES) { s = 0; ph ^= 1; }
            }
        }
        if (!ok && issue) { *abort_flag = 1; atomicExch(a.status, 5); }
    } else if (warp == 2 + CONV_WARPS + EPI_WARPS) {
        // ------------------------------------------------ TMA producer of the src rows
        const bool issue = lane == 0;
        int s = 0;
        uint32_t ph = 1;
        [[maybe_unused]] uint32_t bit = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok && !*abort_flag; t += gridDim.x) {
            const Tile tl = decode_tile(plan, groups, num_n_tiles, t);
            // one copy per stage (issuing a copy costs this thread about as much as the wait): a box of
            // 64, 128 or 192 rows, whichever covers the tile's rows
            const int nbox = (tl.rows + 63) / 64;
            const CUtensorMap *tm = nbox == 1 ? &tmS : nbox == 2 ? &tmS2 : &tmS3;
            for (int kb = 0; kb < num_k_blocks; ++kb) {
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(&b_empty[s], ph))) { ok = false; break; }
                uint8_t *bt = smem + B_OFFSET + s * B_BYTES;
                if (ptx::elect_one()) {
                    ptx::mbar_arrive_expect_tx(&b_full[s], nbox * 64 * GK * 2);
                    ptx::tma_load_2d(bt, tm, &b_full[s], kb * GK, tl.src_row);
                }
                __syncwarp();
                if (issue) GT_TRACE(1, bit);
                ++bit;
                if (++s == B_STAGES) { s = 0; ph ^= 1; }
            }
        }
        if (!ok && issue) { *abort_flag = 1; atomicExch(a.status, 5); }
    } else if (warp == 1 || warp >= MMA_WARP1) {
        // ------------------------------------------------ MMA issuers (warp-uniform loops, an elected thread issues)
        // A warp issues an MMA every 40 to 65 cycles (twice that inside this kernel) and pays two waits
        // and two commits per stage, more than the MMAs of a stage take: four warps share the work,
        // stage by stage, waiting for their tiles and committing while another one issues.  The stages enter the pipe in their own order -
        // each issuer tells the other when its stage is in (a fence and a released store) - so the sums
        // are added in the same order every time and a second execution gives the same bits.
        const int me = warp == 1 ? 0 : warp - MMA_WARP1 + 1;
        const bool issue = lane == 0;
        int sa = 0, sb = 0;
        uint32_t pa = 0, pb = 0; // parities of the full barriers
        uint32_t acc_it = 0, it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok && !*abort_flag; t += gridDim.x, ++acc_it) {
            const Tile tl = decode_tile(plan, groups, num_n_tiles, t);
            const uint32_t n_mma = (uint32_t)max(16, (tl.rows + 15) & ~15);
            const uint32_t idesc = ptx::make_idesc(ptx::CFMT_F32, ptx::FMT_BF16, ptx::FMT_BF16, false, false, GT_N, n_mma);
            const int as = acc_it % ACC_STAGES;
            const uint32_t aph = (acc_it / ACC_STAGES) & 1;
            const uint32_t tmem_d = tmem_base + as * GT_M;
            for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
                if ((int)(it % MMA_WARPS) == me) {
                    if (kb == 0) { // the tile's first stage overwrites the accumulator: the epilogue must have read it
                        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&tmem_empty[as], aph ^ 1))) { ok = false; break; }
                    }
                    if (issue) GT_TRACE(2, it);
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait(&a_full[sa], pa))) { ok = false; break; }
                    if (issue) GT_TRACE(3, it);
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait(&b_full[sb], pb))) { ok = false; break; }
                    if (issue) GT_TRACE(4, it);
                    // the stage before this one (the other issuer's) is in the pipe: a word in shared memory,
                    // polled with plain loads (the hand-off is on the critical path of every stage, and a
                    // woken mbarrier wait costs several hundred cycles more)
                    {
                        uint32_t seen = ptx::ld_acquire_shared(stages_issued);
                        for (int spin = 0; seen < it && spin < (1 << 24); ++spin) seen = ptx::ld_acquire_shared(stages_issued);
                        if (!__all_sync(0xffffffffu, seen >= it)) { ok = false; break; }
                    }
                    ptx::tc_fence_after_sync();
                    if (issue) GT_TRACE(5, it);
                    // src rows K-major: 32 bytes of the row per MMA; the descriptor is built once per stage
                    // and advanced by a constant in its start-address field (16-byte units)
                    const uint64_t sd0 = ptx::smem_desc_sw128(ptx::smem_u32(smem + B_OFFSET + sb * B_BYTES), 0, 1024);
                    const uint32_t ta = tmem_base + A_COL0 + sa * A_SLOT_COLS;
                    if (ptx::elect_one()) { // one elected thread: see elect_one
#pragma unroll
                        for (int kk = 0; kk < GK / 16; ++kk)
                            mma_ts_bf16(tmem_d, ta + 8 * kk, sd0 + (uint64_t)(kk * (32 >> 4)), idesc, (kb | kk) != 0);
                        ptx::tc_fence_before_sync();
                        ptx::st_release_shared(stages_issued, it + 1);
                        // the operand slot and the src tile are reusable once these MMAs have read them
                        ptx::tc_commit(&a_empty[sa]);
                        ptx::tc_commit(&b_empty[sb]);
                    }
                    __syncwarp();
                    if (issue) GT_TRACE(6, it);
                }
                if (++sa == A_SLOTS) { sa = 0; pa ^= 1; }
                if (++sb == B_STAGES) { sb = 0; pb ^= 1; }
            }
            if (!ok) break;
            // this thread's share of the accumulator is complete (tcgen05.commit covers the MMAs of the
            // thread that executes it: the elected lane is the same one, the lowest, every time)
            if (ptx::elect_one()) ptx::tc_commit(&tmem_full[as]);
            __syncwarp();
        }
        if (!ok && issue) { *abort_flag = 1; atomicExch(a.status, 5); }
    } else if (warp < 2 + CONV_WARPS) {
        // ------------------------------------------------ converters: s8 tile -> bf16 operand in tensor memory
        // Warp (q = warp % 4, r): TMEM lanes 32q .. 32q+31, the stages of parity r.  Lane (g, t) reads,
        // per k16 step, the four bytes of columns 32q + 4g .. +3 in the k-rows 2t, 2t+1, 2t+8, 2t+9; byte
        // 2h + i of those goes to TMEM lane 32q + 16h + 8i + g, so one 16-lane store per h carries the
        // stage's four steps.
        const int q = warp & 3, r = (warp - 2) >> 2;
        const int g = lane >> 2, tq = lane & 3;
        const uint32_t chunk = (uint32_t)(2 * q + (g >> 2)), within = (uint32_t)(4 * (g & 3));
        // 128B swizzle of the raw rows: 16-byte chunk index XOR (row & 7)
        uint32_t off[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t row = 2 * tq + (i & 1) + 8 * (i >> 1);
            off[i] = row * 128 + ((chunk ^ (row & 7)) << 4) + within;
        }
        uint32_t it = 0;
        int sr = 0, sa = 0;
        uint32_t pr = 0, pa = 1;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok && !*abort_flag; t += gridDim.x) {
            for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
                if ((int)(it & 1) == r) {
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&raw_full[sr], pr))) { ok = false; break; }
                    if (warp == 2 && lane == 0) GT_TRACE(7, it);
                    const uint8_t *raw = smem + RAW_OFFSET + sr * RAW_BYTES;
                    uint32_t w[4][4]; // [step][k-row]
#pragma unroll
                    for (int st = 0; st < 4; ++st)
#pragma unroll
                        for (int i = 0; i < 4; ++i) w[st][i] = *reinterpret_cast<const uint32_t *>(raw + st * 2048 + off[i]);
                    // the stage's bytes are in registers: the producer may refill it
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&raw_empty[sr]);
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&a_empty[sa], pa))) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    if (warp == 2 && lane == 0) GT_TRACE(8, it);
                    const uint32_t slot = tmem_base + ((uint32_t)(32 * q) << 16) + A_COL0 + sa * A_SLOT_COLS;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t sel = h ? 0x7362u : 0x5140u; // [a.b(2h), b.b(2h), a.b(2h+1), b.b(2h+1)]
                        uint32_t o[16];
#pragma unroll
                        for (int st = 0; st < 4; ++st) {
                            s8x4_to_bf16x4(prmt_(w[st][0], w[st][1], sel), o[4 * st + 0], o[4 * st + 1]);
                            s8x4_to_bf16x4(prmt_(w[st][2], w[st][3], sel), o[4 * st + 2], o[4 * st + 3]);
                        }
                        tmem_st_16x128b_x8(slot + ((uint32_t)(16 * h) << 16), o);
                    }
                    tmem_st_wait_();
                    ptx::tc_fence_before_sync();
                    __syncwarp(); // every lane's stores to tensor memory are done
                    if (lane == 0) ptx::mbar_arrive(&a_full[sa]);
                    if (warp == 2 && lane == 0) GT_TRACE(9, it);
                }
                if (++sr == RAW_STAGES) { sr = 0; pr ^= 1; }
                if (++sa == A_SLOTS) { sa = 0; pa ^= 1; }
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
            const int64_t n = tl.n0 + lane_base + lane_column(lane);
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
    CUtensorMap tw, ts, ts2, ts3;
    { // weights as bytes [G][K][N]: raw tile of 64 k x 128 n, 128B swizzle; a dense [K][N] matrix is one group
        const int64_t groups = a.group_count > 0 ? a.group_count : 1;
        const int64_t group_pitch = a.group_count > 0 ? a.wei_sg : a.K * a.wei_sk;
        cuuint64_t dims[3] = {(cuuint64_t)a.N, (cuuint64_t)a.K, (cuuint64_t)groups};
        cuuint64_t strides[2] = {(cuuint64_t)a.wei_sk, (cuuint64_t)group_pitch};
        cuuint32_t box[3] = {GT_N, GK, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        if (enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(a.wei), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                != CUDA_SUCCESS)
            return 5;
    }
    // src as 16-bit words [M][K]: boxes of 64, 128 and 192 rows x 64 k, 128B swizzle
    CUtensorMap *src_maps[3] = {&ts, &ts2, &ts3};
    for (int i = 0; i < 3; ++i) {
        cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
        cuuint64_t strides[1] = {(cuuint64_t)(a.src_sm * 2)};
        cuuint32_t box[2] = {GK, (cuuint32_t)(64 * (i + 1))};
        cuuint32_t estr[2] = {1, 1};
        if (enc(src_maps[i], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(a.src), dims, strides, box, estr,
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
    {
        cudaLaunchConfig_t cfg {};
        cfg.gridDim = dim3((unsigned)(sm_count > 0 ? sm_count : 148));
        cfg.blockDim = dim3((unsigned)G_THREADS);
        cfg.dynamicSmemBytes = (size_t)G_SMEM_BYTES;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const int4 *plan_c = plan;
        const float *rowsum_c = rowsum;
        if (cudaLaunchKernelEx(&cfg, kern, tw, ts, ts2, ts3, a, plan_c, rowsum_c, num_n_tiles, num_k_blocks) != cudaSuccess) {
            (void)cudaGetLastError(); // the attribute was refused: an ordinary launch
            kern<<<sm_count > 0 ? sm_count : 148, G_THREADS, G_SMEM_BYTES, st>>>(tw, ts, ts2, ts3, a, plan, rowsum, num_n_tiles, num_k_blocks);
        }
    }
    count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

} // namespace qmm
