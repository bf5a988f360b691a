// "cuda:woq:skinny": weight-decompression matmul for few rows (decode):
// dst[M,N] = src[M,K] (bf16/f16) x dequant(weights[K,N] s4/u4), 8 rows per
// pass, scales per column or per (K-group, column), optional zero-points
// (fpmath apply_to_int).
//
// The problem is bound by the HBM stream of the packed weights (half a byte
// per element), and at B200 bandwidth a CUDA-core FMA per weight plus its
// int4->float conversion would exceed the instruction budget (about 2
// lane-operations per weight).  So the multiply-accumulate runs on the tensor
// cores (mma.sync m16n8k16: weights as the 16-row operand, src rows as the
// 8-column operand) and the lanes only rebuild operand registers:
//   * bf16: a nibble u becomes 128+u by OR-ing it into the mantissa of 0x4300;
//     f16: u itself is the subnormal u*2^-24.  One LOP3 per two weights, exact.
//   * the offset and the zero-point leave after the K-group has been summed:
//     sum_k s_k (w_k - zp) scale = scale * (sum_k s_k w'_k - (off + zp) sum_k s_k)
//     in f32, so no rounding of scaled weights is involved (the reference
//     scales each weight in f32, src/cpu/matmul/ref_matmul.cpp:193-214;
//     results differ from it only by f32 summation order).
// Work decomposition ("stream-K"): the (column block, k-step) space is cut
// into one contiguous, equally long range per CTA, one CTA per SM, so every
// SM streams the same number of bytes.  A column block is 256 columns; inside
// a range the 16 warps form 8 pairs that take consecutive k sub-ranges, the
// two warps of a pair side by side on 128 columns each.  Every warp feeds
// itself through its own ring of TMA stages (32 k-rows x 64 bytes, 64B
// swizzle) and keeps only the running group sums in registers: the scaled
// totals live in shared memory, which keeps the kernel under 128 registers
// so that 16 warps hide each other's latencies.  Where several CTAs share a
// column block their partial sums go to a global scratch and the last arriver
// adds them in CTA order (deterministic) and runs the epilogue.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>

#include "device_math.cuh"
#include "launch.h"
#include "sm100_ptx.cuh"

// Profiling aid: -DWOQ_ABLATE=<bits> compiles parts of the kernel out (1 dequantization and MMAs,
// 2 group-end arithmetic, 4 src loads, 8 shared-memory reads, 16 reduction and epilogue) so that
// instruction counts and times of the rest can be measured.  Results are wrong unless it is 0.
#ifndef WOQ_ABLATE
#define WOQ_ABLATE 0
#endif

namespace qmm {

namespace {

constexpr int WARPS = 16;
constexpr int PAIRS = WARPS / 2;
constexpr int STAGES = 4; // per warp
constexpr int STAGE_BYTES = 32 * 64; // 32 k-rows (two MMA k-steps) of 128 packed columns
constexpr int NB = 256; // dst columns per column block
constexpr int MB = 8; // src rows per pass (the MMA's n extent)
constexpr int RING_BYTES = WARPS * STAGES * STAGE_BYTES;
constexpr int TOT_BYTES = WARPS * 8 * 32 * 16; // per warp: [8 column pairs][32 lanes] float4
constexpr int SMEM_BYTES = RING_BYTES + TOT_BYTES + WARPS * STAGES * 8 + 64 + 1024;

struct WoqParams {
    int M; // rows of this pass (<= 8)
    int64_t m_base; // first src/dst row of this pass
    int ksteps; // K / 16
    int group_steps; // k-steps per quantization group; ksteps when not grouped along K
    int nblk; // column blocks
    int per; // (column block, k-step) pairs per CTA
    int max_slots; // partial-sum slots per column block
    int sgn4; // weights are s4 (else u4)
    int zp_mode; // 0 none, 1 per (group, n), 2 per tensor
    float4 *partial; // [nblk][max_slots][512]
    int *counters; // [nblk]
    // zero-point correction through the tensor cores (ZPMMA kernels)
    uint32_t magic_z; // turns a zero-point nibble pair into bf16 (128 [+ 8] + z)
    uint32_t az_const; // bf16 pair of the offset when there are no per-group zero-points
    uint32_t az_diff; // bf16 pair of (weight offset - zero-point offset): 0, 8 or -8
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (x & 0x000F000F) ^ magic : two nibbles -> two 16-bit floats
__device__ __forceinline__ uint32_t nib2(uint32_t x, uint32_t magic) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x000F000F, %2, 0x6a;" : "=r"(r) : "r"(x), "r"(magic));
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
template <bool F16>
__device__ __forceinline__ float pair_sum(uint32_t v) {
    if (F16) {
        const __half2 h = *reinterpret_cast<const __half2 *>(&v);
        return __low2float(h) + __high2float(h);
    }
    return __uint_as_float(v << 16) + __uint_as_float(v & 0xffff0000u);
}
// Read-only loads that stay where they are written (issued well ahead of
// their use; a plain load may be moved down to the use and stalls the warp there)
__device__ __forceinline__ uint4 ldg_v4_here(const void *ptr) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}
__device__ __forceinline__ uint2 ldg_v2_here(const void *ptr) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr));
    return v;
}
__device__ __forceinline__ uint32_t ldg_u32_here(const void *ptr) {
    uint32_t v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(ptr));
    return v;
}

// ZPMMA (bf16 src; no zero-points or 4-bit ones per group): the zero-point
// correction runs on the tensor cores; otherwise FMAs apply it when a group ends.
template <bool F16, bool ZPMMA>
__global__ void __launch_bounds__(WARPS * 32, 1)
woq_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ MatmulArgs a,
        const __grid_constant__ WoqParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float4 *tot_all = reinterpret_cast<float4 *>(smem + RING_BYTES);
    uint64_t *bars = (uint64_t *)(smem + RING_BYTES + TOT_BYTES);
    int *flag = (int *)(bars + WARPS * STAGES);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g = lane >> 2, tig = lane & 3;
    const int pair = warp >> 1, half = warp & 1;
    uint8_t *ring = smem + warp * STAGES * STAGE_BYTES;
    uint64_t *full = bars + warp * STAGES;
    float4 *tot_s = tot_all + warp * 256 + lane; // element t at tot_s[32 t]
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) ptx::mbar_init(&full[s], 1);
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&tmW);
    }
    __syncwarp();

    // bf16: nibble u -> 128+u.  f16: u alone is the subnormal u * 2^-24 (exact in the MMA), so only the
    // s4 bias of 8 remains as offset and the group sum is rescaled by 2^24.
    const uint32_t magic = F16 ? (p.sgn4 ? 0x00080008u : 0u) : (p.sgn4 ? 0x43084308u : 0x43004300u);
    const float off = (F16 ? 0.f : 128.f) + (p.sgn4 ? 8.f : 0.f);
    const float acc_scale = F16 ? 16777216.f : 1.f;
    const bool sc_bf16 = a.wei_scale.dt == DT_BF16;
    const bool zp4 = p.zp_mode == 1 && (a.wei_zp.dt == DT_U4 || a.wei_zp.dt == DT_S4);
    const float zt = p.zp_mode == 2 ? (float)load_int(a.wei_zp.dt, a.wei_zp.ptr, 0) : 0.f;
    const char *src_row = (const char *)a.src + ((p.m_base + g) * a.src_sm) * 2;
    const bool row_ok = g < p.M;

    const int64_t total = (int64_t)p.nblk * p.ksteps;
    int64_t L = (int64_t)blockIdx.x * p.per;
    const int64_t L1 = min(total, L + p.per);
    // Byte offset inside a 16-row half stage of this lane's 8 bytes (16 columns) in k-row 2tig; row
    // 2tig+1 lies 64 bytes further, rows +8 another 512.  64B swizzle: the 16-byte chunk index is
    // XORed with (row >> 1) & 3, which is tig for all four rows.
    const int lds0 = (2 * tig) * 64 + ((((g >> 1) ^ tig) & 3) << 4) + (g & 1) * 8;
    uint32_t git = 0; // stages consumed so far by this warp (ring position and phase)
    bool ok = true;
    // Lane 0 requests the first stages of this warp's k sub-range of the segment that starts at
    // position Ls.  Called before the first segment, and for the following one as soon as the k
    // loop of a segment ends, so that the loads run under the reduction and the epilogue.
    auto prefetch_segment = [&](int64_t Ls) {
        if (lane != 0 || Ls >= L1 || !ok) return;
        const int nb = (int)(Ls / p.ksteps), kb = (int)(Ls % p.ksteps);
        const int ke = (int)min((int64_t)p.ksteps, kb + (L1 - Ls));
        const int sg = ke - kb;
        const int w0 = kb + (int)((int64_t)sg * pair / PAIRS), w1 = kb + (int)((int64_t)sg * (pair + 1) / PAIRS);
        const int nst = (w1 - w0 + 1) >> 1;
        for (int i = 0; i < STAGES && i < nst; ++i) {
            const int s = (git + i) % STAGES;
            ptx::mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
            ptx::tma_load_2d(ring + s * STAGE_BYTES, &tmW, &full[s], nb * (NB / 2) + half * 64, (w0 + 2 * i) * 16);
        }
    };
    prefetch_segment(L);

    while (L < L1) {
        const int nblk = (int)(L / p.ksteps), kb = (int)(L % p.ksteps);
        const int ke = (int)min((int64_t)p.ksteps, kb + (L1 - L));
        const int seg = ke - kb;
        const int ws0 = kb + (int)((int64_t)seg * pair / PAIRS), ws1 = kb + (int)((int64_t)seg * (pair + 1) / PAIRS);
        const int nsteps = ok ? ws1 - ws0 : 0; // after an expired wait the warp only takes part in the barriers
        const int nstages = (nsteps + 1) >> 1;
        const int64_t n0 = (int64_t)nblk * NB + half * 128 + g * 16; // this lane's 16 columns
        const bool cols_ok = n0 < a.N;
        const int xbyte = nblk * (NB / 2) + half * 64;

        float acc[8][4];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
            tot_s[32 * t] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float sp = 0.f; // running sum of this lane's src values (row g) in the current group
        uint32_t scw[8]; // bf16 scale pairs (columns 2t, 2t+1) of the current group
#pragma unroll
        for (int t = 0; t < 8; ++t) scw[t] = 0u; // lanes whose columns lie beyond N keep zeros
        uint2 zq = make_uint2(0, 0); // 4-bit zero-points of the current group
        uint32_t nb0 = 0, nb1 = 0; // src operand of the next k-step
        // this lane's src words of k-step ws0 (k = 16 ws0 + 2 tig, +1 and +8, +9); 8 words per k-step
        const uint32_t *sq = reinterpret_cast<const uint32_t *>(src_row + ((int64_t)ws0 * 16 + 2 * tig) * 2);
        if (!(WOQ_ABLATE & 4) && row_ok && nsteps > 0) {
            nb0 = ldg_u32_here(sq);
            nb1 = ldg_u32_here(sq + 4);
        }
        // all loop-carried positions advance by increments: no division in the loop
        int gi = ws0 / p.group_steps, gpos = ws0 - gi * p.group_steps; // group and k-step inside it
        int s = git % STAGES;
        uint32_t phase = (git / STAGES) & 1;
        git += nstages;

        for (int it = 0; it < nsteps; ++it) {
            const int kstep = ws0 + it;
            const int hs = it & 1; // which 16-row half of the stage
            // quantization parameters of a new group: requested now, used when the group ends
            if ((it == 0 || gpos == 0) && cols_ok) {
                if (sc_bf16) {
                    const int64_t qb = ((a.wei_scale.mask & 1) ? (int64_t)gi * a.wei_scale.ld : 0) + n0;
                    const char *q = (const char *)a.wei_scale.ptr + qb * 2;
                    const uint4 v0 = ldg_v4_here(q), v1 = ldg_v4_here(q + 16);
                    scw[0] = v0.x; scw[1] = v0.y; scw[2] = v0.z; scw[3] = v0.w;
                    scw[4] = v1.x; scw[5] = v1.y; scw[6] = v1.z; scw[7] = v1.w;
                }
                if (zp4) zq = ldg_v2_here((const char *)a.wei_zp.ptr + ((int64_t)gi * a.wei_zp.ld + n0) / 2);
            }
            // a new stage: every lane waits (it reads the stage), and the warp leaves the loop as a whole
            if (!hs && !__all_sync(0xffffffffu, ptx::mbar_wait(&full[s], phase))) { ok = false; break; }
            const uint8_t *st = ring + s * STAGE_BYTES + hs * 1024 + lds0;
            const bool lds = !(WOQ_ABLATE & 8);
            const uint2 R0 = lds ? *reinterpret_cast<const uint2 *>(st) : make_uint2(it, lane); // k-row 2tig
            const uint2 R1 = lds ? *reinterpret_cast<const uint2 *>(st + 64) : make_uint2(s, it); // 2tig+1
            const uint2 R2 = lds ? *reinterpret_cast<const uint2 *>(st + 512) : make_uint2(lane, s); // 2tig+8
            const uint2 R3 = lds ? *reinterpret_cast<const uint2 *>(st + 576) : make_uint2(kstep, kstep); // 2tig+9
            // src operand (row g; k = 16*kstep + {2tig, 2tig+1}, {2tig+8, 2tig+9}): loaded one step ahead
            const uint32_t b0 = nb0, b1 = nb1;
            sq += 8;
            if (!(WOQ_ABLATE & 4) && row_ok && it + 1 < nsteps) {
                nb0 = ldg_u32_here(sq);
                nb1 = ldg_u32_here(sq + 4);
            }
            sp += pair_sum<F16>(b0) + pair_sum<F16>(b1);
#pragma unroll
            for (int t = 0; t < ((WOQ_ABLATE & 1) ? 0 : 8); ++t) {
                // byte t of the four rows: low nibble = column 2t, high nibble = column 2t+1
                const uint32_t sel = ((4 + (t & 3)) << 12) | ((4 + (t & 3)) << 8) | ((t & 3) << 4) | (t & 3);
                const uint32_t x01 = prmt(t < 4 ? R0.x : R0.y, t < 4 ? R1.x : R1.y, sel);
                const uint32_t x23 = prmt(t < 4 ? R2.x : R2.y, t < 4 ? R3.x : R3.y, sel);
                uint32_t af[4];
                af[0] = nib2(x01, magic); // column 2t,   k pair (2tig, 2tig+1)
                af[1] = nib2(x01 >> 4, magic); // column 2t+1
                af[2] = nib2(x23, magic); // column 2t,   k pair (2tig+8, 2tig+9)
                af[3] = nib2(x23 >> 4, magic); // column 2t+1
                if (F16) mma_f16(acc[t], af, b0, b1);
                else mma_bf16(acc[t], af, b0, b1);
            }
            // The MMAs have consumed the registers read from the stage, so every lane's reads are
            // complete: after its second half (or the range's last step) the stage is refilled.
            if (hs || it == nsteps - 1) {
                __syncwarp();
                const int next = (it >> 1) + STAGES;
                if (lane == 0 && next < nstages) {
                    ptx::mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                    ptx::tma_load_2d(ring + s * STAGE_BYTES, &tmW, &full[s], xbyte, (ws0 + 2 * next) * 16);
                }
                if (++s == STAGES) { s = 0; phase ^= 1; }
            }
            // end of a quantization group (or of this warp's range): fold the group into the totals
            const bool group_end = ++gpos == p.group_steps;
            if (ZPMMA && (group_end || it == nsteps - 1)) {
                // The correction -(offset + zp) * S leaves through one more MMA per 16 columns: its first
                // k slots pair (128 [+8] + zp), rebuilt from the zero-point nibble like a weight, with -S
                // cut into three bf16 pieces (8 + 8 + 8 significant bits: exact), and slots 8..11 pair the
                // remaining constant offset with the same pieces.
                sp += __shfl_xor_sync(0xffffffffu, sp, 1);
                sp += __shfl_xor_sync(0xffffffffu, sp, 2); // every lane: S of src row g
                const float ns = -sp;
                sp = 0.f;
                const uint32_t ph = __float_as_uint(ns) & 0xffff0000u;
                const float r1 = ns - __uint_as_float(ph);
                const uint32_t pm = __float_as_uint(r1) & 0xffff0000u;
                const uint32_t pl = __float_as_uint(r1 - __uint_as_float(pm));
                const uint32_t cb0 = tig == 0 ? ((ph >> 16) | pm) : (tig == 1 ? (pl >> 16) : 0u);
                const uint32_t cb1 = p.az_diff ? cb0 : 0u;
                // every lane takes part in the MMAs, also those whose columns lie beyond N
#pragma unroll
                for (int t = 0; t < ((WOQ_ABLATE & 2) ? 0 : 8); ++t) {
                    uint32_t za[4];
                    if (p.zp_mode == 1) {
                        // byte t of the lane's 8 zero-point bytes -> [b, 0, b, 0]
                        const uint32_t sel = (4u << 12) | ((t & 3) << 8) | (4u << 4) | (t & 3);
                        const uint32_t x = prmt(t < 4 ? zq.x : zq.y, 0u, sel);
                        za[0] = nib2(x, p.magic_z);
                        za[1] = nib2(x >> 4, p.magic_z);
                    } else {
                        za[0] = za[1] = p.az_const;
                    }
                    za[2] = za[3] = p.az_diff;
                    mma_bf16(acc[t], za, cb0, cb1);
                    float sc_lo, sc_hi;
                    if (sc_bf16) {
                        sc_lo = __uint_as_float(scw[t] << 16);
                        sc_hi = __uint_as_float(scw[t] & 0xffff0000u);
                    } else {
                        const int64_t qbase = ((a.wei_scale.mask & 1) ? (int64_t)gi * a.wei_scale.ld : 0) + n0;
                        sc_lo = cols_ok ? load_float(a.wei_scale.dt, a.wei_scale.ptr, qbase + 2 * t) : 0.f;
                        sc_hi = cols_ok ? load_float(a.wei_scale.dt, a.wei_scale.ptr, qbase + 2 * t + 1) : 0.f;
                    }
                    float4 v = tot_s[32 * t];
                    v.x = fmaf(sc_lo, acc[t][0], v.x);
                    v.y = fmaf(sc_lo, acc[t][1], v.y);
                    v.z = fmaf(sc_hi, acc[t][2], v.z);
                    v.w = fmaf(sc_hi, acc[t][3], v.w);
                    tot_s[32 * t] = v;
                    acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
                }
                if (group_end) { gpos = 0; ++gi; }
            }
            if (!ZPMMA && (group_end || it == nsteps - 1)) {
                sp += __shfl_xor_sync(0xffffffffu, sp, 1);
                sp += __shfl_xor_sync(0xffffffffu, sp, 2);
                const float S0 = __shfl_sync(0xffffffffu, sp, (2 * tig) * 4);
                const float S1 = __shfl_sync(0xffffffffu, sp, (2 * tig + 1) * 4);
                sp = 0.f;
                if (cols_ok) {
                    const int64_t qbase = ((a.wei_scale.mask & 1) ? (int64_t)gi * a.wei_scale.ld : 0) + n0;
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        float sc_lo, sc_hi;
                        if (sc_bf16) {
                            sc_lo = __uint_as_float(scw[t] << 16);
                            sc_hi = __uint_as_float(scw[t] & 0xffff0000u);
                        } else {
                            sc_lo = load_float(a.wei_scale.dt, a.wei_scale.ptr, qbase + 2 * t);
                            sc_hi = load_float(a.wei_scale.dt, a.wei_scale.ptr, qbase + 2 * t + 1);
                        }
                        float z_lo = zt, z_hi = zt;
                        if (zp4) {
                            const uint32_t byte = ((t < 4 ? zq.x : zq.y) >> ((t & 3) * 8)) & 0xffu;
                            int lo = byte & 0xf, hi = byte >> 4;
                            if (a.wei_zp.dt == DT_S4) { lo = (lo ^ 8) - 8; hi = (hi ^ 8) - 8; }
                            z_lo = (float)lo; z_hi = (float)hi;
                        } else if (p.zp_mode == 1) {
                            const int64_t zb = (int64_t)gi * a.wei_zp.ld + n0 + 2 * t;
                            z_lo = (float)load_int(a.wei_zp.dt, a.wei_zp.ptr, zb);
                            z_hi = (float)load_int(a.wei_zp.dt, a.wei_zp.ptr, zb + 1);
                        }
                        const float oz_lo = off + z_lo, oz_hi = off + z_hi;
                        float4 v = tot_s[32 * t];
                        v.x = fmaf(sc_lo, acc[t][0] * acc_scale - oz_lo * S0, v.x);
                        v.y = fmaf(sc_lo, acc[t][1] * acc_scale - oz_lo * S1, v.y);
                        v.z = fmaf(sc_hi, acc[t][2] * acc_scale - oz_hi * S0, v.z);
                        v.w = fmaf(sc_hi, acc[t][3] * acc_scale - oz_hi * S1, v.w);
                        tot_s[32 * t] = v;
                    }
                }
#pragma unroll
                for (int t = 0; t < 8; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
                if (group_end) { gpos = 0; ++gi; }
            }
        }

        __syncwarp(); // every lane has read the ring's last stage
        prefetch_segment(L + seg);
        if (WOQ_ABLATE & 16) { L += seg; continue; }
        // ---- the pairs' totals meet: thread i adds the 8 pairs' float4 of (half, t, lane) = i
        __syncthreads();
        const int i = threadIdx.x;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int pr = 0; pr < PAIRS; ++pr) {
            const float4 w = tot_all[(2 * pr + (i >> 8)) * 256 + (i & 255)];
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        // CTAs sharing this column block, in k order
        const int first = (int)(((int64_t)nblk * p.ksteps) / p.per);
        const int last = (int)((((int64_t)nblk + 1) * p.ksteps - 1) / p.per);
        bool finalize = true;
        if (last > first) {
            const int count = last - first + 1, slot = (int)blockIdx.x - first;
            float4 *base = p.partial + ((int64_t)nblk * p.max_slots) * 512;
            base[slot * 512 + i] = v;
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) *flag = atomicAdd(&p.counters[nblk], 1) == count - 1;
            __syncthreads();
            finalize = *flag != 0;
            if (finalize) {
                __threadfence();
                v = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sl = 0; sl < count; ++sl) {
                    const float4 w = __ldcg(base + sl * 512 + i);
                    v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
                }
                if (threadIdx.x == 0) p.counters[nblk] = 0; // ready for the next launch
            }
        }
        // v: columns c0 (x, y) and c0 + 1 (z, w), src rows 2tig (x, z) and 2tig + 1 (y, w)
        const int64_t c0 = (int64_t)nblk * NB + (i >> 8) * 128 + g * 16 + 2 * ((i >> 5) & 7);
        if (finalize && c0 < a.N) {
            float ss = 1.f;
            if (a.src_scale.ptr) ss = load_float(a.src_scale.dt, a.src_scale.ptr, 0);
            else if (a.src_scale.on_host) ss = a.src_scale.host_value;
            const float vals[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int m = 2 * tig + (e & 1);
                const int64_t n = c0 + (e >> 1);
                if (m < p.M) {
                    const int64_t mm = p.m_base + m;
                    float d = vals[e] * ss;
                    if (a.bias) d = __fadd_rn(d, load_float(a.bias_dt, a.bias, mm * a.bias_sm + n * a.bias_sn));
                    finish_store(a, d, mm, n, false);
                }
            }
        }
        __syncthreads(); // the totals and the flag are reused by the next segment
        L += seg;
    }
    if (!ok) atomicExch(a.status, 5);
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
        const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
        CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_tiled_fn woq_get_encode() {
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

// The cut of the (column block, k-step) space: `per` pairs per CTA (a multiple
// of 16 so the warp pairs get equal shares of whole stages, at least 32 so a
// CTA is worth its launch), `grid` CTAs, at most `max_slots` CTAs on one
// column block.
struct WoqPlan {
    int nblk, ksteps, per, grid, max_slots;
};
WoqPlan woq_plan(int64_t N, int64_t K, int sm_count) {
    WoqPlan pl;
    pl.nblk = (int)((N + NB - 1) / NB);
    pl.ksteps = (int)(K / 16);
    const int64_t total = (int64_t)pl.nblk * pl.ksteps;
    if (sm_count < 1) sm_count = 148;
    int64_t per = (total + sm_count - 1) / sm_count;
    per = (per + 15) / 16 * 16;
    if (per < 32) per = 32;
    pl.per = (int)per;
    pl.grid = (int)((total + per - 1) / per);
    pl.max_slots = (int)((pl.ksteps + per - 1) / per) + 1;
    return pl;
}

} // namespace

size_t woq_skinny_scratch_bytes(int64_t N, int64_t K, int sm_count) {
    const WoqPlan pl = woq_plan(N, K, sm_count);
    return ((size_t)pl.nblk * sizeof(int) + 255) / 256 * 256
            + (size_t)pl.nblk * pl.max_slots * MB * NB * sizeof(float);
}

// `scratch`: woq_skinny_scratch_bytes(N, K, sm_count) bytes whose counters
// (the first ceil(N/256) ints) are zero before the first launch; the kernel
// leaves them zero.
int launch_woq_skinny(const MatmulArgs &a, void *scratch, int sm_count, cudaStream_t st) {
    if (a.M == 0 || a.N == 0) return 0;
    encode_tiled_fn enc = woq_get_encode();
    if (!enc || !scratch) return 5;
    const WoqPlan pl = woq_plan(a.N, a.K, sm_count);
    CUtensorMap tm;
    cuuint64_t dims[2] = {(cuuint64_t)(a.N / 2), (cuuint64_t)a.K};
    cuuint64_t strides[1] = {(cuuint64_t)(a.wei_sk / 2)};
    cuuint32_t box[2] = {64, 32};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(a.wei), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            != CUDA_SUCCESS)
        return 5;
    WoqParams p {};
    p.ksteps = pl.ksteps;
    const int64_t group = (a.wei_scale.ptr && (a.wei_scale.mask & 1)) ? a.wei_scale.g0
            : (a.wei_zp.ptr && (a.wei_zp.mask & 1))                    ? a.wei_zp.g0
                                                                       : a.K;
    p.group_steps = (int)(group / 16);
    p.nblk = pl.nblk;
    p.per = pl.per;
    p.max_slots = pl.max_slots;
    p.sgn4 = a.wei_dt == DT_S4;
    p.zp_mode = !a.wei_zp.ptr ? 0 : (a.wei_zp.mask ? 1 : 2);
    p.counters = (int *)scratch;
    p.partial = (float4 *)((char *)scratch + ((size_t)pl.nblk * sizeof(int) + 255) / 256 * 256);
    const bool f16 = a.src_dt == DT_F16;
    // tensor-core zero-point correction: bf16 src and either no zero-points or 4-bit ones per group
    const bool zp4 = p.zp_mode == 1 && (a.wei_zp.dt == DT_U4 || a.wei_zp.dt == DT_S4);
    const bool zpmma = !f16 && (p.zp_mode == 0 || zp4);
    if (zpmma) {
        const int off_w = p.sgn4 ? 136 : 128; // a weight nibble becomes off_w + w
        const int off_z = (zp4 && a.wei_zp.dt == DT_S4) ? 136 : 128; // a zero-point nibble becomes off_z + zp
        auto bf16_pair = [](int v) { // small integers are exact in bf16
            const float f = (float)v;
            uint32_t u;
            memcpy(&u, &f, 4);
            return (u >> 16) | (u & 0xffff0000u);
        };
        p.magic_z = off_z == 136 ? 0x43084308u : 0x43004300u;
        p.az_const = bf16_pair(off_w);
        p.az_diff = zp4 ? (off_w == off_z ? 0u : bf16_pair(off_w - off_z)) : 0u;
    }
    const int variant = f16 ? 2 : (zpmma ? 1 : 0);
    auto kern = f16 ? woq_skinny_kernel<true, false>
                    : (zpmma ? woq_skinny_kernel<false, true> : woq_skinny_kernel<false, false>);
    static std::atomic<unsigned long long> configured[3];
    if (!opt_in_dynamic_smem(kern, SMEM_BYTES, configured[variant])) return 5;
    for (int64_t m0 = 0; m0 < a.M; m0 += MB) { // more than 8 rows: one pass over the weights per 8 rows
        p.m_base = m0;
        p.M = (int)((a.M - m0) < MB ? (a.M - m0) : MB);
        kern<<<pl.grid, WARPS * 32, SMEM_BYTES, st>>>(tm, a, p);
        count_launch();
    }
    return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

} // namespace qmm
