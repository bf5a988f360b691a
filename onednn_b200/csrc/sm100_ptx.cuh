// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the GEMM
// kernels use: mbarriers, TMA tiled loads, tensor memory (TMEM) management and
// tcgen05 MMA / load instructions, plus the shared-memory and instruction
// descriptor encodings.  Every wait is bounded: it gives up after a wall-clock
// limit and reports failure instead of spinning forever.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace qmm {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint64_t globaltimer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// True in exactly one lane of a converged warp.  tcgen05.mma issued under this predicate (a branch or
// a guard) takes about 70 cycles per instruction; under a predicate computed from the lane index, which
// the hardware cannot know to be one lane, about 115.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
            "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One poll.  QMM_TRY_WAIT_HINT_NS (a build switch) gives the instruction a suspend-time hint: the
// thread may then sleep in hardware until the phase completes or the time has passed, instead of
// coming back at once and executing the polling loop's instructions.
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
#ifdef QMM_TRY_WAIT_HINT_NS
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)QMM_TRY_WAIT_HINT_NS)
            : "memory");
#else
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
#endif
    return ok != 0;
}
// Waits for the phase with the given parity to complete.  Returns false when
// the wait did not finish within `limit_ns` (default 2 s): the caller then
// records an error status and leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint64_t limit_ns = 2000000000ull) {
    // the common case first, without touching the timer: a wait that is served within a few
    // thousand polls (every wait of a healthy pipeline) never reads %globaltimer
    for (int i = 0; i < 4096; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer();
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer() - t0 > limit_ns) return false;
    }
}
// A 32-bit word in shared memory handed from one warp to another
__device__ __forceinline__ uint32_t ld_acquire_shared(const volatile uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(const_cast<uint32_t *>(p))) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_shared(volatile uint32_t *p, uint32_t v) {
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t *>(p))), "r"(v) : "memory");
}

// A commit under a lane predicate, for the rarely taken paths of warp-uniform issuing code (whole
// warps walk the loops, so that loop counters, addresses and descriptors stay warp-uniform values).
// The hot paths put a stage's tcgen05 / TMA instructions in a branch taken by the thread elect_one()
// picks instead: an instruction guarded by a predicate computed from the lane index costs nearly twice
// as much to issue.
__device__ __forceinline__ void tc_commit_if(bool issue, uint64_t *bar) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
                 "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)), "r"((uint32_t)issue)
                 : "memory");
}

// The same for a whole warp that may wait long: between polls the warp sleeps a few dozen
// nanoseconds, so that a dozen waiting warps do not fill the SM's shared-memory instruction queue
// with polls that the working warps' loads, arrives and tensor-memory stores then queue behind.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t *bar, uint32_t parity, uint64_t limit_ns = 2000000000ull) {
    if (mbar_try_wait(bar, parity)) return true;
    for (int i = 0; i < 8192; ++i) {
        __nanosleep(32);
        if (mbar_try_wait(bar, parity)) return true;
    }
    const uint64_t t0 = globaltimer();
    for (;;) {
        for (int i = 0; i < 256; ++i) {
            __nanosleep(64);
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (globaltimer() - t0 > limit_ns) return false;
    }
}

// ---- TMA ------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2D tiled load global -> shared, completion signalled on `bar` (bytes)
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int y) {
    asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
            : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int y, int z) {
    asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
            : "memory");
}

// ---- tensor memory --------------------------------------------------------
// One full warp allocates `ncols` (power of two >= 32) TMEM columns; the base
// address is written to *dst_smem.
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// arrives on `bar` once every MMA issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives
// lane (lane base of the warp + t), columns [col, col + 32)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr)
            : "memory");
}
// the same for 8 columns
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
            : "r"(taddr)
            : "memory");
}
__device__ __forceinline__ void tmem_ld_32x4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_32xn(uint32_t taddr, uint32_t (&r)[4]) { tmem_ld_32x4(taddr, r); }
__device__ __forceinline__ void tmem_ld_32xn(uint32_t taddr, uint32_t (&r)[8]) { tmem_ld_32x8(taddr, r); }
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- descriptors ----------------------------------------------------------
// Shared-memory matrix descriptor for a tile stored with the 128-byte swizzle
// (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B writes).  Offsets in bytes.
//   K-major operand : rows of 128 B along K; sbo = pitch of an 8-row group
//   MN-major operand: rows of 128 B along M/N, one row per k; sbo = pitch of
//                     an 8-k group, lbo = pitch between 128-B-wide column blocks
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46; // descriptor version of this architecture
    d |= (uint64_t)2 << 61; // SWIZZLE_128B
    return d;
}

enum : uint32_t { FMT_E4M3 = 0, FMT_E5M2 = 1, FMT_U8 = 0, FMT_S8 = 1, FMT_F16 = 0, FMT_BF16 = 1 };
enum : uint32_t { CFMT_F16 = 0, CFMT_F32 = 1, CFMT_S32 = 2 };

// Instruction descriptor of tcgen05.mma (dense, no negation, no saturation)
__host__ __device__ constexpr uint32_t make_idesc(uint32_t cfmt, uint32_t afmt, uint32_t bfmt, bool a_mn_major,
        bool b_mn_major, uint32_t M, uint32_t N) {
    return (cfmt << 4) | (afmt << 7) | (bfmt << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16)
            | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.  KIND: 0 f8f6f4, 1 i8, 2 f16
template <int KIND>
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    if constexpr (KIND == 0) {
        asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
                : "memory");
    } else if constexpr (KIND == 1) {
        asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
                : "memory");
    } else {
        asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
                : "memory");
    }
}

} // namespace ptx
} // namespace qmm
