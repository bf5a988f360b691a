// Host-side entry points of the kernels, one per implementation.  Each
// returns a dnnl_status_t value (0 = success, 3 = this kernel does not cover
// the problem, 5 = CUDA runtime error) and only enqueues work on the stream.
#pragma once
#include <cuda_runtime.h>

#include <atomic>

#include "kernel_args.h"

namespace qmm {

// bumps the per-process kernel launch counter (dnnl_cuda_interop_launch_count)
void count_launch(int n = 1);

// Opt-in to more than 48 KB of dynamic shared memory for `kern`.  The attribute
// belongs to the (kernel, device) pair, so `done` - one word per kernel, a bit
// per device ordinal - remembers the devices on which it has been set; the
// current device is the one the launch that follows goes to.  Two host threads
// that race here both set the attribute, which is harmless.
template <typename Kernel>
inline bool opt_in_dynamic_smem(Kernel kern, int bytes, std::atomic<unsigned long long> &done) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    if (dev < 0 || dev >= 64) // beyond the bitmap: set it every time
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
    const unsigned long long bit = 1ull << dev;
    if (done.load(std::memory_order_acquire) & bit) return true;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    done.fetch_or(bit, std::memory_order_release);
    return true;
}

// generic one-thread-per-element kernels, every attribute (ref_kernel.cu)
int launch_ref(const MatmulArgs &a, cudaStream_t st);

// tcgen05 int8 / fp8 GEMM (gemm_tc.cu).  `scratch` holds the zero-point
// compensation terms: gemm_tc_scratch_bytes(M, N) bytes, may be null when the
// problem has no zero-points.
int launch_gemm_tc(const MatmulArgs &a, void *scratch, int sm_count, cudaStream_t st);
size_t gemm_tc_scratch_bytes(int64_t M, int64_t N);
bool gemm_tc_pointers_ok(const MatmulArgs &a);

// int4 weight-decompression skinny GEMM (woq_skinny.cu).  `scratch`:
// woq_skinny_scratch_bytes(...) bytes, zero-initialised once (split-K partial
// sums and per-column-block arrival counters).
int launch_woq_skinny(const MatmulArgs &a, void *scratch, int sm_count, cudaStream_t st);
size_t woq_skinny_scratch_bytes(int64_t N, int64_t K, int sm_count);

// int4 weight-decompression GEMM for M <= 32 on tcgen05 with the rebuilt
// weights as a tensor-memory operand (woq_tc.cu).  `scratch`:
// woq_tc_scratch_bytes(...) bytes, zero-initialised once (arrival counters
// and split-K partial sums).
int launch_woq_tc(const MatmulArgs &a, void *scratch, int sm_count, cudaStream_t st);
size_t woq_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int sm_count);
bool woq_tc_pointers_ok(const MatmulArgs &a);
bool woq_tc_fits(int64_t M, int64_t K, int64_t group, int scale_dt, int zp_dt);

// tcgen05 grouped (MoE) GEMM, bf16 src x s8 weights (grouped_tc.cu).
// `scratch`: grouped_tc_scratch_bytes(group_count, M) bytes, no initialisation
// (tile ranges per group, and the src row sums that weight zero-points need).
int launch_grouped_tc(const MatmulArgs &a, void *scratch, int sm_count, cudaStream_t st);
size_t grouped_tc_scratch_bytes(int groups, int64_t M);
bool grouped_tc_pointers_ok(const MatmulArgs &a);

} // namespace qmm
