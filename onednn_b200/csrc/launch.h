// Host-side entry points of the kernels, one per implementation.  Each
// returns a dnnl_status_t value (0 = success, 3 = this kernel does not cover
// the problem, 5 = CUDA runtime error) and only enqueues work on the stream.
#pragma once
#include <cuda_runtime.h>

#include "kernel_args.h"

namespace qmm {

// bumps the per-process kernel launch counter (dnnl_cuda_interop_launch_count)
void count_launch(int n = 1);

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

// tcgen05 grouped (MoE) GEMM, bf16 src x s8 weights (grouped_tc.cu).
// `scratch`: grouped_tc_scratch_bytes(group_count, M) bytes, no initialisation
// (tile ranges per group, and the src row sums that weight zero-points need).
int launch_grouped_tc(const MatmulArgs &a, void *scratch, int sm_count, cudaStream_t st);
size_t grouped_tc_scratch_bytes(int groups, int64_t M);
bool grouped_tc_pointers_ok(const MatmulArgs &a);

} // namespace qmm
