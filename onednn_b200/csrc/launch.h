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

} // namespace qmm
