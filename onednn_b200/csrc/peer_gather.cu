// Assembling a sharded dst over NVLink without a collective library: every
// rank stores its block of the result straight into every rank's full dst
// buffer (plain 16-byte peer stores through peer-mapped pointers), then raises
// a flag on every rank; a second, tiny kernel waits (bounded) until the flags
// of all ranks have arrived.  oneDNN is a single-device library and has no
// counterpart; this is the exchange step of the N- / expert-sharded matmul.
//
// The kernels of one rank never wait for each other: the scatter kernel only
// writes, the wait kernel only polls flags that OTHER GPUs write, so each
// GPU's stream makes progress on its own.  No TMA, no multicast: ordinary
// loads from local memory and ordinary stores to peer memory.
#include <cuda_runtime.h>

#include <string>

#include "launch.h"
#include "objects.hpp"
#include "sm100_ptx.cuh"

namespace qmm {

namespace {

constexpr int MAX_SEGMENTS = 64;

struct ScatterArgs {
    int world, rank, nseg;
    const char *local; // this rank's block, rows of row_bytes bytes, pitch src_pitch
    int64_t row_bytes, src_pitch, dst_pitch, dst_col_bytes;
    char *peer_dst[MAX_PEERS]; // every rank's full dst buffer, as mapped on this GPU
    unsigned *peer_flags[MAX_PEERS]; // every rank's flag array [world], as mapped on this GPU
    unsigned epoch;
    unsigned *done; // local counter of finished CTAs (zero before and after a launch)
    // rows [src_row, src_row + rows) of the local block go to rows [dst_row, ...) of the full dst
    int64_t src_row[MAX_SEGMENTS], dst_row[MAX_SEGMENTS], rows[MAX_SEGMENTS];
};

// One CTA walks 16-byte units of the block with a grid stride; a unit is loaded once and stored to
// every rank.  The last CTA to finish publishes the epoch on every rank (after a system-wide fence,
// so that a rank that sees the flag also sees the data).
__global__ void __launch_bounds__(256) peer_scatter_kernel(const __grid_constant__ ScatterArgs a) {
    const int64_t units_per_row = a.row_bytes / 16;
    for (int s = 0; s < a.nseg; ++s) {
        const int64_t total = a.rows[s] * units_per_row;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = i / units_per_row, u = i - r * units_per_row;
            const uint4 v = *reinterpret_cast<const uint4 *>(a.local + (a.src_row[s] + r) * a.src_pitch + u * 16);
            const int64_t off = (a.dst_row[s] + r) * a.dst_pitch + a.dst_col_bytes + u * 16;
#pragma unroll 4
            for (int p = 0; p < a.world; ++p) *reinterpret_cast<uint4 *>(a.peer_dst[p] + off) = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int last;
    if (threadIdx.x == 0) last = atomicAdd(a.done, 1u) == gridDim.x - 1;
    __syncthreads();
    if (last) {
        __threadfence_system();
        if (threadIdx.x < a.world) {
            volatile unsigned *f = a.peer_flags[threadIdx.x] + a.rank;
            *f = a.epoch;
        }
        if (threadIdx.x == 0) *a.done = 0u;
    }
}

// Lane q waits until rank q's flag has reached the epoch; gives up after `limit_ns` and records
// status 5 (the host reads it at its next synchronisation point).
__global__ void peer_wait_kernel(int world, const unsigned *flags, unsigned epoch, int *status, unsigned long long limit_ns) {
    const int q = threadIdx.x;
    if (q >= world) return;
    const volatile unsigned *f = flags + q;
    const unsigned long long t0 = ptx::globaltimer();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if ((int)(*f - epoch) >= 0) { __threadfence_system(); return; }
        if (ptx::globaltimer() - t0 > limit_ns) {
            if (status) atomicExch(status, 5);
            return;
        }
    }
}

} // namespace

} // namespace qmm

using namespace qmm;

// Stores rows of this rank's block into every rank's dst and publishes `epoch` in flags[rank] of
// every rank.  peer_dst / peer_flags: `world` device addresses each, valid on the current device
// (e.g. CUDA IPC or symmetric-memory mappings).  seg: nseg triples (src_row, dst_row, rows).
// row_bytes, the pitches and dst_col_bytes are multiples of 16 and the buffers 16-byte aligned.
// `done`: one zeroed 32-bit word of local device memory, private to these calls.
extern "C" dnnl_status_t dnnl_cuda_interop_peer_scatter(dnnl_stream_t stream, int world, int rank, const void *local,
        int64_t row_bytes, int64_t src_pitch, void *const *peer_dst, int64_t dst_pitch, int64_t dst_col_bytes, int nseg,
        const int64_t *seg, unsigned *const *peer_flags, unsigned epoch, unsigned *done) {
    if (!stream || stream->engine->device < 0) return dnnl_invalid_arguments;
    void *cuda_stream = stream->stream;
    int sm_count = stream->engine->sm_count;
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world || !local || !peer_dst || !peer_flags || !seg || !done
            || nseg < 1 || nseg > MAX_SEGMENTS)
        return dnnl_invalid_arguments;
    if (row_bytes % 16 || src_pitch % 16 || dst_pitch % 16 || dst_col_bytes % 16 || (uintptr_t)local % 16)
        return dnnl_invalid_arguments;
    ScatterArgs a {};
    a.world = world; a.rank = rank; a.nseg = nseg;
    a.local = (const char *)local;
    a.row_bytes = row_bytes; a.src_pitch = src_pitch; a.dst_pitch = dst_pitch; a.dst_col_bytes = dst_col_bytes;
    a.epoch = epoch; a.done = done;
    int64_t units = 0;
    for (int p = 0; p < world; ++p) {
        if (!peer_dst[p] || !peer_flags[p] || (uintptr_t)peer_dst[p] % 16) return dnnl_invalid_arguments;
        a.peer_dst[p] = (char *)peer_dst[p];
        a.peer_flags[p] = peer_flags[p];
    }
    for (int s = 0; s < nseg; ++s) {
        a.src_row[s] = seg[3 * s]; a.dst_row[s] = seg[3 * s + 1]; a.rows[s] = seg[3 * s + 2];
        if (a.rows[s] < 0 || a.src_row[s] < 0 || a.dst_row[s] < 0) return dnnl_invalid_arguments;
        units += a.rows[s] * (row_bytes / 16);
    }
    if (sm_count < 1) sm_count = 148;
    int64_t grid = (units + 255) / 256;
    if (grid > (int64_t)sm_count * 4) grid = (int64_t)sm_count * 4;
    if (grid < 1) grid = 1;
    peer_scatter_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)cuda_stream>>>(a);
    count_launch();
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error(std::string("peer scatter launch: ") + cudaGetErrorString(e));
        return dnnl_runtime_error;
    }
    return dnnl_success;
}

// Enqueues the wait for `epoch` from all `world` ranks on this rank's own flag array.  If a flag
// does not arrive within two seconds the kernel returns and records status 5 on the engine, which
// the next dnnl_stream_wait reports as runtime_error.
extern "C" dnnl_status_t dnnl_cuda_interop_peer_wait(dnnl_stream_t stream, int world, const unsigned *flags, unsigned epoch) {
    if (!stream || stream->engine->device < 0) return dnnl_invalid_arguments;
    if (world < 1 || world > MAX_PEERS || !flags) return dnnl_invalid_arguments;
    void *cuda_stream = stream->stream;
    int *status = stream->engine->status_word;
    peer_wait_kernel<<<1, 32, 0, (cudaStream_t)cuda_stream>>>(world, flags, epoch, status, 2000000000ull);
    count_launch();
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error(std::string("peer wait launch: ") + cudaGetErrorString(e));
        return dnnl_runtime_error;
    }
    return dnnl_success;
}

// Fused form of the scatter for the tcgen05 GEMM: the following executions of `primitive` store
// every dst element into all `world` buffers (the primitive's dst memory must lie inside
// dst_bases[rank]; the same byte offset is used in the others) and publish `epoch` in
// peer_flags[r][rank] of every rank r when the kernel's last CTA has finished, so that
// dnnl_cuda_interop_peer_wait(stream, world, flags, epoch) on each rank is the whole exchange.
// buffer_bytes: size of each buffer.  `done`: one zeroed 32-bit word of local device memory.
// world <= 1 or dst_bases == NULL switches the replication off.  Returns dnnl_unimplemented for
// primitives whose implementation has no fused form (use dnnl_cuda_interop_peer_scatter then).
extern "C" dnnl_status_t dnnl_cuda_interop_primitive_replicate_dst(dnnl_primitive_t primitive, int world, int rank,
        void *const *dst_bases, size_t buffer_bytes, unsigned *const *peer_flags, unsigned *done, unsigned epoch) {
    if (!primitive) return dnnl_invalid_arguments;
    if (world <= 1 || !dst_bases) {
        primitive->peers = PeerReplication {};
        primitive->peers_own_base = nullptr;
        primitive->peers_bytes = 0;
        return dnnl_success;
    }
    if (world > MAX_PEERS || rank < 0 || rank >= world || !peer_flags || !done || !buffer_bytes) return dnnl_invalid_arguments;
    if (primitive->pd.kind != dnnl_matmul || primitive->pd.impl != IMPL_TCGEN05_GEMM) return dnnl_unimplemented;
    // the kernels that carry a post-op chain (or a bias that varies along M) have no replicated form
    if (!primitive->pd.attr.post_ops.entries.empty() || (primitive->pd.bias.ndims > 0 && primitive->pd.bias.dims[0] != 1))
        return dnnl_unimplemented;
    PeerReplication r {};
    r.world = world;
    r.rank = rank;
    r.epoch = epoch;
    r.done = done;
    for (int p = 0; p < world; ++p) {
        if (!dst_bases[p] || !peer_flags[p]) return dnnl_invalid_arguments;
        r.flags[p] = peer_flags[p];
        if (p != rank) r.delta[r.count++] = (const char *)dst_bases[p] - (const char *)dst_bases[rank];
    }
    primitive->peers = r;
    primitive->peers_own_base = (const char *)dst_bases[rank];
    primitive->peers_bytes = buffer_bytes;
    return dnnl_success;
}
