// "cuda:ref" kernels: one thread per dst element, every attribute supported,
// the K loop in the same order as oneDNN's scalar reference so the f32 result
// is reproduced operation for operation.  They are the catch-all entry of the
// implementation list (what ref:any / ref_int8:any / ref_grouped:any are on
// the CPU); the shapes that matter are served by the specialised kernels.
//
//   int8 src   : src/cpu/matmul/ref_matmul_int8.cpp:173-306
//   fp src     : src/cpu/matmul/ref_matmul.cpp:169-332
//   grouped    : src/cpu/matmul/ref_grouped_gemm.cpp:218-444
#include "device_math.cuh"
#include "launch.h"

namespace qmm {

namespace {

__device__ __forceinline__ int64_t ngroups_if_grouped(const QParam &q, int64_t K, int kdim) {
    const int64_t g = kdim == 0 ? q.g0 : q.g1;
    return (q.ptr && g > 1) ? K / g : 1;
}
__device__ __forceinline__ int64_t max3(int64_t a, int64_t b, int64_t c) {
    return max(a, max(b, c));
}

__global__ void __launch_bounds__(256) ref_int8_kernel(const __grid_constant__ MatmulArgs a) {
    const int64_t nb = (a.N + 255) / 256;
    const int64_t n = (int64_t)(blockIdx.x % nb) * 256 + threadIdx.x;
    const int64_t m = blockIdx.x / nb;
    if (n >= a.N) return;
    const int64_t K = a.K;
    const bool with_pr = a.src_pr.ptr != nullptr;
    int64_t ng = max3(ngroups_if_grouped(a.src_zp, K, 1), ngroups_if_grouped(a.wei_zp, K, 0),
            ngroups_if_grouped(a.src_pr, K, 1));
    ng = max3(ng, ngroups_if_grouped(a.src_scale, K, 1), ngroups_if_grouped(a.wei_scale, K, 0));
    const int64_t gk = K / ng;
    float d = 0.f;
    for (int64_t g = 0; g < ng; ++g) {
        int acc = 0;
        const int64_t k0 = g * gk;
        for (int64_t k = k0; k < k0 + gk; ++k) {
            int s = load_int(a.src_dt, a.src, m * a.src_sm + k * a.src_sk);
            int w = load_int(a.wei_dt, a.wei, k * a.wei_sk + n * a.wei_sn);
            if (a.src_zp.ptr) s -= load_int(a.src_zp.dt, a.src_zp.ptr, qoff(a.src_zp, m, k));
            if (a.wei_zp.ptr && !with_pr)
                w -= load_int(a.wei_zp.dt, a.wei_zp.ptr, qoff(a.wei_zp, k, n));
            acc += s * w;
        }
        if (with_pr) {
            const int pr = load_int(a.src_pr.dt, a.src_pr.ptr, qoff(a.src_pr, m, k0));
            const int wz = load_int(a.wei_zp.dt, a.wei_zp.ptr, qoff(a.wei_zp, k0, n));
            acc -= pr * wz;
            if (a.src_zp.ptr) {
                const int sz = load_int(a.src_zp.dt, a.src_zp.ptr, qoff(a.src_zp, m, k0));
                acc += (int)(gk * wz * sz);
            }
        }
        float f = (float)acc;
        if (a.src_scale.ptr)
            f = __fmul_rn(f, load_float(a.src_scale.dt, a.src_scale.ptr, qoff(a.src_scale, m, k0)));
        else if (a.src_scale.on_host)
            f = __fmul_rn(f, a.src_scale.host_value);
        if (a.wei_scale.ptr)
            f = __fmul_rn(f, load_float(a.wei_scale.dt, a.wei_scale.ptr, qoff(a.wei_scale, k0, n)));
        else if (a.wei_scale.on_host)
            f = __fmul_rn(f, a.wei_scale.host_value);
        d = __fadd_rn(d, f);
    }
    if (a.bias) d = __fadd_rn(d, load_float(a.bias_dt, a.bias, m * a.bias_sm + n * a.bias_sn));
    finish_store(a, d, m, n, true);
}

__global__ void __launch_bounds__(256) ref_fp_kernel(const __grid_constant__ MatmulArgs a) {
    const int64_t nb = (a.N + 255) / 256;
    const int64_t n = (int64_t)(blockIdx.x % nb) * 256 + threadIdx.x;
    const int64_t m = blockIdx.x / nb;
    if (n >= a.N) return;
    const int64_t K = a.K;
    const int wdt = a.wei_dt;
    const bool decomp = a.apply_to_int && (wdt == DT_S8 || wdt == DT_U8 || wdt == DT_S4 || wdt == DT_U4);
    // Unless BOTH scales are grouped along K the reference treats every k as
    // a group of its own: each product is scaled, then added.
    const int64_t gs = ((a.src_scale.ptr || a.src_scale.on_host) && a.src_scale.g1 > 1) ? a.src_scale.g1 : 1;
    const int64_t gw = ((a.wei_scale.ptr || a.wei_scale.on_host) && a.wei_scale.g0 > 1) ? a.wei_scale.g0 : 1;
    const int64_t ng = max(K / gs, K / gw);
    const int64_t gk = K / ng;
    float res = 0.f;
    for (int64_t g = 0; g < ng; ++g) {
        float acc = 0.f;
        const int64_t k0 = g * gk;
        for (int64_t k = k0; k < k0 + gk; ++k) {
            const float s = load_float(a.src_dt, a.src, m * a.src_sm + k * a.src_sk);
            float w = load_float(wdt, a.wei, k * a.wei_sk + n * a.wei_sn);
            if (decomp) {
                if (a.wei_zp.ptr)
                    w = __fsub_rn(w, load_float(a.wei_zp.dt, a.wei_zp.ptr, qoff(a.wei_zp, k, n)));
                if (a.wei_scale.ptr)
                    w = __fmul_rn(w, load_float(a.wei_scale.dt, a.wei_scale.ptr, qoff(a.wei_scale, k, n)));
                else if (a.wei_scale.on_host)
                    w = __fmul_rn(w, a.wei_scale.host_value);
            }
            acc = __fadd_rn(acc, __fmul_rn(s, w));
        }
        if (a.src_scale.ptr)
            acc = __fmul_rn(acc, load_float(a.src_scale.dt, a.src_scale.ptr, qoff(a.src_scale, m, k0)));
        else if (a.src_scale.on_host)
            acc = __fmul_rn(acc, a.src_scale.host_value);
        if (!decomp) {
            if (a.wei_scale.ptr)
                acc = __fmul_rn(acc, load_float(a.wei_scale.dt, a.wei_scale.ptr, qoff(a.wei_scale, k0, n)));
            else if (a.wei_scale.on_host)
                acc = __fmul_rn(acc, a.wei_scale.host_value);
        }
        res = __fadd_rn(res, acc);
    }
    if (a.bias) res = __fadd_rn(res, load_float(a.bias_dt, a.bias, m * a.bias_sm + n * a.bias_sn));
    finish_store(a, res, m, n, false);
}

// Checks the runtime offsets of a grouped problem: monotone, within [0, M].
// A violation is recorded in *status (the reference returns
// invalid_arguments, ref_grouped_gemm.cpp:164-213) and the compute kernel
// then leaves dst untouched.
__global__ void grouped_check_offsets(const __grid_constant__ MatmulArgs a) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= a.group_count) return;
    const int64_t b = g == 0 ? 0 : a.offsets[g - 1], e = a.offsets[g];
    const int64_t db = g == 0 ? 0 : a.dst_offsets[g - 1], de = a.dst_offsets[g];
    if (b < 0 || e > a.M || e < b || db < 0 || de > a.M || de < db) atomicExch(a.status, 2);
}

__global__ void __launch_bounds__(256) ref_grouped_kernel(const __grid_constant__ MatmulArgs a) {
    if (*(volatile int *)a.status != 0) return;
    const int64_t nb = (a.N + 255) / 256;
    const int64_t n = (int64_t)(blockIdx.x % nb) * 256 + threadIdx.x;
    const int64_t m = blockIdx.x / nb;
    if (n >= a.N) return;
    // expert owning row m: first group whose END offset exceeds m
    int lo = 0, hi = a.group_count;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (a.offsets[mid] > m) hi = mid; else lo = mid + 1;
    }
    const int gid = lo;
    if (gid >= a.group_count) return; // row beyond the last group: not written
    const int64_t K = a.K, N = a.N;
    const int sdt = a.src_dt, wdt = a.wei_dt;
    const bool wint = wdt == DT_S8 || wdt == DT_U8 || wdt == DT_S4 || wdt == DT_U4;
    const bool use_int = (sdt == DT_S8 || sdt == DT_U8) && wint;
    const bool use_woq = (sdt == DT_F32 || sdt == DT_BF16 || sdt == DT_F16) && wint && a.apply_to_int;
    const int64_t ss_ng = ngroups_if_grouped(a.src_scale, K, 1), ws_ng = ngroups_if_grouped(a.wei_scale, K, 0);
    const int64_t sz_ng = ngroups_if_grouped(a.src_zp, K, 1), wz_ng = ngroups_if_grouped(a.wei_zp, K, 0);
    const int64_t ng = max(max(ss_ng, ws_ng), max(sz_ng, wz_ng));
    const int64_t gk = K / ng;
    const int64_t wbase = (int64_t)gid * a.wei_sg;
    // dst row: same position inside the group, at the dst offsets
    const int64_t row0 = gid == 0 ? 0 : a.offsets[gid - 1];
    const int64_t drow = (gid == 0 ? 0 : a.dst_offsets[gid - 1]) + (m - row0);
    float result = 0.f;
    for (int64_t ig = 0; ig < ng; ++ig) {
        int szp = 0, wzp = 0;
        float wsc = 1.f;
        if (use_int || use_woq) {
            if (a.src_zp.ptr) szp = load_int(a.src_zp.dt, a.src_zp.ptr, m * sz_ng + ig * sz_ng / ng);
            if (a.wei_scale.ptr)
                wsc = load_float(a.wei_scale.dt, a.wei_scale.ptr, gid * ws_ng * N + (ig * ws_ng / ng) * N + n);
            if (a.wei_zp.ptr)
                wzp = load_int(a.wei_zp.dt, a.wei_zp.ptr, gid * wz_ng * N + (ig * wz_ng / ng) * N + n);
        }
        float acc = 0.f;
        const int64_t k0 = ig * gk;
        if (use_int) {
            int ai = 0;
            for (int64_t k = k0; k < k0 + gk; ++k) {
                const int s = load_int(sdt, a.src, m * a.src_sm + k * a.src_sk);
                const int w = load_int(wdt, a.wei, wbase + k * a.wei_sk + n * a.wei_sn);
                ai += (s - szp) * (w - wzp);
            }
            acc = (float)ai;
        } else if (use_woq) {
            for (int64_t k = k0; k < k0 + gk; ++k) {
                const float s = load_float(sdt, a.src, m * a.src_sm + k * a.src_sk);
                const int w = load_int(wdt, a.wei, wbase + k * a.wei_sk + n * a.wei_sn);
                acc = __fadd_rn(acc, __fmul_rn(s, (float)(w - wzp)));
            }
        } else {
            for (int64_t k = k0; k < k0 + gk; ++k) {
                const float s = load_float(sdt, a.src, m * a.src_sm + k * a.src_sk);
                const float w = load_float(wdt, a.wei, wbase + k * a.wei_sk + n * a.wei_sn);
                acc = __fadd_rn(acc, __fmul_rn(s, w));
            }
        }
        if (a.src_scale.ptr)
            acc = __fmul_rn(acc, load_float(a.src_scale.dt, a.src_scale.ptr, m * ss_ng + ig * ss_ng / ng));
        if (use_int || use_woq) {
            result = __fadd_rn(result, __fmul_rn(acc, wsc));
        } else {
            if (a.wei_scale.ptr)
                acc = __fmul_rn(acc,
                        load_float(a.wei_scale.dt, a.wei_scale.ptr, gid * ws_ng * N + (ig * ws_ng / ng) * N + n));
            result = __fadd_rn(result, acc);
        }
    }
    if (a.bias) result = __fadd_rn(result, load_float(a.bias_dt, a.bias, gid * a.bias_sg + n));
    result = apply_post_ops(a, result, 0.f, drow, n, gid);
    store_float(a.dst_dt, result, a.dst, drow * a.dst_sm + n * a.dst_sn);
}

} // namespace

int launch_ref(const MatmulArgs &a, cudaStream_t st) {
    if (a.M == 0 || a.N == 0) return 0;
    const int64_t nblocks = a.M * ((a.N + 255) / 256);
    if (nblocks > 0x7fffffffLL) return 3;
    dim3 block(256), grid((unsigned)nblocks);
    if (a.group_count > 0) {
        grouped_check_offsets<<<(a.group_count + 127) / 128, 128, 0, st>>>(a);
        count_launch();
        ref_grouped_kernel<<<grid, block, 0, st>>>(a);
    } else if (a.src_dt == DT_S8 || a.src_dt == DT_U8) {
        ref_int8_kernel<<<grid, block, 0, st>>>(a);
    } else {
        ref_fp_kernel<<<grid, block, 0, st>>>(a);
    }
    count_launch();
    return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

} // namespace qmm
