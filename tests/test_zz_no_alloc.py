"""The allocation-free entry point against the regular primitive.

`dnnl_cuda_interop_matmul_u8s8s32_zp_static` serves callers that may not
allocate device memory at call time (a host that fixed its memory plan at
start-up, a plugin running while another component records a CUDA graph, a
real-time loop): its scratch - the weight column sums used for the src
zero-point compensation - is a fixed array inside the library instead of a
buffer obtained from cudaMalloc.  The array is shared by all calls and keeps
the previous call's contents, so the test calls it twice in a row, with
different operands, and wants the same bits as the `dnnl_matmul` primitive
(which owns an allocated scratchpad) and as the CPU oracle both times.
Integer results: exact.  The second call must leave the amount of free device
memory as it found it, and the status word the kernels share with the host
must read zero after both.

The file name sorts last so that a run stopping at the first failure has
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from onednn_b200 import api, workloads as W
from onednn_b200.runner import run_problem
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _static_call(eng, p, zero_point):
    """Runs the problem through the allocation-free entry point on buffers
    created up front (library-owned memory objects), returns dst."""
    L = api.lib()
    L.dnnl_cuda_interop_matmul_u8s8s32_zp_static.argtypes = [
        C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]
    md = api.memory.desc
    src = api.memory(md((p.M, p.K), W.U8, api.tag.ab), eng)
    wei = api.memory(md((p.K, p.N), W.S8, api.tag.ab), eng)
    dst = api.memory(md((p.M, p.N), W.S32, api.tag.ab), eng)
    src.write(p.src.data)
    wei.write(p.wei.data)
    dst.write(np.full((p.M, p.N), -7, np.int32))
    strm = api.stream(eng)
    sp = C.c_void_p()
    assert L.dnnl_cuda_interop_stream_get_cuda_stream(strm._h, C.byref(sp)) == 0
    free_before = _free_device_bytes()
    st = L.dnnl_cuda_interop_matmul_u8s8s32_zp_static(
        sp, p.M, p.N, p.K, src.get_data_handle(), wei.get_data_handle(), zero_point, dst.get_data_handle())
    assert st == api.success, st
    # the companion call: waits for the stream, hands back the kernels' sticky status word
    L.dnnl_cuda_interop_matmul_u8s8s32_zp_static_status.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
    word = C.c_int(-1)
    assert L.dnnl_cuda_interop_matmul_u8s8s32_zp_static_status(sp, C.byref(word)) == api.success
    assert word.value == 0, "a kernel of the static entry point reported status %d" % word.value
    free_after = _free_device_bytes()
    strm.wait()
    return dst.read(np.int32).reshape(p.M, p.N), free_before, free_after


def _free_device_bytes():
    """Free device memory of the current context, as the driver reports it (cuMemGetInfo)."""
    drv = C.CDLL("libcuda.so.1")
    free, total = C.c_size_t(0), C.c_size_t(0)
    assert drv.cuMemGetInfo_v2(C.byref(free), C.byref(total)) == 0
    return free.value


def test_static_scratch_entry_point_matches_primitive_twice(gpu):
    eng, strm = gpu
    # two calls in a row on different operands, shapes and zero-points: the
    # second one finds the first one's sums in the shared array
    for seed, (M, K, N), zp in ((1, (256, 1024, 1024), 128), (2, (96, 272, 2064), 17)):
        p = W.int8_zp(M, K, N, seed=seed)
        p.quant["src_zp"] = W.Quant(np.array([zp], np.int32), W.S32, 0)
        want, impl = run_problem(p, eng, strm, impl="tcgen05")
        assert impl == "cuda:tcgen05:int8"
        got, free_before, free_after = _static_call(eng, p, zp)
        assert np.array_equal(got, want), "%d of %d values differ" % (int((got != want).sum()), want.size)
        assert np.array_equal(got, O.run_port(p).reshape(p.M, p.N)), "differs from the CPU oracle"
        if seed == 2:  # the first call on a device may still load its kernels; the second allocates nothing
            assert free_after == free_before, (free_before, free_after)


def test_static_scratch_entry_point_rejects_oversize(gpu):
    L = api.lib()
    L.dnnl_cuda_interop_matmul_u8s8s32_zp_static.argtypes = [
        C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]
    # N beyond the fixed array: refused before anything is launched
    st = L.dnnl_cuda_interop_matmul_u8s8s32_zp_static(None, 16, 131072 + 16, 16, 16, 16, 0, 16)
    assert st == api.invalid_arguments
    assert b"131072" in L.dnnl_cuda_interop_last_error()
