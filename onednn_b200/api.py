"""ctypes binding of the library's C API, shaped after ``dnnl.hpp``.

Class and method names follow oneDNN's C++ API (``engine``, ``stream``,
``memory.desc``, ``memory``, ``primitive_attr``, ``post_ops``,
``matmul.primitive_desc``, ``matmul``; include/oneapi/dnnl/dnnl.hpp) so code
and tests read like their oneDNN counterparts.  Errors raise :class:`error`
carrying the ``dnnl_status_t`` value, as ``dnnl::error`` does
(dnnl_common.hpp:84-106).  There is no fallback: if the CUDA library has not
been built the import of :func:`lib` fails.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))

# status codes (dnnl_common_types.h:45-68)
success, out_of_memory, invalid_arguments, unimplemented, last_impl_reached, runtime_error, \
    not_required = range(7)
_STATUS_NAME = ["success", "out_of_memory", "invalid_arguments", "unimplemented",
                "last_impl_reached", "runtime_error", "not_required"]

# exec-arg ids (dnnl_types.h:2542-2786)
ARG_SRC, ARG_SRC_1, ARG_DST, ARG_WEIGHTS, ARG_BIAS, ARG_SCRATCHPAD = 1, 2, 17, 33, 41, 80
ARG_FROM, ARG_TO = ARG_SRC, ARG_DST
SCRATCHPAD_MODE_LIBRARY, SCRATCHPAD_MODE_USER = 0, 1  # dnnl_scratchpad_mode_t
ARG_ATTR_SCALES, ARG_ATTR_ZERO_POINTS, ARG_ATTR_PRECOMPUTED_REDUCTIONS = 4096, 8192, 512


def ARG_ATTR_MULTIPLE_POST_OP(idx):
    return 32768 * (idx + 1)


MEMORY_ALLOCATE = C.c_void_p(2 ** 64 - 1)
MEMORY_NONE = C.c_void_p(0)

QUERY_IMPL_INFO_STR = 8
QUERY_SRC_MD, QUERY_WEIGHTS_MD, QUERY_DST_MD, QUERY_EXEC_ARG_MD = 129, 131, 133, 255
QUERY_NDIMS, QUERY_DIMS, QUERY_DATA_TYPE, QUERY_FORMAT_KIND, QUERY_STRIDES = 256, 257, 258, 262, 14
QUERY_NUM_HANDLES = 268

KIND_SUM, KIND_ELTWISE, KIND_BINARY, KIND_MATMUL, KIND_PRELU = 4, 7, 13, 14, 18


class tag:
    undef, any, a, ab, abc, abcd, ba, acb, bac, bca, cab, cba = 0, 1, 2, 3, 4, 5, 14, 15, 16, 17, 18, 19


class error(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        name = _STATUS_NAME[status] if 0 <= status < len(_STATUS_NAME) else str(status)
        detail = lib().dnnl_cuda_interop_last_error().decode() if status == runtime_error else ""
        super().__init__("%s: %s %s" % (what, name, detail))


_lib = None
_dims_t = C.c_int64 * 12


class _ExecArg(C.Structure):
    _fields_ = [("arg", C.c_int), ("memory", C.c_void_p)]


def lib_path():
    return os.path.join(_HERE, "lib", "libdnnl.so.3")


def lib():
    """The loaded CUDA library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError("%s is missing: run `python -m onednn_b200.build`" % path)
        L = C.CDLL(path, mode=os.RTLD_LOCAL)
        L.dnnl_engine_get_count.restype = C.c_size_t
        L.dnnl_memory_desc_get_size.restype = C.c_size_t
        L.dnnl_memory_desc_get_size_v2.restype = C.c_size_t
        L.dnnl_data_type_size.restype = C.c_size_t
        L.dnnl_cuda_interop_launch_count.restype = C.c_uint64
        L.dnnl_cuda_interop_last_error.restype = C.c_char_p
        L.dnnl_primitive_desc_query_md.restype = C.c_void_p
        L.dnnl_version.restype = C.c_void_p
        L.dnnl_post_ops_append_eltwise.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_float]
        L.dnnl_post_ops_append_sum.argtypes = [C.c_void_p, C.c_float, C.c_int32, C.c_int]
        L.dnnl_engine_create.argtypes = [C.c_void_p, C.c_int, C.c_size_t]
        _lib = L
    return _lib


def _check(status, what):
    if status != success:
        raise error(status, what)


RUNTIME_DIM_VAL = -(1 << 63)  # DNNL_RUNTIME_DIM_VAL


def _dims(seq):
    d = _dims_t()
    for i, v in enumerate(seq):
        d[i] = int(v)
    return d


class engine:
    class kind:
        any, cpu, gpu = 0, 1, 2

    @staticmethod
    def get_count(kind):
        return int(lib().dnnl_engine_get_count(kind))

    def __init__(self, kind, index):
        self._h = C.c_void_p()
        _check(lib().dnnl_engine_create(C.byref(self._h), kind, index), "could not create an engine")

    def get_kind(self):
        k = C.c_int()
        _check(lib().dnnl_engine_get_kind(self._h, C.byref(k)), "could not get kind of an engine")
        return k.value

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.dnnl_engine_destroy(self._h)


class stream:
    def __init__(self, eng, cuda_stream=None):
        """`cuda_stream`: an existing cudaStream_t value (int) to enqueue on."""
        self._h = C.c_void_p()
        self._eng = eng
        if cuda_stream is None:
            _check(lib().dnnl_stream_create(C.byref(self._h), eng._h, 1), "could not create a stream")
        else:
            _check(lib().dnnl_cuda_interop_stream_create(C.byref(self._h), eng._h, C.c_void_p(cuda_stream)),
                   "could not create a stream")

    def wait(self):
        _check(lib().dnnl_stream_wait(self._h), "could not wait on a stream")
        return self

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.dnnl_stream_destroy(self._h)


class memory:
    class desc:
        def __init__(self, dims=None, data_type=0, fmt=None, _handle=None, _own=True):
            """fmt: a `tag` value or a tuple of strides."""
            self._own = _own
            if _handle is not None:
                self._h = C.c_void_p(_handle)
                return
            self._h = C.c_void_p()
            if dims is None:
                _check(lib().dnnl_memory_desc_create_with_tag(C.byref(self._h), 0, None, 0, 0),
                       "could not create a zero memory descriptor")
            elif isinstance(fmt, (tuple, list)):
                _check(lib().dnnl_memory_desc_create_with_strides(
                    C.byref(self._h), len(dims), _dims(dims), data_type, _dims(fmt)),
                    "could not construct a memory descriptor using strides")
            else:
                _check(lib().dnnl_memory_desc_create_with_tag(
                    C.byref(self._h), len(dims), _dims(dims), data_type, int(fmt)),
                    "could not construct a memory descriptor using a format tag")

        @staticmethod
        def grouped(dims, data_type, variable_dim_idx, group_count, offsets_dt=4):
            h = C.c_void_p()
            _check(lib().dnnl_memory_desc_create_with_grouped_encoding(
                C.byref(h), len(dims), _dims(dims), data_type, variable_dim_idx,
                C.c_int64(group_count), offsets_dt), "could not create a grouped memory descriptor")
            return memory.desc(_handle=h.value)

        @staticmethod
        def host_scalar(data_type):
            h = C.c_void_p()
            _check(lib().dnnl_memory_desc_create_host_scalar(C.byref(h), data_type),
                   "could not create a host scalar memory descriptor")
            return memory.desc(_handle=h.value)

        def _query(self, what, ctype):
            v = ctype()
            _check(lib().dnnl_memory_desc_query(self._h, what, C.byref(v)), "could not query a memory descriptor")
            return v

        def get_ndims(self):
            return self._query(QUERY_NDIMS, C.c_int).value

        def get_dims(self):
            p = self._query(QUERY_DIMS, C.POINTER(_dims_t))
            return tuple(p.contents[i] for i in range(self.get_ndims()))

        def get_strides(self):
            p = self._query(QUERY_STRIDES, C.POINTER(_dims_t))
            return tuple(p.contents[i] for i in range(self.get_ndims()))

        def get_data_type(self):
            return self._query(QUERY_DATA_TYPE, C.c_int).value

        def get_format_kind(self):
            return self._query(QUERY_FORMAT_KIND, C.c_int).value

        def get_num_handles(self):
            return self._query(QUERY_NUM_HANDLES, C.c_int).value

        def get_size(self, index=0):
            return int(lib().dnnl_memory_desc_get_size_v2(self._h, index))

        def __eq__(self, other):
            return bool(lib().dnnl_memory_desc_equal(self._h, other._h))

        def __del__(self):
            if self._own and getattr(self, "_h", None) and _lib is not None:
                _lib.dnnl_memory_desc_destroy(self._h)

    def __init__(self, md, eng, handle=None, handles=None):
        """handle(s): device pointer(s) as int; None lets the library allocate."""
        self._h = C.c_void_p()
        self._md, self._eng = md, eng
        n = md.get_num_handles()
        if handles is None:
            handles = [handle] * n if handle is None else [handle]
        arr = (C.c_void_p * max(1, n))()
        for i in range(n):
            arr[i] = MEMORY_ALLOCATE.value if handles[i] is None else handles[i]
        _check(lib().dnnl_memory_create_v2(C.byref(self._h), md._h, eng._h, n, arr),
               "could not create a memory object")

    @staticmethod
    def host_scalar(md, value_ctypes):
        m = memory.__new__(memory)
        m._h = C.c_void_p()
        m._md, m._eng = md, None
        _check(lib().dnnl_memory_create_host_scalar(C.byref(m._h), md._h, C.byref(value_ctypes)),
               "could not create a host scalar memory object")
        return m

    def get_data_handle(self, index=0):
        p = C.c_void_p()
        _check(lib().dnnl_memory_get_data_handle_v2(self._h, C.byref(p), index), "could not get a native handle")
        return p.value

    def set_data_handle(self, ptr, index=0):
        _check(lib().dnnl_memory_set_data_handle_v2(self._h, C.c_void_p(ptr), index), "could not set a native handle")

    def map_data(self, index=0):
        p = C.c_void_p()
        _check(lib().dnnl_memory_map_data_v2(self._h, C.byref(p), index), "could not map memory object data")
        return p.value

    def unmap_data(self, ptr, index=0):
        _check(lib().dnnl_memory_unmap_data_v2(self._h, C.c_void_p(ptr), index), "could not unmap memory object data")

    def write(self, array, index=0):
        """Copies a numpy array into the buffer through map/unmap."""
        p = self.map_data(index)
        n = self._md.get_size(index)
        assert array.nbytes == n, (array.nbytes, n)
        C.memmove(p, array.ctypes.data, n)
        self.unmap_data(p, index)

    def read(self, np_dtype, index=0):
        import numpy as np
        n = self._md.get_size(index)
        out = np.empty(n, np.uint8)
        p = self.map_data(index)
        C.memmove(out.ctypes.data, p, n)
        self.unmap_data(p, index)
        return out.view(np_dtype)

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.dnnl_memory_destroy(self._h)


class post_ops:
    def __init__(self):
        self._h = C.c_void_p()
        _check(lib().dnnl_post_ops_create(C.byref(self._h)), "could not create post-ops")

    def len(self):
        return lib().dnnl_post_ops_len(self._h)

    def kind(self, index):
        return lib().dnnl_post_ops_get_kind(self._h, index)

    def append_sum(self, scale=1.0, zero_point=0, data_type=0):
        _check(lib().dnnl_post_ops_append_sum(self._h, scale, zero_point, data_type), "could not append a sum post-op")

    def append_eltwise(self, alg, alpha, beta):
        _check(lib().dnnl_post_ops_append_eltwise(self._h, alg, alpha, beta),
               "could not append an elementwise post-op")

    def append_binary(self, alg, src1_desc):
        _check(lib().dnnl_post_ops_append_binary(self._h, alg, src1_desc._h), "could not append a binary post-op")

    def append_prelu(self, mask):
        _check(lib().dnnl_post_ops_append_prelu(self._h, mask), "could not append a prelu post-op")

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.dnnl_post_ops_destroy(self._h)


class fpmath_mode:
    strict, bf16, f16, any, tf32 = range(5)


class primitive_attr:
    def __init__(self):
        self._h = C.c_void_p()
        _check(lib().dnnl_primitive_attr_create(C.byref(self._h)), "could not create primitive attribute")

    def set_fpmath_mode(self, mode, apply_to_int=False):
        _check(lib().dnnl_primitive_attr_set_fpmath_mode_v2(self._h, mode, int(apply_to_int)),
               "could not set fpmath mode primitive attribute")

    def get_fpmath_mode(self):
        m, a = C.c_int(), C.c_int()
        _check(lib().dnnl_primitive_attr_get_fpmath_mode_v2(self._h, C.byref(m), C.byref(a)),
               "could not get fpmath mode primitive attribute")
        return m.value, bool(a.value)

    def set_scales_mask(self, arg, mask):
        _check(lib().dnnl_primitive_attr_set_scales_mask(self._h, arg, mask), "could not set scales primitive attribute")

    def set_scales(self, arg, mask, groups=(), data_type=3, is_on_host=False, qmode=1):
        _check(lib().dnnl_primitive_attr_set_scales_v3(self._h, arg, mask, len(groups), _dims(groups), data_type,
                                                       int(is_on_host), qmode),
               "could not set scales primitive attribute")

    def set_zero_points_mask(self, arg, mask):
        _check(lib().dnnl_primitive_attr_set_zero_points_mask(self._h, arg, mask),
               "could not set zero points primitive attribute")

    def set_zero_points(self, arg, mask, groups=(), data_type=4, is_on_host=False):
        _check(lib().dnnl_primitive_attr_set_zero_points_v2(self._h, arg, mask, len(groups), _dims(groups),
                                                            data_type, int(is_on_host)),
               "could not set zero points primitive attribute")

    def set_precomputed_reductions(self, arg, mask, groups=(), data_type=4):
        _check(lib().dnnl_primitive_attr_set_precomputed_reductions(self._h, arg, mask, len(groups), _dims(groups),
                                                                    data_type),
               "could not set precomputed reductions primitive attribute")

    def set_post_ops(self, po):
        _check(lib().dnnl_primitive_attr_set_post_ops(self._h, po._h), "could not set post-ops primitive attribute")

    def set_scratchpad_mode(self, mode):
        _check(lib().dnnl_primitive_attr_set_scratchpad_mode(self._h, mode),
               "could not set scratchpad mode primitive attribute")

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.dnnl_primitive_attr_destroy(self._h)


class matmul:
    class primitive_desc:
        def __init__(self, eng, src_md, weights_md, dst_md, bias_md=None, attr=None):
            self._h = C.c_void_p()
            self._eng = eng
            _check(lib().dnnl_matmul_primitive_desc_create(
                C.byref(self._h), eng._h, src_md._h, weights_md._h, bias_md._h if bias_md is not None else None,
                dst_md._h, attr._h if attr is not None else None),
                "could not create a primitive descriptor for the matmul primitive")

        def next_impl(self):
            st = lib().dnnl_primitive_desc_next_impl(self._h)
            if st == last_impl_reached:
                return False
            _check(st, "could not advance a primitive descriptor to the next implementation")
            return True

        def impl_info_str(self):
            s = C.c_char_p()
            _check(lib().dnnl_primitive_desc_query(self._h, QUERY_IMPL_INFO_STR, 0, C.byref(s)),
                   "could not retrieve implementation info string")
            return s.value.decode()

        def query_md(self, what, index=0):
            p = lib().dnnl_primitive_desc_query_md(self._h, what, index)
            return memory.desc(_handle=p, _own=False) if p else None

        def src_desc(self):
            return self.query_md(QUERY_SRC_MD)

        def weights_desc(self):
            return self.query_md(QUERY_WEIGHTS_MD)

        def dst_desc(self):
            return self.query_md(QUERY_DST_MD)

        def __del__(self):
            if getattr(self, "_h", None) and _lib is not None:
                _lib.dnnl_primitive_desc_destroy(self._h)

    def __init__(self, pd):
        self._h = C.c_void_p()
        self._pd = pd
        _check(lib().dnnl_primitive_create(C.byref(self._h), pd._h), "could not create a primitive")

    def execute(self, strm, args):
        """args: dict exec-arg id -> memory, as in dnnl::primitive::execute."""
        n = len(args)
        arr = (_ExecArg * max(1, n))()
        for i, (k, m) in enumerate(args.items()):
            arr[i].arg = k
            arr[i].memory = m._h.value
        _check(lib().dnnl_primitive_execute(self._h, strm._h, n, arr), "could not execute a primitive")

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.dnnl_primitive_destroy(self._h)


class reorder(matmul):
    """dnnl::reorder: ``reorder(reorder.primitive_desc(eng, src_md, eng, dst_md, attr)).execute(strm,
    {ARG_FROM: src, ARG_TO: dst, ...})``.  Creation, execution and destruction are the primitive's own."""

    class primitive_desc(matmul.primitive_desc):
        def __init__(self, src_eng, src_md, dst_eng, dst_md, attr=None):
            self._h = C.c_void_p()
            self._eng = src_eng
            _check(lib().dnnl_reorder_primitive_desc_create(
                C.byref(self._h), src_md._h, src_eng._h, dst_md._h, dst_eng._h,
                attr._h if attr is not None else None),
                "could not create a primitive descriptor for a reorder primitive")


def launch_count():
    return int(lib().dnnl_cuda_interop_launch_count())
