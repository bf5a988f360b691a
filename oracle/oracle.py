"""ctypes front-end to the CPU oracle -- TEST INFRASTRUCTURE ONLY.

``run_port``  runs the plain-C restatement (``qmm_oracle.c``).
``run_ref``   runs the unmodified reference library through ``ref_runner.cpp``
              when ``oracle/_ref`` holds a build of it.
Both take a ``onednn_b200.workloads.Problem`` and return the dst buffer.
Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
import ctypes as C
import os

import numpy as np

from onednn_b200 import workloads as W

HERE = os.path.dirname(os.path.abspath(__file__))


class _Quant(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dt", C.c_int32), ("mask", C.c_int32),
                ("g0", C.c_int64), ("g1", C.c_int64), ("ld", C.c_int64)]


class _PostOp(C.Structure):
    _fields_ = [("kind", C.c_int32), ("alg", C.c_int32), ("alpha", C.c_float),
                ("beta", C.c_float), ("scale", C.c_float), ("zero_point", C.c_int32),
                ("src1_dt", C.c_int32), ("src1", C.c_void_p),
                ("src1_sm", C.c_int64), ("src1_sn", C.c_int64)]


class _Problem(C.Structure):
    _fields_ = [("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
                ("src", C.c_void_p), ("src_dt", C.c_int32),
                ("src_sm", C.c_int64), ("src_sk", C.c_int64),
                ("wei", C.c_void_p), ("wei_dt", C.c_int32),
                ("wei_sk", C.c_int64), ("wei_sn", C.c_int64),
                ("bias", C.c_void_p), ("bias_dt", C.c_int32),
                ("bias_sm", C.c_int64), ("bias_sn", C.c_int64),
                ("dst", C.c_void_p), ("dst_dt", C.c_int32),
                ("dst_sm", C.c_int64), ("dst_sn", C.c_int64),
                ("src_scale", _Quant), ("wei_scale", _Quant), ("dst_scale", _Quant),
                ("src_zp", _Quant), ("wei_zp", _Quant), ("dst_zp", _Quant),
                ("src_pr", _Quant),
                ("apply_to_int", C.c_int32), ("non_default_attr", C.c_int32),
                ("sum_dt", C.c_int32), ("n_po", C.c_int32), ("po", _PostOp * 32),
                ("rows", C.c_void_p), ("n_rows", C.c_int64),
                ("group_count", C.c_int64), ("offsets", C.c_void_p),
                ("wei_sg", C.c_int64), ("bias_sg", C.c_int64), ("fpmath_mode", C.c_int32)]


class _RQuant(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dt", C.c_int32), ("mask", C.c_int32),
                ("g0", C.c_int64), ("g1", C.c_int64)]


class _Reorder(C.Structure):
    _fields_ = [("ndims", C.c_int32), ("dims", C.c_int64 * 6),
                ("src", C.c_void_p), ("src_dt", C.c_int32), ("src_strides", C.c_int64 * 6),
                ("dst", C.c_void_p), ("dst_dt", C.c_int32), ("dst_strides", C.c_int64 * 6),
                ("src_scale", _RQuant), ("dst_scale", _RQuant), ("src_zp", _RQuant), ("dst_zp", _RQuant),
                ("beta", C.c_float)]


_port = None
_ref = None


def _load_port():
    global _port
    if _port is None:
        from oracle import build_oracle
        _port = C.CDLL(build_oracle.build_port())
        for f in (_port.qmm_oracle_int8, _port.qmm_oracle_fp, _port.qmm_oracle_grouped):
            f.argtypes = [C.POINTER(_Problem)]
            f.restype = C.c_int
        _port.qmm_oracle_reorder.argtypes = [C.POINTER(_Reorder)]
        _port.qmm_oracle_reorder.restype = C.c_int
    return _port


def ref_available() -> bool:
    return os.path.exists(os.path.join(HERE, "_ref", "libref_runner.so"))


def _load_ref():
    global _ref
    if _ref is None:
        _ref = C.CDLL(os.path.join(HERE, "_ref", "libref_runner.so"), mode=os.RTLD_LOCAL)
        _ref.ref_runner_run.argtypes = [C.POINTER(_Problem), C.c_int, C.c_int,
                                        C.POINTER(C.c_double), C.c_char_p, C.c_int]
        _ref.ref_runner_run.restype = C.c_int
        _ref.ref_runner_reorder.argtypes = [C.POINTER(_Reorder), C.c_char_p, C.c_int]
        _ref.ref_runner_reorder.restype = C.c_int
    return _ref


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _marshal(p: W.Problem, rows=None):
    """Builds the C struct; returns (struct, dst array, keepalive list)."""
    keep = []
    s = _Problem()
    s.M, s.N, s.K = p.M, p.N, p.K
    grouped = p.offsets is not None
    s.src, s.src_dt = _ptr(p.src.data), p.src.dt
    s.src_sm, s.src_sk = p.src.strides
    s.wei, s.wei_dt = _ptr(p.wei.data), p.wei.dt
    if grouped:
        s.wei_sg, s.wei_sk, s.wei_sn = p.wei.strides
    else:
        s.wei_sk, s.wei_sn = p.wei.strides
    if p.bias is not None:
        s.bias, s.bias_dt = _ptr(p.bias.data), p.bias.dt
        if grouped:
            s.bias_sg = p.N
        else:
            s.bias_sm = p.bias.strides[0] if p.bias.dims[0] > 1 else 0
            s.bias_sn = p.bias.strides[1] if p.bias.dims[1] > 1 else 0
    dst = np.zeros(W.nbytes(p.dst_dt, p.M * p.N), np.uint8)
    if p.dst_init is not None:
        dst[:] = p.dst_init.view(np.uint8).reshape(-1)
    keep.append(dst)
    s.dst, s.dst_dt = _ptr(dst), p.dst_dt
    s.dst_sm, s.dst_sn = p.N, 1
    for name in ("src_scale", "wei_scale", "dst_scale", "src_zp", "wei_zp", "dst_zp", "src_pr"):
        q = p.quant.get(name)
        if q is None:
            continue
        cq = getattr(s, name)
        cq.ptr, cq.dt = _ptr(q.data), q.dt
        mask = q.mask
        if grouped and name.startswith("wei"):
            mask = (mask >> 1) & 3  # drop the group dim: bit0 = K, bit1 = N
        cq.mask = mask
        cq.g0, cq.g1 = q.groups
        d1 = {"src": p.K, "wei": p.N, "dst": p.N}[name[:3]]
        cq.ld = (d1 // cq.g1) if (mask & 2) else 1
    s.apply_to_int = int(p.apply_to_int)
    s.fpmath_mode = p.fpmath
    s.non_default_attr = int(bool(p.quant) or bool(p.post_ops) or p.apply_to_int)
    s.sum_dt = p.dst_dt
    s.n_po = len(p.post_ops)
    for i, po in enumerate(p.post_ops):
        e = s.po[i]
        e.kind, e.alg, e.alpha, e.beta, e.scale = po.kind, po.alg, po.alpha, po.beta, po.scale
        e.zero_point = po.zero_point
        if po.src1 is not None:
            e.src1, e.src1_dt = _ptr(po.src1.data), po.src1.dt
            e.src1_sm = po.src1.strides[0] if po.src1.dims[0] > 1 else 0
            e.src1_sn = po.src1.strides[1] if po.src1.dims[1] > 1 else 0
    if rows is not None:
        r = np.ascontiguousarray(rows, dtype=np.int64)
        keep.append(r)
        s.rows, s.n_rows = _ptr(r), len(r)
    if grouped:
        s.group_count = p.groups
        s.offsets = _ptr(p.offsets)
    return s, dst, keep


def _view(dst: np.ndarray, p: W.Problem):
    if p.dst_dt in (W.S4, W.U4):
        return dst
    return dst.view(W.NP_STORAGE[p.dst_dt]).reshape(p.M, p.N)


def run_port(p: W.Problem, rows=None) -> np.ndarray:
    """dst of the C restatement.  With `rows`, only those rows are computed
    (the others stay zero)."""
    lib = _load_port()
    s, dst, keep = _marshal(p, rows)
    if p.offsets is not None:
        rc = lib.qmm_oracle_grouped(C.byref(s))
    elif p.src.dt in (W.S8, W.U8):
        rc = lib.qmm_oracle_int8(C.byref(s))
    else:
        rc = lib.qmm_oracle_fp(C.byref(s))
    if rc != 0:
        raise RuntimeError("oracle status %d" % rc)
    return _view(dst, p)


def run_ref(p: W.Problem, pin_ref=True, iters=0):
    """(dst, implementation name, best ms or None) from the reference library."""
    lib = _load_ref()
    s, dst, keep = _marshal(p)
    ms = C.c_double(0.0)
    name = C.create_string_buffer(256)
    rc = lib.ref_runner_run(C.byref(s), int(pin_ref), int(iters), C.byref(ms), name, 256)
    if rc != 0:
        raise RuntimeError("reference status %d: %s" % (rc, name.value.decode()))
    return _view(dst, p), name.value.decode(), (ms.value if iters > 0 else None)


class _NdTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dt", C.c_int32), ("ndims", C.c_int32),
                ("dims", C.c_int64 * 6), ("strides", C.c_int64 * 6)]


class _NdQuant(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dt", C.c_int32), ("mask", C.c_int32), ("arg", C.c_int32), ("kind", C.c_int32),
                ("g0", C.c_int64), ("g1", C.c_int64)]


class _NdPostOp(C.Structure):
    _fields_ = [("kind", C.c_int32), ("alg", C.c_int32), ("zero_point", C.c_int32), ("mask", C.c_int32),
                ("alpha", C.c_float), ("beta", C.c_float), ("scale", C.c_float), ("src1", _NdTensor)]


class _NdProblem(C.Structure):
    _fields_ = [("src", _NdTensor), ("wei", _NdTensor), ("dst", _NdTensor), ("bias", _NdTensor),
                ("n_quant", C.c_int32), ("n_po", C.c_int32), ("apply_to_int", C.c_int32), ("fpmath_mode", C.c_int32),
                ("quant", _NdQuant * 8), ("po", _NdPostOp * 8)]


def run_ref_nd(src, wei, bias, dst_dims, dst_dt, dst_strides, quant, post_ops, dst_init=None,
               apply_to_int=False, fpmath=0, pin_ref=True):
    """A matmul of any rank on the reference library (batched problems).  src / wei / bias:
    (storage, element strides, data type, dims) or None; quant: name -> Quant with a mask over all
    dims; post_ops: PostOp whose binary src1 is a QTensor of dst's rank; a prelu carries its mask in
    zero_point and its weights in src1.data in the layout the reference defines.  Returns (dst
    storage spanning dst_strides, implementation name)."""
    lib = _load_ref()
    keep = []

    def tensor(t, ptr, dt, dims, strides):
        t.ptr, t.dt, t.ndims = ptr, dt, len(dims)
        for i, (d, st) in enumerate(zip(dims, strides)):
            t.dims[i], t.strides[i] = d, st

    s = _NdProblem()
    for field, given in (("src", src), ("wei", wei), ("bias", bias)):
        if given is not None:
            storage, strides, dt, dims = given
            keep.append(storage)
            tensor(getattr(s, field), _ptr(storage).value, dt, dims, strides)
    span = 1 + sum((d - 1) * st for d, st in zip(dst_dims, dst_strides))
    dst = np.zeros(W.nbytes(dst_dt, span), np.uint8)
    if dst_init is not None:
        dst[:] = np.ascontiguousarray(dst_init).view(np.uint8).reshape(-1)
    tensor(s.dst, _ptr(dst).value, dst_dt, dst_dims, dst_strides)
    arg_of = {"src": 1, "wei": 33, "dst": 17}  # DNNL_ARG_SRC, DNNL_ARG_WEIGHTS, DNNL_ARG_DST
    for i, (name, q) in enumerate(quant.items()):
        cq = s.quant[i]
        cq.ptr, cq.dt, cq.mask, cq.arg = _ptr(q.data).value, q.dt, q.mask, arg_of[name[:3]]
        cq.kind = 0 if name.endswith("scale") else 1
        cq.g0, cq.g1 = q.groups
    s.n_quant = len(quant)
    for i, po in enumerate(post_ops):
        e = s.po[i]
        e.kind, e.alg, e.alpha, e.beta, e.scale, e.zero_point = po.kind, po.alg, po.alpha, po.beta, po.scale, po.zero_point
        if po.kind == W.PO_PRELU:
            e.mask = po.zero_point
            e.src1.ptr = _ptr(po.src1.data).value
        elif po.src1 is not None:
            tensor(e.src1, _ptr(po.src1.data).value, po.src1.dt, po.src1.dims, po.src1.strides)
    s.n_po = len(post_ops)
    s.apply_to_int, s.fpmath_mode = int(apply_to_int), fpmath
    name = C.create_string_buffer(256)
    rc = lib.ref_runner_run_nd(C.byref(s), int(pin_ref), name, 256)
    if rc != 0:
        raise RuntimeError("reference status %d: %s" % (rc, name.value.decode()))
    out = dst if dst_dt in (W.S4, W.U4) else dst.view(W.NP_STORAGE[dst_dt])
    return out, name.value.decode()


def _marshal_reorder(r: W.Reorder):
    s = _Reorder()
    nd = len(r.src.dims)
    s.ndims = nd
    for i in range(nd):
        s.dims[i] = r.src.dims[i]
        s.src_strides[i] = r.src.strides[i]
        s.dst_strides[i] = r.dst_strides[i]
    s.src, s.src_dt = _ptr(r.src.data), r.src.dt
    dst = np.zeros(W.nbytes(r.dst_dt, r.dst_nelems()), np.uint8)
    if r.dst_init is not None:
        dst[:] = r.dst_init.view(np.uint8).reshape(-1)
    s.dst, s.dst_dt = _ptr(dst), r.dst_dt
    for name in ("src_scale", "dst_scale", "src_zp", "dst_zp"):
        q = r.quant.get(name)
        if q is None:
            continue
        cq = getattr(s, name)
        cq.ptr, cq.dt, cq.mask = _ptr(q.data), q.dt, q.mask
        cq.g0, cq.g1 = q.groups
    for name in ("src_scale", "dst_scale", "src_zp", "dst_zp"):
        if r.quant.get(name) is None:
            getattr(s, name).g0 = getattr(s, name).g1 = 1
    s.beta = r.beta
    return s, dst


def _view_reorder(dst: np.ndarray, r: W.Reorder):
    return dst if r.dst_dt in (W.S4, W.U4) else dst.view(W.NP_STORAGE[r.dst_dt])


def run_port_reorder(r: W.Reorder) -> np.ndarray:
    """dst storage (flat, spanning the dst strides) of the C restatement of the reorder."""
    lib = _load_port()
    s, dst = _marshal_reorder(r)
    rc = lib.qmm_oracle_reorder(C.byref(s))
    if rc != 0:
        raise RuntimeError("oracle status %d" % rc)
    return _view_reorder(dst, r)


def run_ref_reorder(r: W.Reorder):
    """(dst storage, implementation name) from the reference library."""
    lib = _load_ref()
    s, dst = _marshal_reorder(r)
    name = C.create_string_buffer(256)
    rc = lib.ref_runner_reorder(C.byref(s), name, 256)
    if rc != 0:
        raise RuntimeError("reference status %d: %s" % (rc, name.value.decode()))
    return _view_reorder(dst, r), name.value.decode()
