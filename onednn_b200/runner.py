"""Runs a :class:`workloads.Problem` through the library's public API.

``Prepared`` holds everything a caller of ``dnnl::matmul`` would hold: the
memory descriptors, the attributes, the primitive and one memory object per
execution argument.  Buffers are either allocated by the library and filled
through map/unmap (``upload``), or wrap device pointers the caller owns
(``bind_device``; used with torch tensors by the benchmark).
"""
import numpy as np

from . import api
from . import workloads as W


def _md(t: W.QTensor):
    return api.memory.desc(t.dims, t.dt, tuple(t.strides))


class Prepared:
    def __init__(self, p: W.Problem, eng, impl=None, user_scratchpad=False, runtime_m=False, dst_ld=None):
        """runtime_m: the primitive is created with M = DNNL_RUNTIME_DIM_VAL in src and dst (their
        strides given), and learns M from the memory objects at execution.  A pair (src mask, weights
        mask) instead of True leaves open the dims whose bits are set (src: bit 0 = M, bit 1 = K;
        weights: bit 0 = K, bit 1 = N), in dst, bias and binary operands too, together with the
        strides that depend on them.
        dst_ld: row pitch of dst in elements when dst is a column slice of a wider matrix."""
        self.p, self.eng = p, eng
        self.user_scratchpad = user_scratchpad
        grouped = p.offsets is not None
        if grouped:
            self.src_md = api.memory.desc.grouped((p.M, p.K), p.src.dt, 0, p.groups)
            self.dst_md = api.memory.desc.grouped((p.M, p.N), p.dst_dt, 0, p.groups)
        else:
            self.src_md = _md(p.src)
            self.dst_md = api.memory.desc((p.M, p.N), p.dst_dt, api.tag.ab if dst_ld is None else (dst_ld, 1))
        self.wei_md = _md(p.wei)
        self.bias_md = _md(p.bias) if p.bias is not None else None

        attr = api.primitive_attr()
        if p.apply_to_int or p.fpmath:
            attr.set_fpmath_mode(p.fpmath, p.apply_to_int)
        arg_of = {"src": api.ARG_SRC, "wei": api.ARG_WEIGHTS, "dst": api.ARG_DST}
        self.quant_args = {}
        for name, q in p.quant.items():
            arg = arg_of[name[:3]]
            groups = tuple(q.groups) if tuple(q.groups) != (1, 1) else ()
            if name.endswith("scale"):
                attr.set_scales(arg, q.mask, groups, q.dt)
                key = api.ARG_ATTR_SCALES | arg
            elif name.endswith("zp"):
                attr.set_zero_points(arg, q.mask, groups, q.dt)
                key = api.ARG_ATTR_ZERO_POINTS | arg
            else:
                attr.set_precomputed_reductions(arg, q.mask, groups, q.dt)
                key = api.ARG_ATTR_PRECOMPUTED_REDUCTIONS | arg
            self.quant_args[key] = q
        po = api.post_ops()
        self.binary_args = {}
        for i, e in enumerate(p.post_ops):
            if e.kind == W.PO_SUM:
                po.append_sum(e.scale, e.zero_point, 0)
            elif e.kind == W.PO_ELTWISE:
                po.append_eltwise(e.alg, e.alpha, e.beta)
            elif e.kind == W.PO_PRELU:
                po.append_prelu(sum(1 << d for d, n in enumerate(e.src1.dims) if n > 1))
                self.binary_args[api.ARG_ATTR_MULTIPLE_POST_OP(i) | api.ARG_WEIGHTS] = e.src1
            else:
                po.append_binary(e.alg, _md(e.src1))
                self.binary_args[api.ARG_ATTR_MULTIPLE_POST_OP(i) | api.ARG_SRC_1] = e.src1
        if p.post_ops:
            attr.set_post_ops(po)
        if user_scratchpad:
            attr.set_scratchpad_mode(api.SCRATCHPAD_MODE_USER)
        self.attr = attr
        pd_src, pd_wei, pd_dst, pd_bias, pd_attr = self.src_md, self.wei_md, self.dst_md, self.bias_md, attr
        if runtime_m is True:
            pd_src = api.memory.desc((api.RUNTIME_DIM_VAL, p.K), p.src.dt, tuple(p.src.strides))
            pd_dst = api.memory.desc((api.RUNTIME_DIM_VAL, p.N), p.dst_dt, (p.N, 1))
        elif runtime_m:
            smask, wmask = runtime_m
            open_m, open_k, open_n = bool(smask & 1), bool((smask & 2) or (wmask & 1)), bool(wmask & 2)

            def opened(dims, strides, dt, flags):
                """The descriptor with the flagged dims, and every stride that depends on one, left open."""
                RT = api.RUNTIME_DIM_VAL
                out, seen = list(strides), False
                for d in sorted(range(len(dims)), key=lambda i: (strides[i], -i)):
                    out[d] = RT if seen else strides[d]
                    seen = seen or flags[d]
                return api.memory.desc(tuple(RT if f else n for n, f in zip(dims, flags)), dt, tuple(out))

            pd_src = opened((p.M, p.K), p.src.strides, p.src.dt, (bool(smask & 1), bool(smask & 2)))
            pd_wei = opened((p.K, p.N), p.wei.strides, p.wei.dt, (bool(wmask & 1), bool(wmask & 2)))
            pd_dst = opened((p.M, p.N), (p.N, 1), p.dst_dt, (open_m, open_n))
            if p.bias is not None:
                pd_bias = opened(p.bias.dims, p.bias.strides, p.bias.dt,
                                 (open_m and p.bias.dims[0] > 1, open_n and p.bias.dims[1] > 1))
            if any(e.kind == W.PO_BINARY for e in p.post_ops):
                pd_attr = api.primitive_attr()
                if p.apply_to_int or p.fpmath:
                    pd_attr.set_fpmath_mode(p.fpmath, p.apply_to_int)
                for name, q in p.quant.items():
                    groups = tuple(q.groups) if tuple(q.groups) != (1, 1) else ()
                    setter = pd_attr.set_scales if name.endswith("scale") else pd_attr.set_zero_points if name.endswith("zp") \
                        else pd_attr.set_precomputed_reductions
                    setter(arg_of[name[:3]], q.mask, groups, q.dt)
                po2 = api.post_ops()
                for e in p.post_ops:
                    if e.kind == W.PO_SUM:
                        po2.append_sum(e.scale, e.zero_point, 0)
                    elif e.kind == W.PO_ELTWISE:
                        po2.append_eltwise(e.alg, e.alpha, e.beta)
                    elif e.kind == W.PO_PRELU:
                        po2.append_prelu(sum(1 << d for d, n in enumerate(e.src1.dims) if n > 1))
                    else:
                        po2.append_binary(e.alg, opened(e.src1.dims, e.src1.strides, e.src1.dt,
                                                        (open_m and e.src1.dims[0] > 1, open_n and e.src1.dims[1] > 1)))
                pd_attr.set_post_ops(po2)
                if user_scratchpad:
                    pd_attr.set_scratchpad_mode(api.SCRATCHPAD_MODE_USER)
        self.pd = api.matmul.primitive_desc(eng, pd_src, pd_wei, pd_dst, pd_bias, pd_attr)
        # descriptors of the quantization parameters come from a descriptor that knows M
        self.md_pd = api.matmul.primitive_desc(eng, self.src_md, self.wei_md, self.dst_md, self.bias_md, attr) \
            if runtime_m else self.pd
        if impl is not None:
            while impl not in self.pd.impl_info_str():
                if not self.pd.next_impl():
                    raise api.error(api.unimplemented, "no implementation named *%s*" % impl)
        self.impl = self.pd.impl_info_str()
        self.prim = api.matmul(self.pd)
        self.args = {}
        self._keep = []

    # ---- buffers owned by the library, filled through map/unmap
    def upload(self):
        p, eng = self.p, self.eng
        grouped = p.offsets is not None

        def put(md, arrays):
            m = api.memory(md, eng)
            for i, a in enumerate(arrays):
                if a is not None and a.nbytes:
                    m.write(np.ascontiguousarray(a), i)
            return m

        self.args[api.ARG_SRC] = put(self.src_md, [p.src.data, p.offsets] if grouped else [p.src.data])
        self.args[api.ARG_WEIGHTS] = put(self.wei_md, [p.wei.data])
        dst_init = p.dst_init
        if dst_init is None:
            dst_init = np.zeros(self.dst_md.get_size(0), np.uint8)
        self.args[api.ARG_DST] = put(self.dst_md, [dst_init, p.offsets] if grouped else [dst_init])
        if p.bias is not None:
            self.args[api.ARG_BIAS] = put(self.bias_md, [p.bias.data])
        for key, q in self.quant_args.items():
            md = self.md_pd.query_md(api.QUERY_EXEC_ARG_MD, key)
            self.args[key] = put(md, [q.data])
        for key, t in self.binary_args.items():
            self.args[key] = put(_md(t), [t.data])
        self._bind_scratchpad()
        return self

    def _bind_scratchpad(self):
        """scratchpad_mode::user: the caller provides the buffer the descriptor asks for
        (a zero-size request needs none); it is filled with a pattern, the library must not
        rely on its contents."""
        if not self.user_scratchpad:
            return
        md = self.pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_SCRATCHPAD)
        size = md.get_size(0)
        if size:
            m = api.memory(md, self.eng)
            m.write(np.full(size, 0xA5, np.uint8), 0)
            self.args[api.ARG_SCRATCHPAD] = m

    # ---- buffers owned by the caller (device pointers)
    def bind_device(self, ptrs):
        """ptrs: dict with device pointers (int) for 'src', 'wei', 'dst',
        optional 'bias', 'offsets', each quant name, and 'po<i>' for binary
        post-op operands."""
        p, eng = self.p, self.eng
        grouped = p.offsets is not None
        if grouped:
            self.args[api.ARG_SRC] = api.memory(self.src_md, eng, handles=[ptrs["src"], ptrs["offsets"]])
            self.args[api.ARG_DST] = api.memory(self.dst_md, eng, handles=[ptrs["dst"], ptrs["offsets"]])
        else:
            self.args[api.ARG_SRC] = api.memory(self.src_md, eng, ptrs["src"])
            self.args[api.ARG_DST] = api.memory(self.dst_md, eng, ptrs["dst"])
        self.args[api.ARG_WEIGHTS] = api.memory(self.wei_md, eng, ptrs["wei"])
        if p.bias is not None:
            self.args[api.ARG_BIAS] = api.memory(self.bias_md, eng, ptrs["bias"])
        arg_of = {"src": api.ARG_SRC, "wei": api.ARG_WEIGHTS, "dst": api.ARG_DST}
        for name in p.quant:
            arg = arg_of[name[:3]]
            base = (api.ARG_ATTR_SCALES if name.endswith("scale") else
                    api.ARG_ATTR_ZERO_POINTS if name.endswith("zp") else api.ARG_ATTR_PRECOMPUTED_REDUCTIONS)
            md = self.pd.query_md(api.QUERY_EXEC_ARG_MD, base | arg)
            self.args[base | arg] = api.memory(md, eng, ptrs[name])
        for i, e in enumerate(p.post_ops):
            if e.kind == W.PO_BINARY:
                self.args[api.ARG_ATTR_MULTIPLE_POST_OP(i) | api.ARG_SRC_1] = api.memory(_md(e.src1), eng, ptrs["po%d" % i])
            elif e.kind == W.PO_PRELU:
                self.args[api.ARG_ATTR_MULTIPLE_POST_OP(i) | api.ARG_WEIGHTS] = api.memory(_md(e.src1), eng, ptrs["po%d" % i])
        return self

    def execute(self, strm):
        self.prim.execute(strm, self.args)

    def download(self):
        dt = self.p.dst_dt
        raw = self.args[api.ARG_DST].read(np.uint8, 0)
        if dt in (W.S4, W.U4):
            return raw
        return raw.view(W.NP_STORAGE[dt]).reshape(self.p.M, self.p.N)


def run_reorder(r: W.Reorder, eng, strm):
    """Runs a :class:`workloads.Reorder` through ``dnnl::reorder``; returns (dst storage, flat and
    spanning the dst strides, implementation name)."""
    src_md = _md(r.src)
    dst_md = api.memory.desc(r.src.dims, r.dst_dt, tuple(r.dst_strides))
    attr = api.primitive_attr()
    arg_of = {"src": api.ARG_SRC, "dst": api.ARG_DST}
    quant_args = {}
    for name, q in r.quant.items():
        arg = arg_of[name[:3]]
        groups = tuple(q.groups) if tuple(q.groups) != (1, 1) else ()
        if name.endswith("scale"):
            attr.set_scales(arg, q.mask, groups, q.dt)
            quant_args[api.ARG_ATTR_SCALES | arg] = q
        else:
            attr.set_zero_points(arg, q.mask, groups, q.dt)
            quant_args[api.ARG_ATTR_ZERO_POINTS | arg] = q
    if r.beta:
        po = api.post_ops()
        po.append_sum(r.beta, 0, 0)
        attr.set_post_ops(po)
    pd = api.reorder.primitive_desc(eng, src_md, eng, dst_md, attr)

    def put(md, a):
        m = api.memory(md, eng)
        if a.nbytes:
            m.write(np.ascontiguousarray(a), 0)
        return m

    args = {api.ARG_FROM: put(src_md, r.src.data)}
    init = r.dst_init if r.dst_init is not None else np.zeros(dst_md.get_size(0), np.uint8)
    args[api.ARG_TO] = put(dst_md, init)
    for key, q in quant_args.items():
        args[key] = put(pd.query_md(api.QUERY_EXEC_ARG_MD, key), q.data)
    prim = api.reorder(pd)
    prim.execute(strm, args)
    strm.wait()
    raw = args[api.ARG_TO].read(np.uint8, 0)
    out = raw if r.dst_dt in (W.S4, W.U4) else raw.view(W.NP_STORAGE[r.dst_dt])
    return out, pd.impl_info_str()


def run_problem(p: W.Problem, eng, strm, impl=None, user_scratchpad=False, runtime_m=False):
    """Uploads, executes, waits, downloads.  Returns (dst, implementation)."""
    r = Prepared(p, eng, impl, user_scratchpad, runtime_m).upload()
    r.execute(strm)
    strm.wait()
    return r.download(), r.impl
