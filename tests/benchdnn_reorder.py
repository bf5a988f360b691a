"""Reorder problems written in the syntax of oneDNN's benchdnn driver
(tests/benchdnn/doc/driver_reorder.md in oneDNN), as `workloads.Reorder`
objects for the CPU oracle and for `dnnl::reorder` of this library.

    --sdt=f32,s8 --ddt=s8 --stag=abx --dtag=axb,xba
    --attr-scales=src:per_dim_1+dst:common:2 --attr-zero-points=src:common:-1+dst:common:2
    --attr-post-ops=sum:0.5
    2x16x3x4 30x1

Plain layouts only: a tag names the dims from the outermost to the innermost,
`x` standing for the dims the tag does not name, in order (normalize_tag,
tests/benchdnn/dnn_types.cpp:1884-1912).  Blocked tags, compensation flags
(--oflag), run-time dim masks and fp4 / f64 types are skipped with their name
as the reason; 4-bit tensors are packed two elements a byte along their
innermost dim."""
import re
import zlib

import numpy as np

import benchdnn_matmul as B
from onednn_b200 import workloads as W

DEFAULTS = {"sdt": "f32", "ddt": "f32", "stag": "abx", "dtag": "abx", "attr-scales": "", "attr-zero-points": "",
            "attr-post-ops": "", "oflag": "", "runtime-dim-mask": "0", "strides": "", "attr-scratchpad": "library",
            "attr-rounding-mode": "", "attr-dropout": ""}
Skip = B.Skip


def expand(path):
    return B.expand(path, defaults=DEFAULTS)


def tag_order(tag, nd):
    """Physical order of the dims, outermost first."""
    if tag in ("any", "undef"):
        return tuple(range(nd))
    if not re.fullmatch(r"[a-lx]+", tag):
        raise Skip("tag " + tag)
    if "x" in tag:
        named = [ord(c) - ord("a") for c in tag if c != "x"]
        start = max(named + [1]) + 1
        tag = tag.replace("x", "".join(chr(ord("a") + i) for i in range(start, max(nd, start))))
    order = [ord(c) - ord("a") for c in tag if ord(c) - ord("a") < nd]
    if sorted(order) != list(range(nd)):
        raise Skip("tag %s for %d dims" % (tag, nd))
    return tuple(order)


def _strides(dims, order):
    strides, acc = [0] * len(dims), 1
    for d in reversed(order):
        strides[d] = acc
        acc *= dims[d]
    return tuple(strides)


def _values(r, dt, dims):
    """Values that exercise rounding and saturation of the narrower types.  No negative zeros,
    as in benchdnn's own fill (integers converted to floats): the reference's reorder
    implementations do not agree on the sign of a zero result (its jit kernels keep -0, the
    scalar `simple:any` path with scales returns +0)."""
    if dt in (W.S8, W.U8, W.S32, W.S4, W.U4):
        lo, hi = {W.U8: (0, 256), W.S8: (-128, 128), W.S32: (-300, 301), W.S4: (-8, 8), W.U4: (0, 16)}[dt]
        return r.integers(lo, hi, dims)
    if dt in (W.F8_E4M3, W.F8_E5M2):
        return r.integers(-16, 17, dims).astype(np.float32) * 0.5
    return np.round(r.standard_normal(dims) * 80.0 * 4) / 4 + 0.0  # quarters, beyond the 8-bit ranges now and then


def build(settings, desc):
    """workloads.Reorder of one expanded problem, or raises Skip."""
    if settings.get("_unknown"):
        raise Skip("option --" + settings["_unknown"][0])
    for k in ("oflag", "strides", "attr-rounding-mode", "attr-dropout"):
        if settings[k]:
            raise Skip("--" + k)
    if settings["runtime-dim-mask"] not in ("", "0"):
        raise Skip("run-time dims")
    if settings["sdt"] not in B.DT or settings["ddt"] not in B.DT:
        raise Skip("data types %s -> %s" % (settings["sdt"], settings["ddt"]))
    sdt, ddt = B.DT[settings["sdt"]], B.DT[settings["ddt"]]
    m = re.fullmatch(r'([0-9x]+)(?:_?n"?([^"]*)"?)?', desc)
    if m is None:
        raise Skip("descriptor " + desc)
    dims = tuple(int(x) for x in m.group(1).split("x"))
    nd = len(dims)
    if 0 in dims or nd > 6:
        raise Skip("descriptor " + desc)
    r = np.random.Generator(np.random.PCG64(zlib.crc32(("--reorder %s %s" % (sorted(settings.items(), key=str), desc)).encode())))
    s_order, d_order = tag_order(settings["stag"], nd), tag_order(settings["dtag"], nd)
    four = (W.S4, W.U4)
    if sdt in four:  # two elements a byte along the innermost dim
        if s_order != tuple(range(nd)) or dims[-1] % 2:
            raise Skip("4-bit src that is not row-major with an even innermost dim")
        src = W.QTensor(W.pack_int4(_values(r, sdt, dims)).reshape(-1), sdt, dims)
    else:
        logical = W.to_storage(_values(r, sdt, dims), sdt)
        src = W.QTensor(np.ascontiguousarray(logical.transpose(s_order)).reshape(-1), sdt, dims, _strides(dims, s_order))
    if ddt in four and dims[d_order[-1]] % 2:
        raise Skip("4-bit dst with an odd innermost dim")
    quant = {}
    for text, suffix, default_dt in ((settings["attr-scales"], "_scale", W.F32), (settings["attr-zero-points"], "_zp", W.S32)):
        for arg, policy, value, dt, groups in B._quant_entries(text):
            if arg not in ("src", "dst"):
                raise Skip("argument " + arg)
            mask = B._policy_mask(policy, nd, False)
            if mask >= (1 << nd):
                raise Skip("policy %s for %d dims" % (policy, nd))
            dt = default_dt if dt is None else dt
            if dt in four and mask == 0:
                raise Skip("a single 4-bit parameter")
            if nd < 2 and groups != (1, 1):
                raise Skip("groups of a 1D tensor")
            shp = [d if (mask >> i) & 1 else 1 for i, d in enumerate(dims)]
            for i, g in zip((-2, -1), groups):
                if g > 1:
                    if not (mask >> (nd + i)) & 1 or dims[i] % g:
                        raise Skip("groups that do not divide the tensor")
                    shp[i] = dims[i] // g
            if suffix == "_scale":
                vals = np.full(shp, 1.0 if value is None else value, np.float32) if mask == 0 \
                    else np.exp2(r.integers(-2, 3, shp)).astype(np.float32)
            elif mask == 0:
                vals = np.full(shp, 0 if value is None else int(value), np.int64)
            else:
                vals = r.integers(-3, 4, shp)
            if dt in four and shp[-1] % 2:
                raise Skip("4-bit parameters with an odd innermost dim")
            if dt == W.U4 and suffix == "_zp" and mask:
                vals = r.integers(0, 6, shp)
            quant[arg + suffix] = W.Quant(W.to_storage(vals, dt), dt, mask, groups)
    beta = 0.0
    for entry in filter(None, settings["attr-post-ops"].split("+")):
        f = entry.split(":")
        if f[0] != "sum" or len(f) > 2:
            raise Skip("post-op " + entry)
        beta = float(f[1]) if len(f) > 1 and f[1] else 1.0
    ro = W.Reorder(desc, src, ddt, _strides(dims, d_order), quant, beta)
    if beta:
        if ddt in four:
            raise Skip("sum into a 4-bit dst")
        init = W.to_storage(_values(r, ddt, dims), ddt)
        ro.dst_init = np.ascontiguousarray(init.transpose(d_order)).reshape(-1)
    return ro


def primitive_desc(ro, eng):
    """The library's reorder primitive descriptor for a Reorder (raises api.error when refused)."""
    from onednn_b200 import api
    src_md = api.memory.desc(ro.src.dims, ro.src.dt, tuple(ro.src.strides))
    dst_md = api.memory.desc(ro.src.dims, ro.dst_dt, tuple(ro.dst_strides))
    attr = api.primitive_attr()
    for name, q in ro.quant.items():
        arg = api.ARG_SRC if name.startswith("src") else api.ARG_DST
        groups = tuple(q.groups) if tuple(q.groups) != (1, 1) else ()
        (attr.set_scales if name.endswith("scale") else attr.set_zero_points)(arg, q.mask, groups, q.dt)
    if ro.beta:
        po = api.post_ops()
        po.append_sum(ro.beta, 0, 0)
        attr.set_post_ops(po)
    return api.reorder.primitive_desc(eng, src_md, eng, dst_md, attr)
