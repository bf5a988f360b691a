"""Runs matmul problems written in the syntax of oneDNN's benchdnn driver
(tests/benchdnn/doc/driver_matmul.md, knobs_attr.md in oneDNN) through this
library and checks each against the CPU oracle.

Input files hold option lines and problem descriptors:

    --reset
    --dt=u8:s8:s8,s8:s8:f32          # a comma list multiplies the problems
    --stag=ab --wtag=ab,ba --dtag=ab
    --bia-dt=undef,f32 --bia_mask=2
    --attr-scales=src:common:0.25+wei:per_oc+dst:common:4
    --attr-post-ops=sum+relu+add:f32:per_oc
    --batch=shapes_file              # a file beside this one
    10x30:30x20                      # MxK:KxN

Every descriptor line is run once per element of the cartesian product of the
option lists in force, as benchdnn does (tests/benchdnn/utils/parser.hpp).
What this library's matmul path covers is run and compared; a problem outside
it is reported as SKIPPED with the reason (benchdnn's own word for a
descriptor the library answers `unimplemented` to), never silently dropped.

Handled: --reset, --batch, --dt, --stag/--wtag/--dtag (ab, ba, any), --bia-dt,
--bia_mask, --runtime_dims_masks (any of M, K, N of a 2D problem), --attr-scales,
--attr-zero-points, --attr-precomputed-reductions, --attr-post-ops (sum, eltwise,
binary, prelu), --attr-fpmath,
--attr-scratchpad, --strides.  Options that select implementations or engines
(--skip-impl, --impl, --engine, --match ...) are accepted and ignored.
Descriptors with batch dims (3D and more, size-1 dims broadcast, tags that
permute the dims such as acb or bac) run as one batched primitive and are checked
matrix by matrix against the oracle's 2D result.  --grouped=0:G:sizes with a
MxK:GxKxN descriptor is a grouped (MoE) problem.  Depthwise post-ops, run-time dims of batched problems and the remaining attributes
are skipped with their name as the reason.

Policy names follow attr_t::policy2mask (tests/benchdnn/dnn_types.cpp:218-268):
for the matmul's src / weights / dst, `per_oc` and `per_dim_1` are the last
dim, `per_ocic` the last two; binary post-op operands use the default masks.

    python tests/benchdnn_matmul.py [--all-impls] FILE [FILE ...]      # needs a B200
"""
import itertools
import os
import re
import sys
import zlib

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from onednn_b200 import workloads as W  # noqa: E402

DT = {"f16": W.F16, "bf16": W.BF16, "f32": W.F32, "s32": W.S32, "s8": W.S8, "u8": W.U8,
      "f8_e5m2": W.F8_E5M2, "f8_e4m3": W.F8_E4M3, "s4": W.S4, "u4": W.U4}

DEFAULTS = {"dt": "f32", "stag": "abx", "wtag": "abx", "dtag": "abx", "bia-dt": "undef", "bia_mask": "2",
            "runtime_dims_masks": "0", "attr-scales": "", "attr-zero-points": "", "attr-post-ops": "",
            "attr-fpmath": "", "attr-scratchpad": "library", "strides": "", "grouped": "",
            "attr-precomputed-reductions": "", "attr-dropout": "", "attr-acc-mode": "", "encoding": "",
            "attr-rounding-mode": "", "attr-deterministic": ""}
# options about which implementation or engine runs, or how benchdnn reports
IGNORED = {"skip-impl", "impl", "engine", "match", "allow-enum-tags-only", "check-ref-impl", "cpu-isa-hints",
           "mode", "max-ms-per-prb", "fix-times-per-prb", "perf-template", "verbose", "v", "mem-check",
           "cold-cache", "stream-kind", "global-impl", "global-skip-impl", "start", "repeats-per-prb",
           "summary", "bia_dt"}
# named here so that a file using them is reported, not mis-run
UNSUPPORTED = ( "attr-dropout", "attr-acc-mode", "encoding",
               "attr-rounding-mode", "attr-deterministic")

ELTWISE_ALIAS = {"srelu": "soft_relu"}


class Skip(Exception):
    """The problem is outside what the driver or the library covers."""


# ------------------------------------------------------------------- reading
def _logical_lines(path):
    with open(path) as f:
        pending = ""
        for raw in f:
            line = raw.split("#", 1)[0].rstrip()
            if line.endswith("\\"):
                pending += line[:-1].strip()
                continue
            line = (pending + line.strip()) if pending else line.strip()
            pending = ""
            if line:
                yield line
        if pending:
            yield pending


def expand(path, state=None, defaults=None):
    """Yields (settings, descriptor) for every problem of an input file, in
    file order.  `settings` maps option names to ONE value each.  `defaults`:
    the options of the driver the file is written for (this module's, for matmul)."""
    defaults = DEFAULTS if defaults is None else defaults
    if state is None:
        state = {"lists": {k: [v] for k, v in defaults.items()}, "unknown": set()}
    lists = state["lists"]
    here = os.path.dirname(os.path.abspath(path))
    for line in _logical_lines(path):
        for tok in line.split():
            if not tok.startswith("--"):
                keys = list(lists)
                for combo in itertools.product(*(lists[k] for k in keys)):
                    s = dict(zip(keys, combo))
                    s["_unknown"] = sorted(state["unknown"])
                    yield s, tok
                continue
            name, _, val = tok[2:].partition("=")
            if name == "reset":
                lists.update({k: [v] for k, v in defaults.items()})
                state["unknown"].clear()
            elif name == "batch":
                yield from expand(os.path.join(here, val), state, defaults)
            elif name in ("matmul", "reorder") or name in IGNORED:
                continue
            elif name not in defaults:
                state["unknown"].add(name)
            else:
                lists[name] = val.split(",") if val != "" else [defaults[name] if name in ("dt",) else ""]


def command_line(settings, desc):
    """The benchdnn command line of one expanded problem (for the report)."""
    parts = ["--matmul"]
    for k, v in settings.items():
        if not k.startswith("_") and v != DEFAULTS[k]:
            parts.append("--%s=%s" % (k, v))
    return " ".join(parts + [desc])


# ------------------------------------------------------------------ building
def _policy_mask(policy, nd, matmul_arg):
    if policy in ("common", "host_scalar"):
        return 0
    if policy.lstrip("-").isdigit():
        return int(policy)
    if matmul_arg and policy in ("per_oc", "per_dim_1"):
        return 1 << (nd - 1)
    if matmul_arg and policy == "per_ocic":
        return 3 << (nd - 2)
    table = {"per_dim_0": 1, "per_dim_1": 2, "per_oc": 2, "per_dim_01": 3, "per_dim_2": 4, "per_dim_3": 8,
             "per_tensor": (1 << nd) - 1}
    if policy in table and table[policy] >= (1 << nd):
        raise Skip("policy %s for %d dims" % (policy, nd))
    if policy not in table:
        raise Skip("policy " + policy)
    return table[policy]


def _is_number(s):
    try:
        float(s)
        return True
    except ValueError:
        return False


def _quant_entries(text):
    """'src:common:0.25+wei:per_ocic:bf16:2x1' -> [(arg, policy, value, dt, groups)]."""
    out = []
    for entry in filter(None, text.split("+")):
        f = entry.split(":")
        arg, policy = f[0], (f[1] if len(f) > 1 else "common")
        arg = {"src0": "src", "src1": "wei"}.get(arg, arg)
        if arg not in ("src", "wei", "dst"):
            raise Skip("argument " + arg)
        value, dt, groups = None, None, (1, 1)
        for t in f[2:]:
            if t.endswith("*"):
                t = t[:-1]
            if _is_number(t):
                value = float(t)
            elif t in DT:
                dt = DT[t]
            elif re.fullmatch(r"\d+x\d+", t):
                groups = tuple(int(x) for x in t.split("x"))
            elif t:
                raise Skip("quantization field " + t)
        out.append((arg, policy, value, dt, groups))
    return out


def _param_shape(mask, groups, dims):
    shape = [d if (mask >> i) & 1 else 1 for i, d in enumerate(dims)]
    for i, g in zip((-2, -1), groups):
        if g > 1:
            if not (mask >> (len(dims) + i)) & 1 or dims[i] % g:
                raise Skip("groups %dx%d do not divide the tensor" % tuple(groups))
            shape[i] = dims[i] // g
    return tuple(shape)


def _fill(r, dt, shape, role):
    """Small values exact in every data type involved, so that products and
    short sums are exact and implementations differ only by summation order."""
    if dt == W.U8:
        v = r.integers(0, 40 if role == "src" else 8, shape)
    elif dt in (W.S8, W.S32):
        v = r.integers(-20, 21, shape) if role in ("src", "wei") else r.integers(-8, 9, shape)
    elif dt == W.S4:
        v = r.integers(-8, 8, shape)
    elif dt == W.U4:
        v = r.integers(0, 16, shape)
    elif dt in (W.F8_E4M3, W.F8_E5M2):
        v = r.integers(-4, 5, shape).astype(np.float32)
    else:
        v = r.integers(-8, 9, shape).astype(np.float32) * (0.25 if role in ("src", "wei") else 1.0)
    return W.to_storage(v, dt)


def _split_strides(text, nd):
    """'8x1::9x1' -> [(8, 1), None, (9, 1)]: element strides of src, weights and dst (None = by tag)."""
    parts = (text.split(":") + ["", "", ""])[:3] if text else ["", "", ""]
    out = []
    for t in parts:
        if not t:
            out.append(None)
            continue
        st = tuple(int(x) for x in t.split("x"))
        if len(st) != nd or any(v < 0 for v in st):
            raise Skip("strides " + t)
        out.append(st)
    return out


def _scatter(logical, strides):
    """Storage of a logical array laid out with the given element strides (the gaps are zero)."""
    offs = sum(np.arange(n).reshape([-1 if i == d else 1 for i in range(logical.ndim)]) * s
               for d, (n, s) in enumerate(zip(logical.shape, strides)))
    offs = np.broadcast_to(offs, logical.shape).reshape(-1)
    if np.unique(offs).size != offs.size:
        raise Skip("strides under which elements overlap")
    storage = np.zeros(int(offs.max()) + 1 if offs.size else 0, logical.dtype)
    storage[offs] = logical.reshape(-1)
    return storage


def _gather(storage, dims, strides):
    isz = storage.itemsize
    return np.lib.stride_tricks.as_strided(storage, dims, tuple(s * isz for s in strides))


def _tensor(r, dt, dims, tag, role, strides=None):
    if strides is not None:
        if dt in (W.S4, W.U4):
            raise Skip("strides of a 4-bit tensor")
        return W.QTensor(_scatter(_fill(r, dt, dims, role), strides), dt, dims, strides)
    if tag in ("ab", "any", "abx"):
        return W.QTensor(_fill(r, dt, dims, role), dt, dims)
    if tag == "ba":
        if dt in (W.S4, W.U4):
            if dims[0] % 2:
                raise Skip("4-bit tensor with an odd leading dim stored transposed")
            t = _fill(r, dt, (dims[1], dims[0]), role)
        else:
            t = _fill(r, dt, (dims[1], dims[0]), role)
        return W.QTensor(t, dt, dims, (1, dims[0]))
    raise Skip("tag " + tag)


def build(settings, desc, seed=None, max_macs=None):
    """(Problem, run options) of one expanded benchdnn problem, or raises Skip.
    max_macs: problems with more multiply-adds are skipped before any data is made."""
    if settings.get("_unknown"):
        raise Skip("option --" + settings["_unknown"][0])
    for k in UNSUPPORTED:
        if settings[k] not in ("", DEFAULTS[k]):
            raise Skip("--" + k)
    m = re.fullmatch(r'([0-9x:]+)(?:_?n"?([^"]*)"?)?', desc)
    if m is None:
        raise Skip("descriptor " + desc)
    shape, name = m.group(1), m.group(2)
    parts = shape.split(":")
    if len(parts) not in (2, 3):
        raise Skip("descriptor " + desc)
    try:
        sdims = [int(x) for x in parts[0].split("x")]
        wdims = [int(x) for x in parts[1].split("x")]
    except ValueError:
        raise Skip("descriptor " + desc)
    if len(sdims) != 2 or len(wdims) != 2:
        raise Skip("batched descriptor")
    (M, K), (K2, N) = sdims, wdims
    if K != K2:
        raise Skip("descriptor " + desc)
    if 0 in (M, K, N):
        raise Skip("zero dim")
    if max_macs is not None and M * K * N > max_macs:
        raise Skip("larger than the cap")
    r = np.random.Generator(np.random.PCG64(zlib.crc32((command_line(settings, desc)).encode())
                                            if seed is None else seed))

    dts = settings["dt"].split(":")
    if len(dts) == 1:
        dts = dts * 3
    if len(dts) != 3 or any(d not in DT for d in dts):
        raise Skip("data types " + settings["dt"])
    sdt, wdt, ddt = (DT[d] for d in dts)
    if ddt not in (W.F32, W.S32, W.BF16, W.F16, W.S8, W.U8, W.F8_E4M3, W.F8_E5M2):
        raise Skip("dst type " + dts[2])
    if wdt in (W.S4, W.U4) and N % 2 and settings["wtag"] != "ba":
        raise Skip("4-bit weights with odd N")
    s_st, w_st, d_st = _split_strides(settings["strides"], 2)
    if d_st is None and settings["dtag"] not in ("ab", "any", "abx"):
        raise Skip("dst tag " + settings["dtag"])
    if d_st is not None and (d_st[1] != 1 or d_st[0] < N):
        raise Skip("dst strides other than a row pitch")
    src = _tensor(r, sdt, (M, K), settings["stag"], "src", s_st)
    wei = _tensor(r, wdt, (K, N), settings["wtag"], "wei", w_st)

    bias = None
    if settings["bia-dt"] != "undef":
        if settings["bia-dt"] not in DT:
            raise Skip("bias type " + settings["bia-dt"])
        bm = int(settings["bia_mask"])
        if bm < 1 or bm > 3:
            raise Skip("bias mask %d" % bm)
        bdims = (M if bm & 1 else 1, N if bm & 2 else 1)
        bias = W.QTensor(_fill(r, DT[settings["bia-dt"]], bdims, "bias"), DT[settings["bia-dt"]], bdims)

    opts = {"runtime_m": False, "user_scratchpad": settings["attr-scratchpad"] == "user",
            "dst_ld": None if d_st is None else d_st[0]}
    rt = settings["runtime_dims_masks"] or "0"
    rs, _, rw = rt.partition(":")
    rs, rw = int(rs or 0), int(rw or 0)
    if rs > 3 or rw > 3:
        raise Skip("run-time mask of a dim the problem does not have")
    if rs or rw:
        opts["runtime_m"] = True if (rs, rw) == (1, 0) else (rs, rw)

    dims_of = {"src": (M, K), "wei": (K, N), "dst": (M, N)}
    quant = {}
    for arg, policy, value, dt, groups in _quant_entries(settings["attr-scales"]):
        mask = _policy_mask(policy, 2, True)
        dt = W.F32 if dt is None else dt
        shp = _param_shape(mask, groups, dims_of[arg])
        if mask == 0:
            vals = np.full(shp, 1.0 if value is None else value, np.float32)
        else:
            vals = np.exp2(r.integers(-3, 2, shp)).astype(np.float32)
        quant[arg + "_scale"] = W.Quant(W.to_storage(vals, dt), dt, mask, groups)
    for arg, policy, value, dt, groups in _quant_entries(settings["attr-zero-points"]):
        mask = _policy_mask(policy, 2, True)
        dt = W.S32 if dt is None else dt
        shp = _param_shape(mask, groups, dims_of[arg])
        if mask == 0:
            vals = np.full(shp, 0 if value is None else int(value), np.int64)
        else:
            lo, hi = (0, 6) if dt in (W.U8, W.U4) else (-3, 4)
            vals = r.integers(lo, hi, shp)
        quant[arg + "_zp"] = W.Quant(W.to_storage(vals, dt), dt, mask, groups)

    for arg, policy, value, dt, groups in _quant_entries(settings["attr-precomputed-reductions"]):
        # the sums of the src values over each K group, which the library may use in place of
        # adding them up itself when it applies weights zero-points
        mask = _policy_mask(policy, 2, True)
        if arg != "src" or sdt not in (W.S8, W.U8) or mask != 3 or groups[0] != 1 or K % groups[1]:
            raise Skip("precomputed reductions other than src sums per K group")
        logical = _gather(src.data, src.dims, src.strides).astype(np.int64)
        sums = logical.reshape(M, K // groups[1], groups[1]).sum(axis=2)
        dt = W.S32 if dt is None else dt
        quant["src_pr"] = W.Quant(W.to_storage(sums, dt), dt, mask, groups)

    post_ops, dst_init = [], None
    for entry in filter(None, settings["attr-post-ops"].split("+")):
        f = entry.split(":")
        kind = f[0][8:] if f[0].startswith("eltwise_") else f[0][7:] if f[0].startswith("binary_") else f[0]
        kind = ELTWISE_ALIAS.get(kind, kind)
        if kind == "sum":
            scale = float(f[1]) if len(f) > 1 and f[1] else 1.0
            zp = int(f[2]) if len(f) > 2 and f[2] else 0
            if len(f) > 3 and f[3] and DT.get(f[3]) != ddt:
                raise Skip("sum with a data type other than dst's")
            post_ops.append(W.PostOp(W.PO_SUM, scale=scale, zero_point=zp))
            dst_init = _fill(r, ddt, (M, N), "dst")
        elif kind in W.ELTWISE:
            alpha = float(f[1]) if len(f) > 1 and f[1] else 0.0
            beta = float(f[2]) if len(f) > 2 and f[2] else 0.0
            if len(f) > 3 and f[3] and float(f[3]) != 1.0:
                raise Skip("eltwise with a scale")
            post_ops.append(W.PostOp(W.PO_ELTWISE, W.ELTWISE[kind], alpha, beta, 1.0))
        elif kind in W.BINARY:
            if len(f) < 2 or f[1] not in DT:
                raise Skip("binary post-op " + entry)
            if len(f) > 3 and f[3] not in ("", "ab", "any", "abx"):
                raise Skip("binary post-op tag " + f[3])
            mask = _policy_mask(f[2] if len(f) > 2 and f[2] else "common", 2, False)
            bdims = (M if mask & 1 else 1, N if mask & 2 else 1)
            vals = _fill(r, DT[f[1]], bdims, "binary")
            if kind == "div":  # no zero divisors
                z = W.to_f32(vals, DT[f[1]]) == 0
                vals = W.to_storage(np.where(z, 2.0, W.to_f32(vals, DT[f[1]])), DT[f[1]])
            post_ops.append(W.PostOp(W.PO_BINARY, W.BINARY[kind], src1=W.QTensor(vals, DT[f[1]], bdims)))
        elif kind == "prelu":  # f32 weights over the dst dims the policy names
            mask = _policy_mask(f[1] if len(f) > 1 and f[1] else "common", 2, False)
            wdims = (M if mask & 1 else 1, N if mask & 2 else 1)
            post_ops.append(W.PostOp(W.PO_PRELU, src1=W.QTensor(_fill(r, W.F32, wdims, "src"), W.F32, wdims)))
        else:
            raise Skip("post-op " + f[0])

    fpmath, apply_to_int = 0, False
    if settings["attr-fpmath"]:
        mode, _, flag = settings["attr-fpmath"].partition(":")
        modes = {"strict": 0, "bf16": 1, "f16": 2, "any": 3, "tf32": 4}
        if mode not in modes:
            raise Skip("fpmath " + mode)
        fpmath, apply_to_int = modes[mode], flag == "true"

    p = W.Problem(name or desc, M, N, K, src, wei, ddt, bias, quant, post_ops, apply_to_int, fpmath)
    p.dst_init = dst_init
    if s_st is not None or w_st is not None:  # the same problem with dense tensors, for the allowance formulas
        dense = [W.QTensor(np.ascontiguousarray(_gather(t.data, t.dims, t.strides)), t.dt, t.dims) for t in (src, wei)]
        opts["dense"] = W.Problem(p.name, M, N, K, dense[0], dense[1], ddt, bias, quant, post_ops, apply_to_int, fpmath)
        opts["dense"].dst_init = dst_init
    return p, opts


# ------------------------------------------------------------------- grouped
def build_grouped(settings, desc, max_macs=None):
    """Problem of a grouped (MoE) descriptor `--grouped=0:G:s0+s1+... MxK:GxKxN`: the rows of src
    and dst are split into G groups of the given sizes, group g multiplying weights [g].  Masks are
    written as numbers in these inputs: src 1 = per row, 3 with groups 1xg = per row and K group;
    weights 5 = per (expert, column), 7 with groups gx1 = per (expert, K group, column)."""
    if settings.get("_unknown"):
        raise Skip("option --" + settings["_unknown"][0])
    for k in UNSUPPORTED:
        if settings[k] not in ("", DEFAULTS[k]):
            raise Skip("--" + k)
    g = settings["grouped"].split(":")
    if len(g) < 3 or g[0] != "0":
        raise Skip("grouping of a dim other than M")
    G, sizes = int(g[1]), [int(x) for x in g[2].split("+")]
    m = re.fullmatch(r'([0-9x:]+)(?:_?n"?([^"]*)"?)?', desc)
    parts = m.group(1).split(":") if m else []
    if len(parts) != 2:
        raise Skip("descriptor " + desc)
    sdims = tuple(int(x) for x in parts[0].split("x"))
    wdims = tuple(int(x) for x in parts[1].split("x"))
    if len(sdims) != 2 or len(wdims) != 3 or wdims[0] != G or len(sizes) != G or sum(sizes) != sdims[0] \
            or sdims[1] != wdims[1]:
        raise Skip("descriptor " + desc)
    (M, K), N = sdims, wdims[2]
    if max_macs is not None and M * K * N > max_macs:
        raise Skip("larger than the cap")
    if settings["strides"] or (settings["runtime_dims_masks"] or "0") not in ("0", "0:0"):
        raise Skip("strides / run-time dims of a grouped problem")
    r = np.random.Generator(np.random.PCG64(zlib.crc32(command_line(settings, desc).encode())))
    dts = settings["dt"].split(":")
    dts = dts * 3 if len(dts) == 1 else dts
    if len(dts) != 3 or any(d not in DT for d in dts):
        raise Skip("data types " + settings["dt"])
    sdt, wdt, ddt = (DT[d] for d in dts)
    if ddt not in (W.F32, W.BF16, W.F16, W.S8, W.U8, W.S32) or sdt in (W.S4, W.U4):
        raise Skip("data types " + settings["dt"])
    if settings["stag"] not in ("ab", "abx", "any") or settings["dtag"] not in ("ab", "abx", "any"):
        raise Skip("tags of src / dst of a grouped problem")
    src = W.QTensor(_fill(r, sdt, (M, K), "src"), sdt, (M, K))
    if settings["wtag"] in ("abc", "abx", "any"):
        if wdt in (W.S4, W.U4) and N % 2:
            raise Skip("4-bit weights with odd N")
        wei = W.QTensor(_fill(r, wdt, (G, K, N), "wei"), wdt, (G, K, N))
    elif settings["wtag"] == "acb":
        if wdt in (W.S4, W.U4) and K % 2:
            raise Skip("4-bit weights with odd K stored transposed")
        wei = W.QTensor(_fill(r, wdt, (G, N, K), "wei"), wdt, (G, K, N), (K * N, 1, K))
    else:
        raise Skip("tag " + settings["wtag"])
    bias = None
    if settings["bia-dt"] != "undef":
        if settings["bia-dt"] not in DT or settings["bia_mask"] != "2":
            raise Skip("bias of a grouped problem other than [G, N]")
        bias = W.QTensor(_fill(r, DT[settings["bia-dt"]], (G, N), "bias"), DT[settings["bia-dt"]], (G, N))
    quant = {}
    for text, suffix, default_dt in ((settings["attr-scales"], "_scale", W.F32), (settings["attr-zero-points"], "_zp", W.S32)):
        for arg, policy, value, dt, groups in _quant_entries(text):
            if not policy.isdigit():
                raise Skip("policy %s of a grouped problem" % policy)
            mask, dt = int(policy), default_dt if dt is None else dt
            if arg == "src" and mask in (1, 3) and groups[0] == 1 and K % groups[1] == 0 and (mask == 3) == (groups[1] > 1):
                shp = (M, K // groups[1] if mask == 3 else 1)
            elif arg == "wei" and mask in (5, 7) and groups[1] == 1 and K % groups[0] == 0 and (mask == 7) == (groups[0] > 1):
                shp = (G, K // groups[0] if mask == 7 else 1, N)
            elif mask == 0:
                shp = (1,) * (3 if arg == "wei" else 2)
            else:
                raise Skip("mask %d on %s of a grouped problem" % (mask, arg))
            if suffix == "_scale":
                vals = np.full(shp, 1.0 if value is None else value, np.float32) if mask == 0 \
                    else np.exp2(r.integers(-3, 2, shp)).astype(np.float32)
            elif mask == 0:
                vals = np.full(shp, 0 if value is None else int(value), np.int64)
            else:
                vals = r.integers(*((0, 6) if dt in (W.U8, W.U4) else (-3, 4)), shp)
            quant[arg + suffix] = W.Quant(W.to_storage(vals, dt), dt, mask, groups)
    post_ops = []
    for entry in filter(None, settings["attr-post-ops"].split("+")):
        f = entry.split(":")
        kind = f[0][8:] if f[0].startswith("eltwise_") else f[0][7:] if f[0].startswith("binary_") else f[0]
        kind = ELTWISE_ALIAS.get(kind, kind)
        if kind in W.ELTWISE:
            if len(f) > 3 and f[3] and float(f[3]) != 1.0:
                raise Skip("eltwise with a scale")
            post_ops.append(W.PostOp(W.PO_ELTWISE, W.ELTWISE[kind], float(f[1]) if len(f) > 1 and f[1] else 0.0,
                                     float(f[2]) if len(f) > 2 and f[2] else 0.0, 1.0))
        elif kind in W.BINARY and len(f) >= 3 and f[1] in DT and f[2] == "1" and len(f) == 3:
            post_ops.append(W.PostOp(W.PO_BINARY, W.BINARY[kind], src1=W.QTensor(_fill(r, DT[f[1]], (M, 1), "binary"), DT[f[1]], (M, 1))))
        else:
            raise Skip("post-op %s of a grouped problem" % entry)
    fpmath, apply_to_int = 0, False
    if settings["attr-fpmath"]:
        mode, _, flag = settings["attr-fpmath"].partition(":")
        modes = {"strict": 0, "bf16": 1, "f16": 2, "any": 3, "tf32": 4}
        if mode not in modes:
            raise Skip("fpmath " + mode)
        fpmath, apply_to_int = modes[mode], flag == "true"
    return W.Problem(desc, M, N, K, src, wei, ddt, bias, quant, post_ops, apply_to_int, fpmath,
                     offsets=np.cumsum(sizes).astype(np.int32))


# ------------------------------------------------------------------- batched
class Batched:
    """A descriptor with batch dims: the tensors as the library gets them (storage
    arrays with dims and strides) and, for the oracle, one 2D Problem per matrix
    of the dst batch (size-1 batch dims of src / weights / bias / binary operands
    broadcast, src/common/matmul.cpp:630-744)."""

    def __init__(self):
        self.mats = []  # (batch index tuple, W.Problem)
        self.tensors = {}  # name -> (storage, dt, dims, strides)
        self.quant = {}  # name -> (W.Quant with the nd mask)
        self.post_ops = []  # W.PostOp; binary src1 dims are nd
        self.fpmath, self.apply_to_int = 0, False
        self.user_scratchpad = False


def _tag_order(tag, nd):
    """Physical order of the dims, outermost first: 'acb' -> (0, 2, 1)."""
    if tag in ("any", "abx"):
        return tuple(range(nd))
    if len(tag) != nd or sorted(tag) != [chr(ord("a") + i) for i in range(nd)]:
        raise Skip("tag %s for %d dims" % (tag, nd))
    return tuple(ord(c) - ord("a") for c in tag)


def _layout(logical, order):
    """(storage, strides in elements) of a logical array stored in `order`."""
    phys = np.ascontiguousarray(logical.transpose(order))
    strides = [0] * logical.ndim
    acc = 1
    for d in reversed(order):
        strides[d] = acc
        acc *= logical.shape[d]
    return phys.reshape(-1), tuple(strides)


def build_batched(settings, desc):
    """Batched of one expanded problem whose descriptor has batch dims, or raises Skip."""
    if settings.get("_unknown"):
        raise Skip("option --" + settings["_unknown"][0])
    for k in UNSUPPORTED:
        if settings[k] not in ("", DEFAULTS[k]):
            raise Skip("--" + k)
    m = re.fullmatch(r'([0-9x:]+)(?:_?n"?([^"]*)"?)?', desc)
    parts = m.group(1).split(":") if m else []
    if len(parts) not in (2, 3):
        raise Skip("descriptor " + desc)
    sdims = tuple(int(x) for x in parts[0].split("x"))
    wdims = tuple(int(x) for x in parts[1].split("x"))
    nd = len(sdims)
    if nd < 3 or len(wdims) != nd or nd > 6 or sdims[-1] != wdims[-2]:
        raise Skip("descriptor " + desc)
    nb = nd - 2
    for a, b in zip(sdims[:nb], wdims[:nb]):
        if a != b and 1 not in (a, b):
            raise Skip("descriptor " + desc)
    bdims = tuple(max(a, b) for a, b in zip(sdims[:nb], wdims[:nb]))
    M, K, N = sdims[-2], sdims[-1], wdims[-1]
    ddims = bdims + (M, N)
    if 0 in ddims or K == 0:
        raise Skip("zero dim")
    if (settings["runtime_dims_masks"] or "0") not in ("0", "0:0"):
        raise Skip("run-time dims of a batched problem")
    r = np.random.Generator(np.random.PCG64(zlib.crc32(command_line(settings, desc).encode())))
    dts = settings["dt"].split(":")
    dts = dts * 3 if len(dts) == 1 else dts
    if len(dts) != 3 or any(d not in DT for d in dts):
        raise Skip("data types " + settings["dt"])
    sdt, wdt, ddt = (DT[d] for d in dts)
    if W.S4 in (sdt, wdt, ddt) or W.U4 in (sdt, wdt, ddt):
        raise Skip("4-bit types in a batched problem")
    if ddt not in (W.F32, W.S32, W.BF16, W.F16, W.S8, W.U8, W.F8_E4M3, W.F8_E5M2):
        raise Skip("dst type " + dts[2])
    bp = Batched()
    bp.ddt, bp.ddims = ddt, ddims
    bp.user_scratchpad = settings["attr-scratchpad"] == "user"
    src_l = _fill(r, sdt, sdims, "src")
    wei_l = _fill(r, wdt, wdims, "wei")
    s_st, w_st, d_st = _split_strides(settings["strides"], nd)
    bp.tensors["src"] = (_scatter(src_l, s_st), s_st, sdt, sdims) if s_st is not None \
        else (*_layout(src_l, _tag_order(settings["stag"], nd)), sdt, sdims)
    bp.tensors["wei"] = (_scatter(wei_l, w_st), w_st, wdt, wdims) if w_st is not None \
        else (*_layout(wei_l, _tag_order(settings["wtag"], nd)), wdt, wdims)
    bp.dst_strides = d_st if d_st is not None else _layout(np.empty(ddims, np.uint8), _tag_order(settings["dtag"], nd))[1]
    bias_l = None
    if settings["bia-dt"] != "undef":
        if settings["bia-dt"] not in DT:
            raise Skip("bias type " + settings["bia-dt"])
        bm = int(settings["bia_mask"])
        if bm < 1 or bm >= (1 << nd):
            raise Skip("bias mask %d" % bm)
        bia_dims = tuple(d if (bm >> i) & 1 else 1 for i, d in enumerate(ddims))
        bias_l = _fill(r, DT[settings["bia-dt"]], bia_dims, "bias")
        bp.tensors["bias"] = (*_layout(bias_l, tuple(range(nd))), DT[settings["bia-dt"]], bia_dims)

    dims_of = {"src": (M, K), "wei": (K, N), "dst": (M, N)}
    quant2d = {}
    for text, suffix, default_dt in ((settings["attr-scales"], "_scale", W.F32), (settings["attr-zero-points"], "_zp", W.S32)):
        for arg, policy, value, dt, groups in _quant_entries(text):
            mask = _policy_mask(policy, nd, True)
            if mask & ((1 << nb) - 1):
                raise Skip("a quantization parameter that varies along the batch")
            dt = default_dt if dt is None else dt
            shp = _param_shape(mask >> nb, groups, dims_of[arg])
            if suffix == "_scale":
                vals = np.full(shp, 1.0 if value is None else value, np.float32) if mask == 0 \
                    else np.exp2(r.integers(-3, 2, shp)).astype(np.float32)
            elif mask == 0:
                vals = np.full(shp, 0 if value is None else int(value), np.int64)
            else:
                vals = r.integers(*((0, 6) if dt in (W.U8, W.U4) else (-3, 4)), shp)
            data = W.to_storage(vals, dt)
            quant2d[arg + suffix] = W.Quant(data, dt, mask >> nb, groups)
            bp.quant[arg + suffix] = W.Quant(data, dt, mask, groups)

    dst_init_l = None
    binaries = {}
    for i, entry in enumerate(filter(None, settings["attr-post-ops"].split("+"))):
        f = entry.split(":")
        kind = f[0][8:] if f[0].startswith("eltwise_") else f[0][7:] if f[0].startswith("binary_") else f[0]
        kind = ELTWISE_ALIAS.get(kind, kind)
        if kind == "sum":
            if len(f) > 3 and f[3] and DT.get(f[3]) != ddt:
                raise Skip("sum with a data type other than dst's")
            bp.post_ops.append(W.PostOp(W.PO_SUM, scale=float(f[1]) if len(f) > 1 and f[1] else 1.0,
                                        zero_point=int(f[2]) if len(f) > 2 and f[2] else 0))
            dst_init_l = _fill(r, ddt, ddims, "dst")
        elif kind in W.ELTWISE:
            if len(f) > 3 and f[3] and float(f[3]) != 1.0:
                raise Skip("eltwise with a scale")
            bp.post_ops.append(W.PostOp(W.PO_ELTWISE, W.ELTWISE[kind], float(f[1]) if len(f) > 1 and f[1] else 0.0,
                                        float(f[2]) if len(f) > 2 and f[2] else 0.0, 1.0))
        elif kind in W.BINARY:
            if len(f) < 2 or f[1] not in DT or (len(f) > 3 and f[3] and _tag_order(f[3], nd) != tuple(range(nd))):
                raise Skip("binary post-op " + entry)
            mask = _policy_mask(f[2] if len(f) > 2 and f[2] else "common", nd, False)
            odims = tuple(d if (mask >> j) & 1 else 1 for j, d in enumerate(ddims))
            vals = _fill(r, DT[f[1]], odims, "binary")
            if kind == "div":
                v = W.to_f32(vals, DT[f[1]])
                vals = W.to_storage(np.where(v == 0, 2.0, v), DT[f[1]])
            binaries[i] = vals
            bp.post_ops.append(W.PostOp(W.PO_BINARY, W.BINARY[kind], src1=W.QTensor(vals.reshape(-1), DT[f[1]], odims)))
        elif kind == "prelu":
            # weights are dense with dim 1 innermost (acb, acdb ...: src/cpu/primitive_attr_postops.cpp:219-242)
            mask = _policy_mask(f[1] if len(f) > 1 and f[1] else "common", nd, False)
            odims = tuple(d if (mask >> j) & 1 else 1 for j, d in enumerate(ddims))
            vals = _fill(r, W.F32, odims, "src")
            binaries[i] = vals
            storage, strides = _layout(vals, (0,) + tuple(range(2, nd)) + (1,))
            bp.post_ops.append(W.PostOp(W.PO_PRELU, zero_point=mask, src1=W.QTensor(storage, W.F32, odims, strides)))
        else:
            raise Skip("post-op " + f[0])
    if settings["attr-fpmath"]:
        mode, _, flag = settings["attr-fpmath"].partition(":")
        modes = {"strict": 0, "bf16": 1, "f16": 2, "any": 3, "tf32": 4}
        if mode not in modes:
            raise Skip("fpmath " + mode)
        bp.fpmath, bp.apply_to_int = modes[mode], flag == "true"
    bp.dst_init = None if dst_init_l is None else _scatter(dst_init_l, bp.dst_strides)

    def pick(arr, idx):  # the matrix of `arr` that batch index idx sees (size-1 dims broadcast)
        return arr[tuple(i if arr.shape[d] > 1 else 0 for d, i in enumerate(idx))]

    for idx in np.ndindex(*bdims):
        s2, w2 = np.ascontiguousarray(pick(src_l, idx)), np.ascontiguousarray(pick(wei_l, idx))
        bias2 = None
        if bias_l is not None:
            b2 = np.ascontiguousarray(pick(bias_l, idx))
            bias2 = W.QTensor(b2, DT[settings["bia-dt"]], b2.shape)
        pos = []
        for i, po in enumerate(bp.post_ops):
            if po.kind in (W.PO_BINARY, W.PO_PRELU):
                o2 = np.ascontiguousarray(pick(binaries[i], idx))
                pos.append(W.PostOp(po.kind, po.alg, src1=W.QTensor(o2, po.src1.dt, o2.shape)))
            else:
                pos.append(po)
        p = W.Problem("%s%s" % (desc, list(idx)), M, N, K, W.QTensor(s2, sdt, (M, K)), W.QTensor(w2, wdt, (K, N)), ddt,
                      bias2, quant2d, pos, bp.apply_to_int, bp.fpmath)
        if dst_init_l is not None:
            p.dst_init = np.ascontiguousarray(dst_init_l[idx])
        bp.mats.append((idx, p))
    return bp


def run_batched(bp, eng, strm, impl=None):
    """Creates the batched primitive (optionally walking to the named implementation),
    executes it once and returns (dst as a logical array, implementation, primitive desc)."""
    from onednn_b200 import api
    md = {k: api.memory.desc(dims, dt, strides) for k, (_, strides, dt, dims) in bp.tensors.items()}
    nd = len(bp.ddims)
    dst_md = api.memory.desc(bp.ddims, bp.ddt, tuple(bp.dst_strides))
    attr = api.primitive_attr()
    if bp.apply_to_int or bp.fpmath:
        attr.set_fpmath_mode(bp.fpmath, bp.apply_to_int)
    arg_of = {"src": api.ARG_SRC, "wei": api.ARG_WEIGHTS, "dst": api.ARG_DST}
    qkeys = {}
    for name, q in bp.quant.items():
        groups = tuple(q.groups) if tuple(q.groups) != (1, 1) else ()
        if name.endswith("scale"):
            attr.set_scales(arg_of[name[:3]], q.mask, groups, q.dt)
            qkeys[name] = api.ARG_ATTR_SCALES | arg_of[name[:3]]
        else:
            attr.set_zero_points(arg_of[name[:3]], q.mask, groups, q.dt)
            qkeys[name] = api.ARG_ATTR_ZERO_POINTS | arg_of[name[:3]]
    po = api.post_ops()
    bin_md = {}
    for i, e in enumerate(bp.post_ops):
        if e.kind == W.PO_SUM:
            po.append_sum(e.scale, e.zero_point, 0)
        elif e.kind == W.PO_ELTWISE:
            po.append_eltwise(e.alg, e.alpha, e.beta)
        elif e.kind == W.PO_PRELU:
            bin_md[i] = api.memory.desc(e.src1.dims, e.src1.dt, tuple(e.src1.strides))
            po.append_prelu(e.zero_point)  # the mask
        else:
            bin_md[i] = api.memory.desc(e.src1.dims, e.src1.dt, tuple(e.src1.strides))
            po.append_binary(e.alg, bin_md[i])
    if bp.post_ops:
        attr.set_post_ops(po)
    if bp.user_scratchpad:
        attr.set_scratchpad_mode(api.SCRATCHPAD_MODE_USER)
    pd = api.matmul.primitive_desc(eng, md["src"], md["wei"], dst_md, md.get("bias"), attr)
    if impl is not None:
        while impl not in pd.impl_info_str():
            if not pd.next_impl():
                raise api.error(api.unimplemented, "no implementation named *%s*" % impl)
    if eng is None or strm is None:
        return None, pd.impl_info_str(), pd
    prim = api.matmul(pd)

    def mem(d, array):
        m = api.memory(d, eng)
        m.write(np.ascontiguousarray(array).view(np.uint8).reshape(-1), 0)
        return m

    args = {api.ARG_SRC: mem(md["src"], bp.tensors["src"][0]), api.ARG_WEIGHTS: mem(md["wei"], bp.tensors["wei"][0]),
            api.ARG_DST: mem(dst_md, bp.dst_init if bp.dst_init is not None else np.zeros(dst_md.get_size(0), np.uint8))}
    if "bias" in md:
        args[api.ARG_BIAS] = mem(md["bias"], bp.tensors["bias"][0])
    for name, key in qkeys.items():
        args[key] = mem(pd.query_md(api.QUERY_EXEC_ARG_MD, key), bp.quant[name].data)
    for i, d in bin_md.items():
        which = api.ARG_WEIGHTS if bp.post_ops[i].kind == W.PO_PRELU else api.ARG_SRC_1
        args[api.ARG_ATTR_MULTIPLE_POST_OP(i) | which] = mem(d, bp.post_ops[i].src1.data)
    if bp.user_scratchpad:
        smd = pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_SCRATCHPAD)
        if smd.get_size(0):
            args[api.ARG_SCRATCHPAD] = mem(smd, np.full(smd.get_size(0), 0xA5, np.uint8))
    prim.execute(strm, args)
    strm.wait()
    raw = args[api.ARG_DST].read(np.uint8, 0).view(W.NP_STORAGE[bp.ddt])
    return _gather(raw, bp.ddims, bp.dst_strides), pd.impl_info_str(), pd


# ------------------------------------------------------------------ checking
# eltwise algorithms of the form x * (1 + f(x)) / 2: for negative x the sum 1 + f(x) cancels
CANCELLING = {W.ELTWISE["gelu_erf"]: 1.0, W.ELTWISE["gelu_tanh"]: 1.0}


def cancellation_slack(p):
    """Absolute allowance for a chain holding gelu_erf / gelu_tanh, or None.

    0.5 x (1 + f(x)) is evaluated in f32 by the reference and by the device
    alike, but erff / tanhf of two math libraries differ by a few units in the
    last place of f(x) ~ -1, and the sum 1 + f(x) turns that into an error of
    those few units of 2^-24 times |x| / 2 however small the result is
    (benchdnn's own eltwise check judges these algorithms by absolute error for
    the same reason, tests/benchdnn/eltwise/eltwise.cpp).  The allowance is four
    units: 4 * 2^-24 * |x|, carried through the factors the rest of the chain
    multiplies by.  x comes from the oracle run on the chain cut before f."""
    from oracle import oracle as O
    idx = next((i for i, po in enumerate(p.post_ops) if po.kind == W.PO_ELTWISE and po.alg in CANCELLING), None)
    if idx is None:
        return None
    quant = {k: v for k, v in p.quant.items() if k not in ("dst_scale", "dst_zp")}
    q = W.Problem(p.name + "/pre", p.M, p.N, p.K, p.src, p.wei, W.F32, p.bias, quant, p.post_ops[:idx],
                  p.apply_to_int, p.fpmath, offsets=p.offsets)
    if p.dst_init is not None:
        init = p.dst_init if p.dst_dt in (W.S4, W.U4) else p.dst_init.reshape(p.M, p.N)
        q.dst_init = np.ascontiguousarray(W.to_f32(init, p.dst_dt), dtype=np.float32)
    x = np.abs(O.run_port(q).astype(np.float64))
    amp = np.ones((p.M, p.N))
    for po in p.post_ops[idx + 1:]:
        if po.kind == W.PO_BINARY and po.alg in (W.BINARY["mul"], W.BINARY["div"]):
            v = np.abs(W.to_f32(po.src1.data, po.src1.dt).astype(np.float64)).reshape(po.src1.dims)
            amp = amp * v if po.alg == W.BINARY["mul"] else amp / v
        elif po.kind == W.PO_ELTWISE and po.alg == W.ELTWISE["linear"]:
            amp = amp * abs(po.alpha)
        elif po.kind == W.PO_PRELU:
            amp = amp * np.maximum(1.0, np.abs(po.src1.data.astype(np.float64)).reshape(po.src1.dims))
    ds = p.quant.get("dst_scale")
    if ds is not None:
        amp = amp / np.abs(W.to_f32(ds.data, ds.dt).astype(np.float64)).reshape(-1)[0]
    return 4.0 * 2.0 ** -24 * x * amp


# ------------------------------------------------------------------- running
def run_one(settings, desc, eng, strm, all_impls=False):
    """('PASSED' | 'SKIPPED' | 'FAILED', detail).  With all_impls, every
    implementation that accepts the problem is run, not only the first."""
    from onednn_b200 import api
    from onednn_b200.runner import Prepared
    from oracle import oracle as O
    from oracle.parity import compare, summation_slack, summation_slack_grouped
    try:
        if settings["grouped"]:
            p, opts = build_grouped(settings, desc), {"user_scratchpad": False, "runtime_m": False, "dst_ld": None}
        else:
            p, opts = build(settings, desc)
    except Skip as e:
        if str(e) == "batched descriptor":
            return _run_one_batched(settings, desc, eng, strm, all_impls)
        return "SKIPPED", str(e)
    try:
        first = Prepared(p, eng, None, opts["user_scratchpad"], opts["runtime_m"], opts["dst_ld"])
    except api.error as e:
        if e.status == api.unimplemented:
            return "SKIPPED", "unimplemented"
        return "FAILED", "create: %s" % e
    want = O.run_port(p)
    dense = opts.get("dense", p)
    libm_slack = cancellation_slack(dense)
    ld = opts["dst_ld"]
    p_lib = p
    if ld is not None and p.dst_init is not None:  # the old dst values at the row pitch the library is given
        import copy
        p_lib = copy.copy(p)
        p_lib.dst_init = _scatter(p.dst_init.reshape(p.M, p.N), (ld, 1))
    impls = [first.impl]
    if all_impls:
        while first.pd.next_impl():
            impls.append(first.pd.impl_info_str())
    for impl in impls:
        run = Prepared(p_lib, eng, impl, opts["user_scratchpad"], opts["runtime_m"], ld).upload()
        run.execute(strm)
        strm.wait()
        slack = libm_slack
        if not impl.startswith("cuda:ref") and p.src.dt not in (W.S8, W.U8):
            base = summation_slack_grouped(p) if p.offsets is not None else summation_slack(dense)
            slack = base + (0.0 if libm_slack is None else libm_slack)
        if ld is None:
            got = run.download()
        else:
            raw = run.args[api.ARG_DST].read(np.uint8, 0).view(W.NP_STORAGE[p.dst_dt])
            got = np.ascontiguousarray(_gather(raw, (p.M, p.N), (ld, 1)))
        ok, why = compare(got, want, p.dst_dt, slack)
        if not ok:
            return "FAILED", "%s: %s" % (impl, why)
    return "PASSED", ",".join(impls)


def _run_one_batched(settings, desc, eng, strm, all_impls):
    from onednn_b200 import api
    from oracle import oracle as O
    from oracle.parity import compare, summation_slack, summation_slack_grouped
    try:
        bp = build_batched(settings, desc)
    except Skip as e:
        return "SKIPPED", str(e)
    try:
        _, first, pd = run_batched(bp, eng, None)
    except api.error as e:
        if e.status == api.unimplemented:
            return "SKIPPED", "unimplemented"
        return "FAILED", "create: %s" % e
    impls = [first]
    if all_impls:
        while pd.next_impl():
            impls.append(pd.impl_info_str())
    wants = [(idx, p, O.run_port(p), cancellation_slack(p)) for idx, p in bp.mats]
    for impl in impls:
        got, _, _ = run_batched(bp, eng, strm, impl)
        for idx, p, want, libm_slack in wants:
            slack = libm_slack
            if not impl.startswith("cuda:ref") and p.src.dt not in (W.S8, W.U8):
                slack = summation_slack(p) + (0.0 if libm_slack is None else libm_slack)
            ok, why = compare(np.ascontiguousarray(got[idx]), want, p.dst_dt, slack)
            if not ok:
                return "FAILED", "%s, matrix %s: %s" % (impl, list(idx), why)
    return "PASSED", ",".join(impls)


def run_file(path, eng, strm, all_impls=False, out=None, limit=None):
    """Runs every problem of an input file.  Returns a dict: the counts by
    status, the skip reasons, the implementations that passed (with counts)
    and the failures.  `out` receives one benchdnn-style line a problem."""
    rep = {"PASSED": 0, "SKIPPED": 0, "FAILED": 0, "reasons": {}, "impls": {}, "failures": []}
    for i, (settings, desc) in enumerate(expand(path)):
        if limit is not None and i >= limit:
            break
        status, detail = run_one(settings, desc, eng, strm, all_impls)
        rep[status] += 1
        line = command_line(settings, desc)
        if status == "SKIPPED":
            rep["reasons"][detail] = rep["reasons"].get(detail, 0) + 1
        elif status == "PASSED":
            for impl in detail.split(","):
                rep["impls"][impl] = rep["impls"].get(impl, 0) + 1
        else:
            rep["failures"].append((line, detail))
        if out is not None:
            out.write("%d:%s (%s) __REPRO: %s\n" % (i, status, detail, line))
    return rep


def main(argv):
    from onednn_b200 import api
    all_impls = "--all-impls" in argv
    files = [a for a in argv if not a.startswith("--")]
    if not files:
        print(__doc__)
        return 2
    eng = api.engine(api.engine.kind.gpu, 0)
    strm = api.stream(eng)
    total = {"PASSED": 0, "SKIPPED": 0, "FAILED": 0}
    for path in files:
        rep = run_file(path, eng, strm, all_impls, sys.stdout)
        for k in total:
            total[k] += rep[k]
        for why, n in sorted(rep["reasons"].items(), key=lambda kv: -kv[1]):
            print("  skipped %5d: %s" % (n, why))
        for impl, n in sorted(rep["impls"].items(), key=lambda kv: -kv[1]):
            print("  passed  %5d: %s" % (n, impl))
    print("tests:%d passed:%d skipped:%d failed:%d" % (sum(total.values()), total["PASSED"], total["SKIPPED"],
                                                        total["FAILED"]))
    return 1 if total["FAILED"] else 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
