"""Comparison rules of the parity checks -- TEST INFRASTRUCTURE (the checker), like the rest of
this package: used by the tests, by the smoke check and by the benchmark's parity leg, never by
the product.

* s32 and every integer/byte/index result: bit-exact.
* f32: |got - want| <= 1e-5 * |want|.
* bf16 / f16 / f8_e4m3 / f8_e5m2: at most 1 ulp of the output type from the reference value.
* s8 / u8 (a requantized f32): at most 1 apart.

Kernels that add the K products in another order than the scalar reference
(tensor-core and split-K kernels with f32 accumulators) get, on top of the
above, the summation slack of an f32 dot product: 4 * 2^-24 * sum_k |s_k w_k|
(times the scales), i.e. four units of f32 roundoff on the sum of magnitudes.
It only matters where the reference value itself is cancellation noise (a
result many orders below the magnitude of its terms); the rigorous bound for
ANY summation order, K * 2^-24 * sum|terms| (Higham, Accuracy and Stability of
Numerical Algorithms, ch. 4), is K/4 times larger.  Integer-accumulated paths
never get slack.

`check_rows` applies these rules to a subset of dst rows and, for floating-point results, also
counts the elements beyond the STRICT rule (1 ulp / 1e-5, no slack) and judges each of them
against an fp64 evaluation of the same row.  Such an element is explained when the checked value
is no farther from the fp64 result than the reference is, plus one unit of the output type ("the
reference's own rounding"), or when it lies within one unit plus the summation slack of the fp64
result itself (a result of cancellation, where the unit of the output type is smaller than the
f32 roundoff of any summation order, the reference's included).  Anything else is a kernel error.
"""
import numpy as np

from onednn_b200 import workloads as W


def _ordered(bits: np.ndarray) -> np.ndarray:
    """Maps sign-magnitude 16-bit float patterns to monotone integers."""
    b = bits.astype(np.int32)
    return np.where(b & 0x8000, -(b & 0x7FFF), b)


def _ordered8(bits: np.ndarray) -> np.ndarray:
    """Maps sign-magnitude 8-bit float patterns to monotone integers."""
    b = bits.astype(np.int32)
    return np.where(b & 0x80, -(b & 0x7F), b)


def _ulp8(want_bits: np.ndarray, dt: int) -> np.ndarray:
    """One unit in the last place of each 8-bit float value, as float64."""
    mant, bias = (3, 7) if dt == W.F8_E4M3 else (2, 15)
    e = np.maximum((want_bits.astype(np.int32) >> mant) & ((1 << (7 - mant)) - 1), 1)
    return np.ldexp(1.0, e - bias - mant)


def _ulp16(want_bits: np.ndarray, dt: int) -> np.ndarray:
    """One unit in the last place of each 16-bit float value, as float64."""
    mant = 7 if dt == W.BF16 else 10
    bias = 127 if dt == W.BF16 else 15
    e = ((want_bits.astype(np.int32) >> mant) & ((1 << (15 - mant)) - 1))
    e = np.maximum(e, 1)  # subnormals share the spacing of the smallest normal
    return np.ldexp(1.0, e - bias - mant)


def summation_slack(p: W.Problem) -> np.ndarray:
    """4 * 2^-24 * sum_k |s_k| |w_k| scaled like the result, per dst element.
    Dense floating-point problems with per-tensor / per-row / per-column scales."""
    s = np.abs(W.to_f32(p.src.data.reshape(p.M, p.K), p.src.dt)).astype(np.float64)
    wdt = p.wei.dt
    wraw = p.wei.data
    if p.wei.strides[-1] != 1:  # `ba` storage
        w = W.to_f32(wraw.reshape(p.N, -1), wdt).T
    else:
        w = W.to_f32(wraw.reshape(p.K, -1), wdt)
    w = np.abs(w.astype(np.float64))
    if "wei_zp" in p.quant:  # magnitude bound with the largest zero-point folded in
        zq = p.quant["wei_zp"]
        w = w + max(16.0, float(np.abs(W.to_f32(zq.data, zq.dt)).max(initial=0)))
    mag = s @ w
    for name in ("src_scale", "wei_scale"):
        q = p.quant.get(name)
        if q is not None:
            sc = np.abs(W.to_f32(q.data, q.dt).astype(np.float64))
            if sc.size == 1:
                mag = mag * float(sc.reshape(-1)[0])
            elif name == "src_scale":
                mag = mag * sc.reshape(p.M, 1)
            elif sc.size == p.N:
                mag = mag * sc.reshape(1, p.N)
            else:  # K-grouped weight scales: bound with the largest scale per column
                mag = mag * sc.reshape(-1, p.N).max(axis=0, keepdims=True)
    return 4.0 * 2.0 ** -24 * mag


def summation_slack_grouped(p: W.Problem) -> np.ndarray:
    """The same allowance for a grouped problem: every expert's rows against
    that expert's weights and per-(expert, column) scales."""
    s = np.abs(W.to_f32(p.src.data.reshape(p.M, p.K), p.src.dt)).astype(np.float64)
    w = np.abs(W.to_f32(p.wei.data.reshape(p.groups, p.K, p.N), p.wei.dt).astype(np.float64))
    q = p.quant.get("wei_scale")
    sc = np.abs(W.to_f32(q.data, q.dt).astype(np.float64)).reshape(p.groups, -1, p.N).max(axis=1) if q is not None \
        else np.ones((p.groups, p.N))
    zq = p.quant.get("wei_zp")
    if zq is not None:  # per-(expert, column) zero-points join the magnitude of every term
        w = w + np.abs(W.to_f32(zq.data, zq.dt).astype(np.float64)).reshape(p.groups, 1, -1)
    mag = np.zeros((p.M, p.N))
    begin = 0
    for g, end in enumerate(p.offsets.astype(np.int64)):
        if end > begin:
            mag[begin:end] = (s[begin:end] @ w[g]) * sc[g][None, :]
        begin = int(end)
    return 4.0 * 2.0 ** -24 * mag


def compare(got: np.ndarray, want: np.ndarray, dt: int, slack=None):
    """Returns (ok, message).  `slack`: per-element absolute allowance in real
    units (see the module docstring), or None for the plain rules."""
    assert got.shape == want.shape, (got.shape, want.shape)
    if dt == W.S32:
        bad = got != want
        return not bad.any(), "s32 mismatches: %d" % int(bad.sum())
    if dt == W.F32:
        err = np.abs(got.astype(np.float64) - want.astype(np.float64))
        tol = 1e-5 * np.abs(want.astype(np.float64)) + 1e-30
        if slack is not None:
            tol = tol + slack
        bad = ~(err <= tol)
        worst = float((err / (np.abs(want) + 1e-30)).max()) if err.size else 0.0
        return not bad.any(), "f32 beyond 1e-5 rel: %d (worst rel %.3g)" % (int(bad.sum()), worst)
    if dt in (W.BF16, W.F16):
        d = np.abs(_ordered(got) - _ordered(want))
        n1, n0 = int((d > 1).sum()), int((d > 0).sum())
        if slack is None:
            return n1 == 0, "16-bit float ulp distance max %d, >1 at %d, !=0 at %d" % (int(d.max(initial=0)), n1, n0)
        err = np.abs(W.to_f32(got, dt).astype(np.float64) - W.to_f32(want, dt).astype(np.float64))
        bad = ~(err <= _ulp16(want, dt) + slack)
        return not bad.any(), "beyond 1 ulp + summation slack: %d of %d (>1 ulp at %d, !=0 at %d, max abs err %.3g)" % (
            int(bad.sum()), d.size, n1, n0, float(err.max(initial=0)))
    if dt in (W.F8_E4M3, W.F8_E5M2):  # like the 16-bit floats: one unit of the output type
        d = np.abs(_ordered8(got) - _ordered8(want))
        n1, n0 = int((d > 1).sum()), int((d > 0).sum())
        if slack is None:
            return n1 == 0, "8-bit float ulp distance max %d, >1 at %d, !=0 at %d" % (int(d.max(initial=0)), n1, n0)
        decode = W.e4m3_to_f32 if dt == W.F8_E4M3 else (lambda b: (b.astype(np.uint16) << 8).view(np.float16).astype(np.float32))
        err = np.abs(decode(got).astype(np.float64) - decode(want).astype(np.float64))
        bad = ~((err <= _ulp8(want, dt) + slack) | (got == want))
        return not bad.any(), "beyond 1 ulp + slack: %d of %d (>1 ulp at %d)" % (int(bad.sum()), d.size, n1)
    if dt in (W.S8, W.U8):
        d = np.abs(got.astype(np.int32) - want.astype(np.int32))
        return int(d.max(initial=0)) <= 1, "8-bit int distance max %d, !=0 at %d" % (
            int(d.max(initial=0)), int((d > 0).sum()))
    raise ValueError(dt)


def assert_parity(got, want, dt, what="", slack=None):
    ok, msg = compare(got, want, dt, slack)
    assert ok, "%s: %s" % (what, msg)
    return msg


def exact_rows_f64(p: W.Problem, rows) -> np.ndarray:
    """fp64 evaluation of dst rows of a floating-point problem without post-ops: sum_k s_k *
    (w_k - zp) * scale, times the src scale, plus the bias -- the value both the reference and the
    kernels approximate.  Supports what the benchmark's floating-point configurations use:
    per-tensor src scale; weight scales / zero-points per tensor, per column, per (K-group, column)
    or per (expert, column)."""
    assert not p.post_ops and p.src.dt not in (W.S8, W.U8)
    rows = np.asarray(rows, dtype=np.int64)
    src = W.to_f32(p.src.data.reshape(p.M, p.K)[rows], p.src.dt).astype(np.float64)
    grouped = p.offsets is not None

    def wq(name, g):
        """[K, N] float64 view of a weight parameter for expert g (None when absent)."""
        q = p.quant.get(name)
        if q is None:
            return None
        v = W.to_f32(q.data, q.dt).astype(np.float64)
        if v.size == 1:
            return v.reshape(1, 1)
        if grouped:
            return v.reshape(p.groups, -1, p.N)[g]  # [1, N]
        v = v.reshape(-1, p.N)  # [K/g or 1, N]
        return np.repeat(v, p.K // v.shape[0], axis=0) if v.shape[0] > 1 else v

    def weights(g):
        if grouped:
            w = W.to_f32(p.wei.data.reshape(p.groups, p.K, p.N)[g], p.wei.dt)
        elif p.wei.strides[-1] != 1:
            w = W.to_f32(p.wei.data.reshape(p.N, -1), p.wei.dt).T
        else:
            w = W.to_f32(p.wei.data.reshape(p.K, -1), p.wei.dt)
        w = w.astype(np.float64)
        z, s = wq("wei_zp", g), wq("wei_scale", g)
        if z is not None:
            w = w - z
        if s is not None:
            w = w * s
        return w

    out = np.zeros((len(rows), p.N))
    if grouped:
        ends = p.offsets.astype(np.int64)
        owner = np.searchsorted(ends, rows, side="right")
        for g in np.unique(owner):
            sel = owner == g
            out[sel] = src[sel] @ weights(int(g))
    else:
        out = src @ weights(0)
    q = p.quant.get("src_scale")
    if q is not None:
        sc = W.to_f32(q.data, q.dt).astype(np.float64)
        out = out * (float(sc.reshape(-1)[0]) if sc.size == 1 else sc.reshape(p.M, 1)[rows])
    if p.bias is not None:
        b = W.to_f32(p.bias.data, p.bias.dt).astype(np.float64)
        if grouped:
            out = out + b.reshape(p.groups, p.N)[np.searchsorted(p.offsets.astype(np.int64), rows, side="right")]
        else:
            b = b.reshape(p.bias.dims)
            out = out + (b[rows] if b.shape[0] > 1 else b)
    q = p.quant.get("dst_scale")
    if q is not None:
        out = out / float(W.to_f32(q.data, q.dt).reshape(-1)[0])
    return out


def rows_slack(p: W.Problem, rows) -> np.ndarray:
    """Summation slack of the given dst rows only (the whole-problem helpers would widen the full
    weight tensor once per call; here one expert / the dense matrix at a time)."""
    rows = np.asarray(rows, dtype=np.int64)
    if p.offsets is None:
        return summation_slack(p.take_rows(rows))
    src = np.abs(W.to_f32(p.src.data.reshape(p.M, p.K)[rows], p.src.dt)).astype(np.float64)
    q = p.quant.get("wei_scale")
    sc = np.abs(W.to_f32(q.data, q.dt).astype(np.float64)).reshape(p.groups, -1, p.N).max(axis=1) if q is not None \
        else np.ones((p.groups, p.N))
    zq = p.quant.get("wei_zp")
    ends = p.offsets.astype(np.int64)
    owner = np.searchsorted(ends, rows, side="right")
    out = np.zeros((len(rows), p.N))
    for g in np.unique(owner):
        w = np.abs(W.to_f32(p.wei.data.reshape(p.groups, p.K, p.N)[g], p.wei.dt).astype(np.float64))
        if zq is not None:
            w = w + np.abs(W.to_f32(zq.data, zq.dt).astype(np.float64)).reshape(p.groups, 1, -1)[g]
        sel = owner == g
        out[sel] = (src[sel] @ w) * sc[g][None, :]
    return 4.0 * 2.0 ** -24 * out


def check_rows(p: W.Problem, got: np.ndarray, rows, reordered_fp: bool, want_rows=None) -> dict:
    """Compares dst rows `rows` of `got` ([M, N] storage of the full problem) with the oracle's.
    `reordered_fp`: the checked kernel adds the K products in another order than the reference
    (floating-point problems only), so the summation slack applies.  Returns
    {"rows", "ok", "msg", "beyond_strict", "strict_misses_explained"}; `want_rows` lets the caller
    pass oracle rows it already has."""
    from oracle import oracle as O
    rows = np.unique(np.asarray(rows, dtype=np.int64))
    if want_rows is None:
        want_rows = O.run_port(p, rows=rows).reshape(p.M, -1)[rows]
    g = got.reshape(p.M, -1)[rows]
    fp = p.src.dt not in (W.S8, W.U8)
    slack = rows_slack(p, rows) if (fp and reordered_fp) else None
    ok, msg = compare(g, want_rows, p.dst_dt, slack)
    res = {"rows": int(len(rows)), "ok": bool(ok), "msg": msg, "beyond_strict": 0, "strict_misses_explained": True}
    if not fp or p.dst_dt not in (W.BF16, W.F16, W.F32) or p.post_ops:
        return res
    # elements beyond the strict rule (no slack), each judged against fp64
    gv = W.to_f32(g, p.dst_dt).astype(np.float64)
    wv = W.to_f32(want_rows, p.dst_dt).astype(np.float64)
    if p.dst_dt == W.F32:
        unit = 1e-5 * np.abs(wv) + 1e-30
        miss = np.abs(gv - wv) > unit
    else:
        unit = _ulp16(want_rows, p.dst_dt)
        miss = np.abs(_ordered(g) - _ordered(want_rows)) > 1
    res["beyond_strict"] = int(miss.sum())
    if miss.any():
        exact = exact_rows_f64(p, rows)
        d_gpu, d_ref = np.abs(gv - exact)[miss], np.abs(wv - exact)[miss]
        sl = (slack if slack is not None else np.zeros_like(gv))[miss]
        by_reference = d_gpu <= d_ref + unit[miss]
        by_roundoff = d_gpu <= unit[miss] + sl
        explained = by_reference | by_roundoff
        res["strict_misses_explained"] = bool(explained.all())
        res["strict_misses_gpu_closer"] = int((d_gpu <= d_ref).sum())
        res["strict_misses_within_roundoff_of_fp64"] = int(by_roundoff.sum())
        if not explained.all():
            res["ok"] = False
            res["msg"] += "; %d strict-rule misses are farther from the fp64 value than the reference" % int((~explained).sum())
    return res
