"""Comparison rules of the parity tests.

* s32 and every integer/byte/index result: bit-exact.
* f32: |got - want| <= 1e-5 * |want| (+ 1e-30 for exact zeros).
* bf16 / f16: at most 1 ulp apart, measured on the ordered bit patterns.
* s8 / u8 (a requantized f32): at most 1 apart.
"""
import numpy as np

from onednn_b200 import workloads as W


def _ordered(bits: np.ndarray) -> np.ndarray:
    """Maps sign-magnitude 16-bit float patterns to monotone integers."""
    b = bits.astype(np.int32)
    return np.where(b & 0x8000, -(b & 0x7FFF), b)


def compare(got: np.ndarray, want: np.ndarray, dt: int):
    """Returns (ok, message)."""
    assert got.shape == want.shape, (got.shape, want.shape)
    if dt == W.S32:
        bad = got != want
        return not bad.any(), "s32 mismatches: %d" % int(bad.sum())
    if dt == W.F32:
        err = np.abs(got.astype(np.float64) - want.astype(np.float64))
        tol = 1e-5 * np.abs(want.astype(np.float64)) + 1e-30
        bad = ~(err <= tol)
        worst = float((err / (np.abs(want) + 1e-30)).max()) if err.size else 0.0
        return not bad.any(), "f32 beyond 1e-5 rel: %d (worst rel %.3g)" % (int(bad.sum()), worst)
    if dt in (W.BF16, W.F16):
        d = np.abs(_ordered(got) - _ordered(want))
        return int(d.max(initial=0)) <= 1, "16-bit float ulp distance max %d, >1 at %d, !=0 at %d" % (
            int(d.max(initial=0)), int((d > 1).sum()), int((d > 0).sum()))
    if dt in (W.S8, W.U8):
        d = np.abs(got.astype(np.int32) - want.astype(np.int32))
        return int(d.max(initial=0)) <= 1, "8-bit int distance max %d, !=0 at %d" % (
            int(d.max(initial=0)), int((d > 0).sum()))
    raise ValueError(dt)


def assert_parity(got, want, dt, what=""):
    ok, msg = compare(got, want, dt)
    assert ok, "%s: %s" % (what, msg)
    return msg
