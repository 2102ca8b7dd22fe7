"""Comparison helpers shared by the tests: bit equality and the floating-point tolerances."""
from __future__ import annotations

import numpy as np


def bits(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    if a.dtype == np.float32:
        return a.view(np.uint32)
    if a.dtype == np.bool_:
        return a.view(np.uint8)
    return a


def assert_bit_equal(got: np.ndarray, ref: np.ndarray, what: str = "", *, any_nan: bool = False) -> None:
    """Bit-for-bit equality.  any_nan=True is for results of floating-point ARITHMETIC: which NaN
    bit pattern an operation produces is a property of the executing hardware (x86 propagates an
    input NaN's payload, NVIDIA GPUs return the canonical 0x7fffffff), so there every NaN matches
    every NaN; everything else, including the sign of zero, is still compared bit for bit."""
    got = np.asarray(got)
    ref = np.asarray(ref)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} != {ref.shape}"
    if any_nan and got.dtype == np.float32:
        assert np.array_equal(np.isnan(got), np.isnan(ref)), f"{what}: NaN positions differ"
        got = np.where(np.isnan(got), np.float32(0), got)
        ref = np.where(np.isnan(ref), np.float32(0), ref)
    g, r = bits(got), bits(ref)
    if not np.array_equal(g, r):
        bad = np.flatnonzero(g.ravel() != r.ravel())
        i = int(bad[0])
        raise AssertionError(
            f"{what}: {bad.size} of {g.size} elements differ; first at {i}: got {got.ravel()[i]!r} "
            f"(0x{int(g.ravel()[i]):x}) ref {ref.ravel()[i]!r} (0x{int(r.ravel()[i]):x})")


def ulp(ref: np.ndarray) -> np.ndarray:
    """Size of one unit in the last place at |ref| (f32)."""
    ref = np.abs(ref.astype(np.float32))
    return np.maximum(np.spacing(ref), np.float32(1.4e-45)).astype(np.float64)


CVT_NAMES = ["uint8", "int8", "int16", "int32", "int64", "float16", "bf16", "float32", "float64", "bool"]
_CVT_NP = {"uint8": np.uint8, "int8": np.int8, "int16": np.int16, "int32": np.int32, "int64": np.int64,
           "float16": np.float16, "bf16": np.uint16, "float32": np.float32, "float64": np.float64, "bool": np.bool_}


def cvt_case(golden, src: str, dst: str):
    """(input, expected) of one conversion fixture, in the array types the bindings take
    (bfloat16 as uint16 bit patterns, bool as numpy bool)."""
    key = f"cvt_src_{src}_for_uint8" if dst == "uint8" and src not in ("uint8", "bool") else f"cvt_src_{src}"
    return golden[key].view(_CVT_NP[src]), golden[f"cvt_{src}_to_{dst}"].view(_CVT_NP[dst])


def assert_close_ulp(got, ref, *, ulps: float = 2.0, rel: float = 1e-6, abs_floor: float = 0.0, what: str = ""):
    """|got - ref| <= max(ulps * ulp(ref), rel * |ref|, abs_floor); NaN/inf must match exactly.

    silu uses (2 ulp, 1e-6, 0); erf-GELU adds abs_floor = 2e-6 because the CPU kernel's own two
    code paths differ by up to 1.43e-6 where 1 + erf(x / sqrt(2)) cancels.
    """
    got = np.asarray(got, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} != {ref.shape}"
    special = ~np.isfinite(ref)
    if special.any():
        assert np.array_equal(np.isnan(got[special]), np.isnan(ref[special])), f"{what}: NaN pattern differs"
        inf = special & ~np.isnan(ref)
        assert np.array_equal(got[inf], ref[inf]), f"{what}: infinities differ"
    fin = ~special
    err = np.abs(got[fin].astype(np.float64) - ref[fin].astype(np.float64))
    tol = np.maximum(np.maximum(ulps * ulp(ref[fin]), rel * np.abs(ref[fin].astype(np.float64))), abs_floor)
    bad = err > tol
    if bad.any():
        i = int(np.flatnonzero(bad)[0])
        raise AssertionError(f"{what}: {int(bad.sum())} of {err.size} outside tolerance; first: got {got[fin][i]!r} "
                             f"ref {ref[fin][i]!r} err {err[i]:.3e} tol {tol[i]:.3e}")
    return float(err.max()) if err.size else 0.0


def max_ulp_distance(got: np.ndarray, ref: np.ndarray) -> float:
    fin = np.isfinite(ref) & np.isfinite(got)
    if not fin.any():
        return 0.0
    return float((np.abs(got[fin].astype(np.float64) - ref[fin].astype(np.float64)) / ulp(ref[fin])).max())
