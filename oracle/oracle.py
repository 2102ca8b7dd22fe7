"""ctypes front end of the CPU oracle (oracle/twg_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the CPU-baseline
leg of bench.py as the checker / timed baseline.  The shipped package never imports it.

Arrays are numpy; views with arbitrary (non-negative or negative) strides and broadcasting are
described to the C code the same way the reference describes them to its shaders: a logical
shape plus per-operand element strides and offsets (csrc/ops/binary.h:108-124).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
MAX_DIMS = 8

UNARY = {"copy": 0, "relu": 1, "gelu_tanh": 2, "silu": 3, "gelu_erf": 4, "abs": 5,
         "silu_shader": 6, "gelu_tanh_shader": 7}
BINARY = {"add": 0, "mul": 1, "fused_add_relu": 2, "div": 3}
COMPARE = {"eq": 0, "ne": 1, "lt": 2, "le": 3, "gt": 4, "ge": 5}


class TwgoIter(ctypes.Structure):
    _fields_ = [
        ("ndim", ctypes.c_int32),
        ("pad", ctypes.c_int32),
        ("length", ctypes.c_int64),
        ("shape", ctypes.c_int64 * MAX_DIMS),
        ("out_strides", ctypes.c_int64 * MAX_DIMS),
        ("a_strides", ctypes.c_int64 * MAX_DIMS),
        ("b_strides", ctypes.c_int64 * MAX_DIMS),
        ("out_offset", ctypes.c_int64),
        ("a_offset", ctypes.c_int64),
        ("b_offset", ctypes.c_int64),
    ]


def build(force: bool = False) -> Path:
    """Compile liboracle.so next to its source if it is missing or stale."""
    so = HERE / "liboracle.so"
    src = HERE / "twg_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B" if force else "-s"], check=True, capture_output=True)
    return so


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        so = HERE / "liboracle.so"
        if not so.exists():
            build()
        _lib = ctypes.CDLL(str(so))
        _lib.twgo_masked_select_f32.restype = ctypes.c_int64
    return _lib


def num_threads() -> int:
    return int(lib().twgo_num_threads())


def set_num_threads(n: int) -> None:
    lib().twgo_set_num_threads(int(n))


def _ptr(a: np.ndarray):
    return ctypes.c_void_p(a.ctypes.data)


def _elem_strides(a: np.ndarray) -> list[int]:
    return [s // a.itemsize for s in a.strides]


def _iter(shape, out: np.ndarray | None, a: np.ndarray, b: np.ndarray | None) -> TwgoIter:
    if len(shape) > MAX_DIMS:
        raise RuntimeError(f"tensors of more than {MAX_DIMS} dimensions are not supported")
    it = TwgoIter()
    it.ndim = len(shape)
    it.length = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    for d, s in enumerate(shape):
        it.shape[d] = s
    for name, arr in (("out_strides", out), ("a_strides", a), ("b_strides", b)):
        if arr is None:
            continue
        view = np.broadcast_to(arr, shape) if arr.shape != tuple(shape) else arr
        dst = getattr(it, name)
        for d, s in enumerate(_elem_strides(view)):
            dst[d] = s
    return it


def unary(op: str, x: np.ndarray) -> np.ndarray:
    assert x.dtype == np.float32
    out = np.empty(x.shape, dtype=np.float32)
    it = _iter(x.shape, out, x, None)
    rc = lib().twgo_unary_f32(UNARY[op], ctypes.byref(it), _ptr(x), _ptr(out))
    assert rc == 0
    return out


def binary(op: str, a: np.ndarray, b: np.ndarray, alpha: float = 1.0) -> np.ndarray:
    assert a.dtype == np.float32 and b.dtype == np.float32
    shape = np.broadcast_shapes(a.shape, b.shape)
    out = np.empty(shape, dtype=np.float32)
    it = _iter(shape, out, a, b)
    rc = lib().twgo_binary_f32(BINARY[op], ctypes.byref(it), _ptr(a), _ptr(b), ctypes.c_float(alpha), _ptr(out))
    assert rc == 0
    return out


def sub(a: np.ndarray, b: np.ndarray, alpha: float = 1.0) -> np.ndarray:
    """a - alpha*b the way ATen computes it: add with the negated alpha (one rounding)."""
    return binary("add", a, b, -alpha)


DTYPES = {"uint8": 0, "int8": 1, "int16": 2, "int32": 3, "int64": 4, "float16": 5, "bf16": 6, "float32": 7,
          "float64": 8, "bool": 9}
_NP_OF = {"uint8": np.uint8, "int8": np.int8, "int16": np.int16, "int32": np.int32, "int64": np.int64,
          "float16": np.float16, "bf16": np.uint16, "float32": np.float32, "float64": np.float64, "bool": np.bool_}


def convert(x: np.ndarray, src: str, dst: str) -> np.ndarray:
    """Element-type conversion; bfloat16 travels as uint16 bit patterns under the name "bf16"."""
    xs = np.ascontiguousarray(x)
    assert xs.dtype == _NP_OF[src], (xs.dtype, src)
    out = np.empty(xs.shape, dtype=_NP_OF[dst])
    rc = lib().twgo_convert(ctypes.c_int64(xs.size), DTYPES[src], DTYPES[dst], _ptr(xs), _ptr(out))
    assert rc == 0
    return out


def where(cond: np.ndarray, a: np.ndarray, b: np.ndarray) -> np.ndarray:
    assert cond.dtype == np.bool_ and a.dtype == np.float32 and b.dtype == np.float32
    shape = np.broadcast_shapes(cond.shape, a.shape, b.shape)
    c, x, y = (np.ascontiguousarray(np.broadcast_to(t, shape)) for t in (cond.view(np.uint8), a, b))
    out = np.empty(shape, dtype=np.float32)
    rc = lib().twgo_where_f32(ctypes.c_int64(out.size), _ptr(c), _ptr(x), _ptr(y), _ptr(out))
    assert rc == 0
    return out


def masked_fill(x: np.ndarray, mask: np.ndarray, value: float) -> np.ndarray:
    assert mask.dtype == np.bool_ and x.dtype == np.float32
    shape = np.broadcast_shapes(x.shape, mask.shape)
    xs, m = (np.ascontiguousarray(np.broadcast_to(t, shape)) for t in (x, mask.view(np.uint8)))
    out = np.empty(shape, dtype=np.float32)
    rc = lib().twgo_masked_fill_f32(ctypes.c_int64(out.size), _ptr(xs), _ptr(m), ctypes.c_float(value), _ptr(out))
    assert rc == 0
    return out


def compare(op: str, a: np.ndarray, b) -> np.ndarray:
    assert a.dtype == np.float32
    if isinstance(b, np.ndarray):
        assert b.dtype == np.float32
        shape = np.broadcast_shapes(a.shape, b.shape)
        out = np.empty(shape, dtype=np.uint8)
        it = _iter(shape, out, a, b)
        rc = lib().twgo_compare_f32(COMPARE[op], ctypes.byref(it), _ptr(a), _ptr(b), ctypes.c_float(0.0), _ptr(out))
    else:
        out = np.empty(a.shape, dtype=np.uint8)
        it = _iter(a.shape, out, a, None)
        rc = lib().twgo_compare_f32(COMPARE[op], ctypes.byref(it), _ptr(a), None, ctypes.c_float(float(b)), _ptr(out))
    assert rc == 0
    return out.view(np.bool_)


def bitwise_and(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    assert a.dtype == b.dtype
    shape = np.broadcast_shapes(a.shape, b.shape)
    if a.dtype == np.bool_:
        out = np.empty(shape, dtype=np.uint8)
        a8, b8 = a.view(np.uint8), b.view(np.uint8)
        it = _iter(shape, out, a8, b8)
        rc = lib().twgo_and_bool(ctypes.byref(it), _ptr(a8), _ptr(b8), _ptr(out))
        assert rc == 0
        return out.view(np.bool_)
    out = np.empty(shape, dtype=a.dtype)
    it = _iter(shape, out, a, b)
    rc = lib().twgo_and_bytes(ctypes.byref(it), a.itemsize, _ptr(a), _ptr(b), _ptr(out))
    assert rc == 0
    return out


def copy(x: np.ndarray) -> np.ndarray:
    """Strided gather of `x` into a fresh C-contiguous array (UnaryOp::Copy)."""
    out = np.empty(x.shape, dtype=x.dtype)
    it = _iter(x.shape, out, x, None)
    rc = lib().twgo_copy_bytes(ctypes.byref(it), x.itemsize, _ptr(x), _ptr(out))
    assert rc == 0
    return out


def masked_select(x: np.ndarray, mask: np.ndarray) -> np.ndarray:
    assert x.dtype == np.float32
    if mask.dtype != np.bool_:
        raise RuntimeError("masked_select: expected BoolTensor for mask")
    shape = np.broadcast_shapes(x.shape, mask.shape)
    m8 = mask.view(np.uint8)
    it = _iter(shape, None, x, m8)
    out = np.empty(int(it.length), dtype=np.float32)
    k = lib().twgo_masked_select_f32(ctypes.byref(it), _ptr(x), _ptr(m8), _ptr(out))
    assert k >= 0
    return out[:k].copy()


def chain_mask(a: np.ndarray, b: np.ndarray, c: np.ndarray, want_y: bool = False):
    """y = relu(silu(a + b) + c); m = (y == 0) & (a != 0) on dense arrays."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    c = np.ascontiguousarray(c, dtype=np.float32)
    m = np.empty(a.shape, dtype=np.uint8)
    y = np.empty(a.shape, dtype=np.float32) if want_y else None
    rc = lib().twgo_chain_mask(ctypes.c_int64(a.size), _ptr(a), _ptr(b), _ptr(c), _ptr(y) if want_y else None, _ptr(m))
    assert rc == 0
    return (y, m.view(np.bool_)) if want_y else m.view(np.bool_)


if __name__ == "__main__":
    print(build(force=bool(os.environ.get("FORCE"))))
