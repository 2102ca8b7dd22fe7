"""ctypes binding of the library's C ABI (include/twg.h -> lib/libtwg.so).

This is the thin foreign-function layer a host language binds against; the PyTorch extension
(`torch_webgpu._C`) calls the same entry points from C++.  Nothing here computes on the CPU: if
the shared library is missing the import of any entry point raises, there is no fallback.

The numpy-level helpers at the bottom (`unary`, `binary`, `compare`, `bitwise_and`, `copy`,
`masked_select`, `fused`) upload their operands, run ONE library call on the device and download
the result; they exist so that parity tests and small scripts can drive the C ABI without torch.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

import numpy as np

MAX_DIMS = 8
MAX_TENSORS = 8

UNARY = {"copy": 0, "relu": 1, "gelu_tanh": 2, "silu": 3, "gelu_erf": 4, "abs": 5}
BINARY = {"add": 0, "mul": 1, "fused_add_relu": 2, "div": 3}
COMPARE = {"eq": 0, "ne": 1, "lt": 2, "le": 3, "gt": 4, "ge": 5}
PATHS = {0: "none", 1: "dense", 2: "tile", 3: "strided32", 4: "strided64"}

TWG_OK, TWG_ERR_INVALID, TWG_ERR_CUDA, TWG_ERR_OOM, TWG_ERR_TIMEOUT, TWG_ERR_UNSUPPORTED = 0, -1, -2, -3, -4, -5

# fused-program opcodes (TwgFusedOpcode)
F_INPUT_F32, F_INPUT_BOOL, F_CONST_F32, F_ADD, F_MUL, F_RELU, F_SILU, F_GELU_ERF, F_GELU_TANH, F_ABS = range(10)
F_EQ, F_NE, F_LT, F_LE, F_GT, F_GE, F_AND, F_OUTPUT = range(10, 18)


class TwgError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"twg error {code}: {message}")
        self.code = code


class IterDesc(ctypes.Structure):
    _fields_ = [
        ("ndim", c_int32),
        ("ntensors", c_int32),
        ("numel", c_int64),
        ("shape", c_int64 * MAX_DIMS),
        ("strides", (c_int64 * MAX_DIMS) * MAX_TENSORS),
    ]


class MemStats(ctypes.Structure):
    _fields_ = [(n, c_int64) for n in (
        "allocated_bytes", "reserved_bytes", "peak_allocated_bytes", "peak_reserved_bytes",
        "num_allocs", "num_cache_hits", "num_device_mallocs", "num_device_frees")]


class FusedInstr(ctypes.Structure):
    _fields_ = [("opcode", c_int32), ("a", c_int32), ("b", c_int32), ("imm", c_float)]


LIB_PATH = Path(__file__).resolve().parent / "lib" / "libtwg.so"
_lib = None

# name -> (restype, argtypes); every symbol include/twg.h declares
SIGNATURES = {
    "twg_iter_contiguous": (c_int, [POINTER(IterDesc), c_int, c_int64]),
    "twg_iter_coalesce": (c_int, [POINTER(IterDesc)]),
    "twg_last_error": (c_char_p, []),
    "twg_version": (c_char_p, []),
    "twg_device_count": (c_int, [POINTER(c_int)]),
    "twg_set_device": (c_int, [c_int]),
    "twg_get_device": (c_int, [POINTER(c_int)]),
    "twg_get_stream": (c_int, [c_int, c_int, POINTER(c_void_p)]),
    "twg_stream_sync": (c_int, [c_void_p]),
    "twg_device_sync": (c_int, [c_int]),
    "twg_stream_query": (c_int, [c_void_p, POINTER(c_int)]),
    "twg_event_create": (c_int, [POINTER(c_void_p)]),
    "twg_event_destroy": (c_int, [c_void_p]),
    "twg_event_record": (c_int, [c_void_p, c_void_p]),
    "twg_event_wait": (c_int, [c_void_p, c_void_p]),
    "twg_event_query": (c_int, [c_void_p, POINTER(c_int)]),
    "twg_event_sync": (c_int, [c_void_p]),
    "twg_event_elapsed_ms": (c_int, [c_void_p, c_void_p, POINTER(c_float)]),
    "twg_malloc": (c_int, [POINTER(c_void_p), c_size_t, c_int, c_void_p]),
    "twg_free": (c_int, [c_void_p]),
    "twg_record_stream": (c_int, [c_void_p, c_void_p]),
    "twg_trim": (c_int, [c_void_p, c_size_t]),
    "twg_block_size": (c_int, [c_void_p, POINTER(c_size_t), POINTER(c_int)]),
    "twg_empty_cache": (c_int, [c_int]),
    "twg_memory_stats": (c_int, [c_int, POINTER(MemStats)]),
    "twg_reset_peak_stats": (c_int, [c_int]),
    "twg_set_memory_budget": (c_int, [c_int, c_size_t]),
    "twg_set_guard_words": (c_int, [c_int]),
    "twg_check_guard_words": (c_int, [c_int, POINTER(c_int64), POINTER(c_void_p)]),
    "twg_memcpy_h2d": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "twg_memcpy_d2h": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_int]),
    "twg_memcpy_d2d": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "twg_memset": (c_int, [c_void_p, c_int, c_size_t, c_void_p]),
    "twg_host_alloc_pinned": (c_int, [POINTER(c_void_p), c_size_t]),
    "twg_host_free_pinned": (c_int, [c_void_p]),
    "twg_copy_strided": (c_int, [POINTER(IterDesc), c_int, c_void_p, c_void_p, c_void_p]),
    "twg_fill": (c_int, [POINTER(IterDesc), c_int, ctypes.c_uint64, c_void_p, c_void_p]),
    "twg_unary_f32": (c_int, [c_int, POINTER(IterDesc), c_void_p, c_void_p, c_void_p]),
    "twg_binary_f32": (c_int, [c_int, POINTER(IterDesc), c_void_p, c_void_p, c_float, c_void_p, c_void_p]),
    "twg_compare_f32": (c_int, [c_int, POINTER(IterDesc), c_void_p, c_void_p, c_float, c_void_p, c_void_p]),
    "twg_binary_scalar_f32": (c_int, [c_int, POINTER(IterDesc), c_void_p, c_float, c_float, c_void_p, c_void_p]),
    "twg_convert": (c_int, [POINTER(IterDesc), c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "twg_where_f32": (c_int, [POINTER(IterDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "twg_masked_fill_f32": (c_int, [POINTER(IterDesc), c_void_p, c_void_p, c_float, c_void_p, c_void_p]),
    "twg_bitwise_and": (c_int, [POINTER(IterDesc), c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "twg_masked_select_workspace_bytes": (c_size_t, [c_int64]),
    "twg_masked_select_f32": (c_int, [POINTER(IterDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_size_t, c_void_p]),
    "twg_masked_select_set_poll_budget": (c_int, [c_int64]),
    "twg_masked_select_static_max_numel": (c_int64, []),
    "twg_masked_select_f32_static": (c_int, [POINTER(IterDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "twg_fused_compile": (c_int, [POINTER(FusedInstr), c_int, POINTER(c_void_p)]),
    "twg_fused_kind": (c_int, [c_void_p, POINTER(c_int)]),
    "twg_fused_launch": (c_int, [c_void_p, POINTER(IterDesc), POINTER(c_void_p), c_void_p]),
    "twg_fused_release": (c_int, [c_void_p]),
    "twg_fused_select_workspace_bytes": (c_size_t, [c_int64]),
    "twg_predicate_bits_bytes": (c_size_t, [c_int64]),
    "twg_fused_predicate_bits": (c_int, [c_void_p, c_int64, POINTER(c_void_p), c_void_p, c_void_p]),
    "twg_masked_select_bits_f32": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "twg_masked_select_bits_f32_publish": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_size_t,
                                                   c_void_p, c_int64, c_void_p]),
    "twg_fused_select_f32": (c_int, [c_void_p, c_int, c_int64, POINTER(c_void_p), c_void_p, c_void_p, c_void_p,
                                     c_size_t, c_void_p]),
    "twg_fused_select_f32_publish": (c_int, [c_void_p, c_int, c_int64, POINTER(c_void_p), c_void_p, c_void_p, c_void_p,
                                             c_size_t, c_void_p, c_int64, c_void_p]),
    "twg_fused_set_nvrtc_path": (c_int, [c_char_p]),
    "twg_fused_source": (c_int, [c_void_p, POINTER(c_char_p)]),
    "twg_fused_set_cache_dir": (c_int, [c_char_p]),
    "twg_fused_cache_stats": (c_int, [POINTER(c_int64), POINTER(c_int64)]),
    "twg_comm_set_nccl_path": (c_int, [c_char_p]),
    "twg_comm_unique_id": (c_int, [c_void_p]),
    "twg_comm_init_rank": (c_int, [c_void_p, c_int, c_int, POINTER(c_void_p)]),
    "twg_comm_destroy": (c_int, [c_void_p]),
    "twg_allgather_i64": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "twg_exchange_create": (c_int, [c_int, c_int, c_int, POINTER(c_void_p)]),
    "twg_exchange_handle": (c_int, [c_void_p, c_void_p]),
    "twg_exchange_connect_ipc": (c_int, [c_void_p, c_int, c_void_p]),
    "twg_exchange_connect_local": (c_int, [c_void_p, c_int, c_void_p]),
    "twg_exchange_publish": (c_int, [c_void_p, c_int64, c_void_p, c_void_p]),
    "twg_exchange_collect": (c_int, [c_void_p, c_int64, c_void_p]),
    "twg_masked_select_f32_publish": (c_int, [POINTER(IterDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_size_t, c_void_p, c_int64, c_void_p]),
    "twg_exchange_wait": (c_int, [c_void_p, c_int64, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64),
                                  POINTER(c_int64), c_int]),
    "twg_exchange_gathered": (c_int, [c_void_p, c_int64, POINTER(c_void_p)]),
    "twg_exchange_set_timeout_ns": (c_int, [c_void_p, c_int64]),
    "twg_exchange_destroy": (c_int, [c_void_p]),
    "twg_set_tracing": (c_int, [c_int]),
    "twg_get_tracing": (c_int, []),
    "twg_launch_count": (c_int64, []),
    "twg_reset_launch_count": (None, []),
    "twg_last_launch_path": (c_int, []),
}


def lib() -> ctypes.CDLL:
    """Load libtwg.so (once).  Raises if it has not been built - there is no CPU fallback."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python torch-webgpu_b200/build.py kernels`; "
                               "this package has no CPU fallback")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise TwgError(rc, lib().twg_last_error().decode(errors="replace"))


def last_path() -> str:
    return PATHS[lib().twg_last_launch_path()]


def device_count() -> int:
    n = c_int(0)
    check(lib().twg_device_count(byref(n)))
    return n.value


# ---------------------------------------------------------------------------------------------
# device memory
# ---------------------------------------------------------------------------------------------
class DeviceBuffer:
    """A block from the library's caching allocator."""

    def __init__(self, nbytes: int, device: int = 0, stream=None):
        self.nbytes = int(nbytes)
        self.device = device
        p = c_void_p()
        check(lib().twg_malloc(byref(p), self.nbytes, device, stream))
        self.ptr = p.value or 0

    def free(self) -> None:
        if self.ptr:
            check(lib().twg_free(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def upload(self, host: np.ndarray, stream=None) -> None:
        host = np.ascontiguousarray(host)
        assert host.nbytes <= self.nbytes
        check(lib().twg_memcpy_h2d(self.ptr, host.ctypes.data, host.nbytes, stream))

    def download(self, dtype, count: int, stream=None, offset_bytes: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        if out.nbytes:
            check(lib().twg_memcpy_d2h(out.ctypes.data, self.ptr + offset_bytes, out.nbytes, stream, 1))
        return out


def _root(a: np.ndarray) -> np.ndarray:
    while isinstance(a.base, np.ndarray):
        a = a.base
    return a


class DeviceArray:
    """Device mirror of a numpy array *view*: the owning buffer is uploaded whole and the view's
    shape, element strides and offset are kept, so non-contiguous and broadcast layouts reach the
    kernels exactly as they are."""

    def __init__(self, host: np.ndarray, device: int = 0, stream=None, pad_front: int = 0):
        root = _root(host)
        flat = np.ascontiguousarray(root).reshape(-1) if root.flags.c_contiguous else None
        if flat is None:
            raise ValueError("the owning array must be C-contiguous")
        self.dtype = host.dtype
        self.shape = tuple(host.shape)
        self.strides = tuple(s // host.itemsize for s in host.strides)
        self.offset = (host.__array_interface__["data"][0] - root.__array_interface__["data"][0]) // host.itemsize
        self.pad = pad_front * host.itemsize  # deliberately misalign the data by `pad_front` elements
        self.buf = DeviceBuffer(max(flat.nbytes + self.pad, 1), device, stream)
        if flat.nbytes:
            check(lib().twg_memcpy_h2d(self.buf.ptr + self.pad, flat.ctypes.data, flat.nbytes, stream))
        self.root_size = flat.size

    @classmethod
    def empty(cls, shape, dtype, device: int = 0, stream=None, pad_front: int = 0) -> "DeviceArray":
        self = cls.__new__(cls)
        self.dtype = np.dtype(dtype)
        self.shape = tuple(shape)
        st, acc = [], 1
        for s in reversed(self.shape):
            st.append(acc)
            acc *= max(s, 1)
        self.strides = tuple(reversed(st))
        self.offset = 0
        self.pad = pad_front * self.dtype.itemsize
        self.root_size = int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1
        self.buf = DeviceBuffer(max(self.root_size * self.dtype.itemsize + self.pad, 1), device, stream)
        return self

    @property
    def ptr(self) -> int:
        return self.buf.ptr + self.pad + self.offset * self.dtype.itemsize

    def numpy(self, stream=None) -> np.ndarray:
        """Download the owning buffer and re-apply the view."""
        flat = self.buf.download(self.dtype, self.root_size, stream, offset_bytes=self.pad)
        return np.lib.stride_tricks.as_strided(flat[self.offset:], self.shape,
                                               tuple(s * self.dtype.itemsize for s in self.strides)).copy()


def make_desc(shape, operands) -> IterDesc:
    """Descriptor for `operands` (DeviceArray or (shape, strides) pairs) broadcast to `shape`.

    Logical dimensions are reversed so that dimension 0 is the fastest one, the order
    at::TensorIterator hands to the reference's launchers.
    """
    shape = tuple(shape)
    if len(shape) > MAX_DIMS:
        raise TwgError(TWG_ERR_INVALID, f"tensors of more than {MAX_DIMS} dimensions are not supported")
    d = IterDesc()
    d.ndim = len(shape)
    d.ntensors = len(operands)
    d.numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
    for k, s in enumerate(reversed(shape)):
        d.shape[k] = s
    for t, op in enumerate(operands):
        oshape, ostrides = (op.shape, op.strides) if isinstance(op, DeviceArray) else op
        lead = len(shape) - len(oshape)
        for k in range(len(shape)):
            dim = len(shape) - 1 - k  # logical dimension
            if dim < lead or (oshape[dim - lead] == 1 and shape[dim] != 1):
                d.strides[t][k] = 0
            else:
                d.strides[t][k] = ostrides[dim - lead]
    return d


# ---------------------------------------------------------------------------------------------
# numpy-level helpers: one library call each
# ---------------------------------------------------------------------------------------------
def _sync(stream=None) -> None:
    check(lib().twg_stream_sync(stream))


def unary(op: str, x: np.ndarray, *, out_like: np.ndarray | None = None, pad: int = 0, stream=None) -> np.ndarray:
    """out_like: an array view whose layout the output should have (default: dense)."""
    dx = DeviceArray(x, stream=stream, pad_front=pad)
    do = DeviceArray(out_like, stream=stream) if out_like is not None else DeviceArray.empty(x.shape, np.float32,
                                                                                          stream=stream, pad_front=pad)
    d = make_desc(x.shape, [do, dx])
    check(lib().twg_unary_f32(UNARY[op], byref(d), dx.ptr, do.ptr, stream))
    return do.numpy(stream)


# TwgDtype by numpy dtype; bfloat16 travels as its uint16 bit pattern with dtype name "bf16"
DTYPES = {"uint8": 0, "int8": 1, "int16": 2, "int32": 3, "int64": 4, "float16": 5, "bf16": 6, "float32": 7,
          "float64": 8, "bool": 9}
_NP_OF = {"uint8": np.uint8, "int8": np.int8, "int16": np.int16, "int32": np.int32, "int64": np.int64,
          "float16": np.float16, "bf16": np.uint16, "float32": np.float32, "float64": np.float64, "bool": np.bool_}


def convert(x: np.ndarray, src: str, dst: str, *, pad: int = 0, stream=None) -> np.ndarray:
    """x holds `src` elements (uint16 bit patterns for "bf16"); returns the `dst` elements."""
    raw = x.view(np.uint8) if src == "bool" else x
    dx = DeviceArray(raw, stream=stream, pad_front=pad)
    out_np = np.uint8 if dst == "bool" else _NP_OF[dst]
    do = DeviceArray.empty(x.shape, out_np, stream=stream, pad_front=pad)
    d = make_desc(x.shape, [do, dx])
    check(lib().twg_convert(byref(d), DTYPES[src], DTYPES[dst], dx.ptr, do.ptr, stream))
    out = do.numpy(stream)
    return out.view(np.bool_) if dst == "bool" else out


def binary_scalar(op: str, a: np.ndarray, scalar: float, alpha: float = 1.0, *, pad: int = 0, stream=None) -> np.ndarray:
    da = DeviceArray(a, stream=stream, pad_front=pad)
    do = DeviceArray.empty(a.shape, np.float32, stream=stream, pad_front=pad)
    d = make_desc(a.shape, [do, da])
    check(lib().twg_binary_scalar_f32(BINARY[op], byref(d), da.ptr, scalar, alpha, do.ptr, stream))
    return do.numpy(stream)


def where(cond: np.ndarray, a: np.ndarray, b: np.ndarray, *, pad: int = 0, stream=None) -> np.ndarray:
    shape = np.broadcast_shapes(cond.shape, a.shape, b.shape)
    dc = DeviceArray(cond.view(np.uint8), stream=stream, pad_front=pad)
    da, db = DeviceArray(a, stream=stream, pad_front=pad), DeviceArray(b, stream=stream, pad_front=pad)
    do = DeviceArray.empty(shape, np.float32, stream=stream, pad_front=pad)
    d = make_desc(shape, [do, dc, da, db])
    check(lib().twg_where_f32(byref(d), dc.ptr, da.ptr, db.ptr, do.ptr, stream))
    return do.numpy(stream)


def masked_fill(x: np.ndarray, mask: np.ndarray, value: float, *, pad: int = 0, stream=None) -> np.ndarray:
    shape = np.broadcast_shapes(x.shape, mask.shape)
    dx = DeviceArray(x, stream=stream, pad_front=pad)
    dm = DeviceArray(mask.view(np.uint8), stream=stream, pad_front=pad)
    do = DeviceArray.empty(shape, np.float32, stream=stream, pad_front=pad)
    d = make_desc(shape, [do, dx, dm])
    check(lib().twg_masked_fill_f32(byref(d), dx.ptr, dm.ptr, value, do.ptr, stream))
    return do.numpy(stream)


def binary(op: str, a: np.ndarray, b: np.ndarray, alpha: float = 1.0, *, pad: int = 0, stream=None) -> np.ndarray:
    shape = np.broadcast_shapes(a.shape, b.shape)
    da, db = DeviceArray(a, stream=stream, pad_front=pad), DeviceArray(b, stream=stream, pad_front=pad)
    do = DeviceArray.empty(shape, np.float32, stream=stream, pad_front=pad)
    d = make_desc(shape, [do, da, db])
    check(lib().twg_binary_f32(BINARY[op], byref(d), da.ptr, db.ptr, alpha, do.ptr, stream))
    return do.numpy(stream)


def compare(op: str, a: np.ndarray, b, *, pad: int = 0, stream=None) -> np.ndarray:
    da = DeviceArray(a, stream=stream, pad_front=pad)
    if isinstance(b, np.ndarray):
        shape = np.broadcast_shapes(a.shape, b.shape)
        db = DeviceArray(b, stream=stream, pad_front=pad)
        do = DeviceArray.empty(shape, np.uint8, stream=stream, pad_front=pad)
        d = make_desc(shape, [do, da, db])
        check(lib().twg_compare_f32(COMPARE[op], byref(d), da.ptr, db.ptr, 0.0, do.ptr, stream))
    else:
        do = DeviceArray.empty(a.shape, np.uint8, stream=stream, pad_front=pad)
        d = make_desc(a.shape, [do, da])
        check(lib().twg_compare_f32(COMPARE[op], byref(d), da.ptr, None, float(b), do.ptr, stream))
    return do.numpy(stream).view(np.bool_)


def bitwise_and(a: np.ndarray, b: np.ndarray, *, pad: int = 0, stream=None) -> np.ndarray:
    assert a.dtype == b.dtype
    is_bool = a.dtype == np.bool_
    if is_bool:
        a, b = a.view(np.uint8), b.view(np.uint8)
    shape = np.broadcast_shapes(a.shape, b.shape)
    da, db = DeviceArray(a, stream=stream, pad_front=pad), DeviceArray(b, stream=stream, pad_front=pad)
    do = DeviceArray.empty(shape, a.dtype, stream=stream, pad_front=pad)
    d = make_desc(shape, [do, da, db])
    check(lib().twg_bitwise_and(byref(d), a.itemsize, int(is_bool), da.ptr, db.ptr, do.ptr, stream))
    out = do.numpy(stream)
    return out.view(np.bool_) if is_bool else out


def copy(x: np.ndarray, *, stream=None) -> np.ndarray:
    """Gather a strided view into a dense array on the device."""
    dx = DeviceArray(x, stream=stream)
    do = DeviceArray.empty(x.shape, x.dtype, stream=stream)
    d = make_desc(x.shape, [do, dx])
    check(lib().twg_copy_strided(byref(d), x.itemsize, dx.ptr, do.ptr, stream))
    return do.numpy(stream)


def fill(like: np.ndarray, value, *, pad: int = 0, stream=None) -> np.ndarray:
    """Upload `like` (a view: its layout is what gets filled), fill the view with `value`, download."""
    do = DeviceArray(like, stream=stream, pad_front=pad)
    d = make_desc(like.shape, [do])
    pattern = int.from_bytes(np.array(value, dtype=like.dtype).tobytes().ljust(8, b"\0"), "little")
    check(lib().twg_fill(byref(d), like.itemsize, pattern, do.ptr, stream))
    flat = do.buf.download(like.dtype, do.root_size, stream, offset_bytes=do.pad)
    return flat


def masked_select(x: np.ndarray, mask: np.ndarray, *, pad: int = 0, stream=None, return_status: bool = False):
    if mask.dtype != np.bool_:
        raise RuntimeError("masked_select: expected BoolTensor for mask")
    shape = np.broadcast_shapes(x.shape, mask.shape)
    dx = DeviceArray(x, stream=stream, pad_front=pad)
    dm = DeviceArray(mask.view(np.uint8), stream=stream, pad_front=pad)
    d = make_desc(shape, [dx, dm])
    n = int(d.numel)
    out = DeviceBuffer(max(4 * n, 4), stream=stream)
    result = DeviceBuffer(16, stream=stream)
    ws_bytes = lib().twg_masked_select_workspace_bytes(n)
    ws = DeviceBuffer(ws_bytes, stream=stream)
    check(lib().twg_masked_select_f32(byref(d), dx.ptr, dm.ptr, out.ptr, result.ptr, ws.ptr, ws_bytes, stream))
    k, status = (int(v) for v in result.download(np.int64, 2, stream))
    if return_status:
        return out.download(np.float32, max(k, 0), stream), status
    if status != 0:
        raise TwgError(status, "masked_select: the device-side scan reported an error")
    return out.download(np.float32, k, stream)


def fused_compile(instrs) -> int:
    arr = (FusedInstr * len(instrs))(*[FusedInstr(*i) for i in instrs])
    handle = c_void_p()
    check(lib().twg_fused_compile(arr, len(instrs), byref(handle)))
    return handle.value


def fused_kind(handle: int) -> str:
    k = c_int()
    check(lib().twg_fused_kind(handle, byref(k)))
    return "aot" if k.value == 0 else "nvrtc"


def fused(instrs, inputs, out_dtypes, *, shape=None, stream=None):
    """Run a fused program on numpy inputs; returns (list of outputs, kind)."""
    handle = fused_compile(instrs)
    shape = tuple(shape) if shape is not None else np.broadcast_shapes(*[i.shape for i in inputs])
    dins = [DeviceArray(i.view(np.uint8) if i.dtype == np.bool_ else i, stream=stream) for i in inputs]
    douts = [DeviceArray.empty(shape, np.uint8 if np.dtype(t) == np.bool_ else t, stream=stream) for t in out_dtypes]
    ops = douts + dins
    d = make_desc(shape, ops)
    ptrs = (c_void_p * len(ops))(*[o.ptr for o in ops])
    check(lib().twg_fused_launch(handle, byref(d), ptrs, stream))
    outs = []
    for t, o in zip(out_dtypes, douts):
        a = o.numpy(stream)
        outs.append(a.view(np.bool_) if np.dtype(t) == np.bool_ else a)
    return outs, fused_kind(handle)


def fused_select(instrs, inputs, src: int, *, stream=None):
    """out = inputs[src][program(inputs)] with the mask as bits (dense f32 inputs); returns (values, kind)."""
    handle = fused_compile(instrs)
    n = int(inputs[0].size)
    dins = [DeviceArray(np.ascontiguousarray(i), stream=stream) for i in inputs]
    out = DeviceBuffer(max(4 * n, 4), stream=stream)
    result = DeviceBuffer(16, stream=stream)
    ws_bytes = lib().twg_fused_select_workspace_bytes(n)
    ws = DeviceBuffer(ws_bytes, stream=stream)
    ptrs = (c_void_p * len(dins))(*[d.ptr for d in dins])
    check(lib().twg_fused_select_f32(handle, src, n, ptrs, out.ptr, result.ptr, ws.ptr, ws_bytes, stream))
    k, status = (int(v) for v in result.download(np.int64, 2, stream))
    if status != 0:
        raise TwgError(status, "fused select: the device-side scan reported an error")
    return out.download(np.float32, k, stream), fused_kind(handle)


def predicate_bits(instrs, inputs, *, stream=None):
    """The predicate `instrs` over dense f32 inputs as a bool array, computed on the device as one
    bit per element (twg_fused_predicate_bits) and unpacked here."""
    handle = fused_compile(instrs)
    n = int(inputs[0].size)
    dins = [DeviceArray(np.ascontiguousarray(i), stream=stream) for i in inputs]
    nbytes = lib().twg_predicate_bits_bytes(n)
    bits = DeviceBuffer(max(nbytes, 16), stream=stream)
    ptrs = (c_void_p * len(dins))(*[d.ptr for d in dins])
    check(lib().twg_fused_predicate_bits(handle, n, ptrs, bits.ptr, stream))
    packed = bits.download(np.uint8, nbytes, stream)
    unpacked = np.unpackbits(packed, bitorder="little")
    assert not unpacked[n:].any(), "bits at and beyond numel must be zero"
    return unpacked[:n].astype(np.bool_)


def masked_select_bits(src, mask, *, stream=None):
    """masked_select of dense f32 `src` by a bool array handed over as bits (twg_masked_select_bits_f32)."""
    src = np.ascontiguousarray(src, dtype=np.float32).ravel()
    n = src.size
    nbytes = lib().twg_predicate_bits_bytes(n)
    packed = np.zeros(max(nbytes, 16), np.uint8)
    packed[:(n + 7) // 8] = np.packbits(np.asarray(mask, np.bool_).ravel(), bitorder="little")
    dsrc, dbits = DeviceArray(src if n else np.zeros(4, np.float32), stream=stream), DeviceArray(packed, stream=stream)
    out = DeviceBuffer(max(4 * n, 4), stream=stream)
    result = DeviceBuffer(16, stream=stream)
    ws_bytes = lib().twg_masked_select_workspace_bytes(n)
    ws = DeviceBuffer(max(ws_bytes, 256), stream=stream)
    check(lib().twg_masked_select_bits_f32(dsrc.ptr, dbits.ptr, n, out.ptr, result.ptr, ws.ptr, ws_bytes, stream))
    k, status = (int(v) for v in result.download(np.int64, 2, stream))
    if status != 0:
        raise TwgError(status, "masked_select by bits: the device-side scan reported an error")
    return out.download(np.float32, k, stream)


# the benchmark's chain  m = (relu(silu(a + b) + c) == 0) & (a != 0)  as the compile backend emits it
CHAIN_MASK_PROGRAM = [
    (F_INPUT_F32, 0, 0, 0.0), (F_INPUT_F32, 1, 0, 0.0), (F_INPUT_F32, 2, 0, 0.0),
    (F_ADD, 0, 1, 1.0), (F_SILU, 3, 0, 0.0), (F_ADD, 4, 2, 1.0), (F_RELU, 5, 0, 0.0),
    (F_CONST_F32, 0, 0, 0.0), (F_EQ, 6, 7, 0.0), (F_CONST_F32, 0, 0, 0.0), (F_NE, 0, 9, 0.0),
    (F_AND, 8, 10, 0.0), (F_OUTPUT, 11, 0, 0.0),
]
