"""`torch.webgpu`: the device module of the webgpu backend.

The reference exports `is_initialized` and `current_device` only
(python/torch_webgpu/webgpu/__init__.py:1-9).  Current PyTorch also asks a device module for
`is_available` (torch.accelerator / dynamo), and a multi-device backend needs device selection,
synchronisation and allocator statistics, so those are here too.
"""
from __future__ import annotations

import contextlib

import torch

from .. import _C

__all__ = [
    "is_initialized", "is_available", "current_device", "device_count", "set_device", "device",
    "synchronize", "memory_stats", "memory_allocated", "memory_reserved", "max_memory_allocated",
    "reset_peak_memory_stats", "empty_cache", "current_stream_handle", "launch_count",
]


def is_initialized() -> bool:
    return True


def is_available() -> bool:
    return _C.device_count() > 0


def _is_in_bad_fork() -> bool:
    return False


def device_count() -> int:
    return _C.device_count()


def current_device() -> int:
    return _C.current_device()


def _index(device) -> int:
    if device is None:
        return _C.current_device()
    if isinstance(device, int):
        return device
    d = torch.device(device)
    return _C.current_device() if d.index is None else d.index


def set_device(device) -> None:
    _C.set_device(_index(device))


@contextlib.contextmanager
def device(device):
    prev = _C.current_device()
    _C.set_device(_index(device))
    try:
        yield
    finally:
        _C.set_device(prev)


def synchronize(device=None) -> None:
    _C.synchronize(_index(device))


def memory_stats(device=None) -> dict:
    return dict(_C.memory_stats(_index(device)))


def memory_allocated(device=None) -> int:
    return memory_stats(device)["allocated_bytes"]


def memory_reserved(device=None) -> int:
    return memory_stats(device)["reserved_bytes"]


def max_memory_allocated(device=None) -> int:
    return memory_stats(device)["peak_allocated_bytes"]


def reset_peak_memory_stats(device=None) -> None:
    _C.reset_peak_memory_stats(_index(device))


def empty_cache() -> None:
    _C.empty_cache()


def current_stream_handle(device=None) -> int:
    """cudaStream_t of the calling thread's current stream on `device`, as an integer."""
    return _C.current_stream_handle(_index(device))


def launch_count() -> int:
    """Kernels launched by the library since the last reset."""
    return _C.launch_count()


def manual_seed_all(seed: int) -> None:  # the backend has no random ops; accepted for API parity
    return None
