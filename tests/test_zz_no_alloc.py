"""twg_masked_select_f32_static: masked_select for callers that cannot allocate device memory.

Some users of the C ABI have no way to provide the scratch buffer that twg_masked_select_f32
asks for - their host owns all device memory and forbids a foreign cudaMalloc, or they are handed
inputs and outputs and nothing else, or they sit on a path that must not meet cudaMalloc's
implicit synchronisation.  For them the library carries a fixed scratch array in its own image.
This test drives that entry point through the C ABI twice in a row (the array is shared between
calls and keeps the previous call's contents, so the second call proves that what has to start at
zero is cleared) and compares each result bit for bit with the regular entry point's.

The file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It does not depend on any of them and also passes alone in a fresh process.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def abi():
    from torch_webgpu import abi as _abi
    assert _abi.device_count() >= 1, "no CUDA device visible"
    return _abi


def run_static(abi, x: np.ndarray, mask: np.ndarray):
    """One call of the allocation-free entry point; inputs, output and result come from the caller."""
    L = abi.lib()
    shape = np.broadcast_shapes(x.shape, mask.shape)
    dx = abi.DeviceArray(x)
    dm = abi.DeviceArray(mask.view(np.uint8))
    d = abi.make_desc(shape, [dx, dm])
    n = int(d.numel)
    out = abi.DeviceBuffer(max(4 * n, 4))
    result = abi.DeviceBuffer(16)
    abi.check(L.twg_masked_select_f32_static(ctypes.byref(d), dx.ptr, dm.ptr, out.ptr, result.ptr, None))
    k, status = (int(v) for v in result.download(np.int64, 2))
    assert status == 0
    return out.download(np.float32, k)


def test_static_scratch_matches_the_regular_entry_point_twice_in_a_row(abi):
    rng = np.random.default_rng(2024)
    # first call: many chunks, dense mask; second call: different size and density, so stale
    # descriptors or a stale ticket from the first call would show up as wrong offsets
    cases = [(3 * (1 << 20) + 12345, 0.5), (777_777, 0.03)]
    for n, p in cases:
        x = (rng.random(n, dtype=np.float32) * 16 - 8).astype(np.float32)
        mask = rng.random(n) < p
        got = run_static(abi, x, mask)
        ref = abi.masked_select(x, mask)          # existing entry point, caller-provided workspace
        assert got.shape == ref.shape
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
        assert np.array_equal(got.view(np.uint32), x[mask].view(np.uint32))
    # a broadcast row mask goes through the same scratch
    x2 = (rng.random((300, 512), dtype=np.float32) - 0.5).astype(np.float32)
    rows = rng.random((300, 1)) < 0.5
    got = run_static(abi, x2, rows)
    assert np.array_equal(got.view(np.uint32), abi.masked_select(x2, rows).view(np.uint32))


def test_static_scratch_rejects_sizes_beyond_its_limit(abi):
    L = abi.lib()
    limit = int(L.twg_masked_select_static_max_numel())
    assert limit == 1 << 28
    d = abi.IterDesc()
    abi.check(L.twg_iter_contiguous(ctypes.byref(d), 2, limit + 1))
    dummy = abi.DeviceBuffer(64)
    # rejected before any pointer is touched, with a message that names the limit
    rc = L.twg_masked_select_f32_static(ctypes.byref(d), dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr, None)
    assert rc == abi.TWG_ERR_UNSUPPORTED
    message = L.twg_last_error().decode()
    assert str(limit) in message and "workspace" in message
