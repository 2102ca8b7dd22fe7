"""The count exchange of the batch-sharded path on real GPUs, through the C ABI.

One GPU is enough for the protocol itself: several ranks' exchange objects live on the same device
and every publish is enqueued before the collects that wait for it, on one stream, so no kernel
ever waits for a launch that is not already complete.  The bounded wait is tested with a rank that
never publishes (a flag nothing sets): the collect kernel returns TWG_ERR_TIMEOUT after its time
limit and the context stays usable.  With two or more GPUs the batch-sharded chain is run on two
devices and the concatenated shards are compared with the single-GPU result and the CPU oracle.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

from oracle import oracle
from util import assert_bit_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def abi():
    from torch_webgpu import abi as _abi
    assert _abi.device_count() >= 1, "no CUDA device visible"
    return _abi


def result_buffer(abi, count: int, status: int = 0, device: int = 0):
    buf = abi.DeviceBuffer(16, device)
    buf.upload(np.array([count, status], dtype=np.int64))
    return buf


def test_single_rank_exchange_round_trips_counts(abi):
    from torch_webgpu.sharding import PeerStoreExchange
    x = PeerStoreExchange(abi, 0, 1, ring=4)
    try:
        for seq in range(1, 12):                      # wraps the ring several times
            res = result_buffer(abi, 1000 + seq)
            x.publish(seq, res.ptr, None)
            x.collect(seq, None)
            counts, offset, total = x.wait(seq, timeout_ms=5000)
            assert (counts, offset, total) == ([1000 + seq], 0, 1000 + seq)
        rec = ctypes.c_void_p()
        abi.check(abi.lib().twg_exchange_gathered(x.handle, 11, ctypes.byref(rec)))
        dev = (ctypes.c_int64 * 4)()
        abi.check(abi.lib().twg_memcpy_d2h(dev, rec, 32, None, 1))
        assert list(dev) == [1011, 0, 0, 1011]        # count, status, offset, total
    finally:
        x.close()


def test_three_ranks_on_one_device_exchange_in_stream_order(abi):
    """Ranks 0..2 share a device and a stream: all publishes of a step are enqueued before its
    collects, so every collect finds its mailbox complete."""
    from torch_webgpu.sharding import PeerStoreExchange
    world = 3
    xs = [PeerStoreExchange(abi, r, world, ring=4) for r in range(world)]
    try:
        for x in xs:
            x.connect_local(xs)
        for seq in range(1, 10):
            mine = [7 * seq + r for r in range(world)]
            bufs = [result_buffer(abi, mine[r]) for r in range(world)]
            for r, x in enumerate(xs):
                x.publish(seq, bufs[r].ptr, None)
            for x in xs:
                x.collect(seq, None)
            for r, x in enumerate(xs):
                counts, offset, total = x.wait(seq, timeout_ms=5000)
                assert counts == mine and offset == sum(mine[:r]) and total == sum(mine)
    finally:
        for x in xs:
            x.close()


@pytest.mark.parametrize("n", [0, 5, 4096 * 3 + 17, (1 << 22) + 3])
def test_compaction_publishes_its_own_count(abi, n):
    """twg_masked_select_f32_publish: the compaction's last chunk writes the mailboxes itself (the
    publish kernel is only used for empty inputs and for layouts of the one-tile-per-CTA kernel)."""
    from torch_webgpu.sharding import PeerStoreExchange
    L = abi.lib()
    world = 3
    xs = [PeerStoreExchange(abi, r, world, ring=4) for r in range(world)]
    try:
        for x in xs:
            x.connect_local(xs)
        rng = np.random.default_rng(n + 1)
        for seq in (1, 2):
            expect, keep = [], []
            for r, x in enumerate(xs):
                src = rng.standard_normal(n).astype(np.float32)
                mask = rng.random(n) < (0.2 + 0.3 * r)
                dsrc, dmask = abi.DeviceArray(src), abi.DeviceArray(mask.view(np.uint8))
                out, res = abi.DeviceBuffer(max(4 * n, 4)), abi.DeviceBuffer(16)
                ws_bytes = L.twg_masked_select_workspace_bytes(n)
                ws = abi.DeviceBuffer(max(ws_bytes, 256))
                d = abi.IterDesc()
                abi.check(L.twg_iter_contiguous(ctypes.byref(d), 2, n))
                L.twg_reset_launch_count()
                x.masked_select_publish(seq, d, dsrc.ptr, dmask.ptr, out.ptr, res.ptr, ws.ptr, ws_bytes, None)
                assert L.twg_launch_count() == 2        # clear + compaction, or clear + publish for the empty input
                expect.append(oracle.masked_select(src, mask))
                keep.append((dsrc, dmask, out, res, ws))
            for x in xs:
                x.collect(seq, None)
            for r, x in enumerate(xs):
                counts, offset, total = x.wait(seq, timeout_ms=5000)
                assert counts == [e.size for e in expect] and offset == sum(counts[:r]) and total == sum(counts)
                assert_bit_equal(keep[r][2].download(np.float32, counts[r]), expect[r], f"rank {r} values")
    finally:
        for x in xs:
            x.close()


@pytest.mark.parametrize("n", [0, 129, 4096 * 5 + 1, (1 << 22) + 3])
def test_fused_select_publishes_its_own_count(abi, n):
    """twg_fused_select_f32_publish: predicate bits, then the compaction whose last chunk writes the
    mailboxes; same counts and values as the byte mask followed by masked_select."""
    from torch_webgpu.sharding import PeerStoreExchange
    L = abi.lib()
    world = 2
    xs = [PeerStoreExchange(abi, r, world, ring=4) for r in range(world)]
    program = abi.fused_compile(abi.CHAIN_MASK_PROGRAM)
    try:
        for x in xs:
            x.connect_local(xs)
        rng = np.random.default_rng(n + 7)
        expect, keep = [], []
        for r, x in enumerate(xs):
            a, b, c = (rng.uniform(-3, 3, n).astype(np.float32) for _ in range(3))
            a[::4 + r] = 0.0
            (m,), _ = abi.fused(abi.CHAIN_MASK_PROGRAM, [a, b, c], [np.bool_]) if n else ((np.zeros(0, np.bool_),), None)
            ins = [abi.DeviceArray(v) if n else abi.DeviceBuffer(16) for v in (a, b, c)]
            out, res = abi.DeviceBuffer(max(4 * n, 4)), abi.DeviceBuffer(16)
            ws_bytes = L.twg_fused_select_workspace_bytes(n)
            ws = abi.DeviceBuffer(max(ws_bytes, 256))
            in_ptrs = (ctypes.c_void_p * 3)(*[i.ptr for i in ins])
            L.twg_reset_launch_count()
            x.fused_select_publish(1, program, 0, n, in_ptrs, out.ptr, res.ptr, ws.ptr, ws_bytes, None)
            assert L.twg_launch_count() == (3 if n else 2)   # bits + clear + compaction; clear + publish when empty
            expect.append(oracle.masked_select(a, m))
            keep.append((ins, out, res, ws))
        for x in xs:
            x.collect(1, None)
        for r, x in enumerate(xs):
            counts, offset, total = x.wait(1, timeout_ms=5000)
            assert counts == [e.size for e in expect] and offset == sum(counts[:r]) and total == sum(counts)
            assert_bit_equal(keep[r][1].download(np.float32, counts[r]), expect[r], f"rank {r} values")
    finally:
        for x in xs:
            x.close()


def test_a_device_status_travels_with_the_count(abi):
    from torch_webgpu.sharding import PeerStoreExchange
    xs = [PeerStoreExchange(abi, r, 2, ring=2) for r in range(2)]
    try:
        for x in xs:
            x.connect_local(xs)
        bufs = [result_buffer(abi, 5, 0), result_buffer(abi, 6, abi.TWG_ERR_TIMEOUT)]
        for r, x in enumerate(xs):
            x.publish(1, bufs[r].ptr, None)
        xs[0].collect(1, None)
        with pytest.raises(abi.TwgError) as err:
            xs[0].wait(1, timeout_ms=5000)
        assert err.value.code == abi.TWG_ERR_TIMEOUT
        statuses = (ctypes.c_int64 * 2)()
        rc = abi.lib().twg_exchange_wait(xs[0].handle, 1, None, statuses, None, None, 5000)
        assert rc == abi.TWG_ERR_TIMEOUT and list(statuses) == [0, abi.TWG_ERR_TIMEOUT]
    finally:
        for x in xs:
            x.close()


def test_collect_gives_up_after_its_time_limit_when_a_rank_never_publishes(abi):
    """Rank 1 never publishes.  Rank 0's collect kernel waits for the 50 ms it is given, reports
    TWG_ERR_TIMEOUT for rank 1 and returns; the device keeps working afterwards."""
    from torch_webgpu.sharding import PeerStoreExchange
    xs = [PeerStoreExchange(abi, r, 2, ring=2) for r in range(2)]
    try:
        for x in xs:
            x.connect_local(xs)
        xs[0].set_timeout_ns(50_000_000)
        res = result_buffer(abi, 42)
        xs[0].publish(1, res.ptr, None)
        xs[0].collect(1, None)
        counts = (ctypes.c_int64 * 2)()
        statuses = (ctypes.c_int64 * 2)()
        rc = abi.lib().twg_exchange_wait(xs[0].handle, 1, counts, statuses, None, None, 10000)
        assert rc == abi.TWG_ERR_TIMEOUT
        assert list(counts) == [42, 0] and list(statuses) == [0, abi.TWG_ERR_TIMEOUT]
        # the host-side wait has its own limit: a sequence nobody collects
        rc = abi.lib().twg_exchange_wait(xs[0].handle, 2, None, None, None, None, 20)
        assert rc == abi.TWG_ERR_TIMEOUT and b"did not complete" in abi.lib().twg_last_error()
        x = np.linspace(-3, 3, 1000, dtype=np.float32)
        assert_bit_equal(abi.unary("relu", x), oracle.unary("relu", x), "relu after the timeout")
    finally:
        for x in xs:
            x.close()


def test_nccl_allgather_through_the_c_abi_on_one_rank(abi):
    from torch_webgpu.sharding import NcclExchange
    uid = NcclExchange.make_unique_id(abi)
    assert len(uid) == 128 and any(uid)
    ex = NcclExchange(abi, 0, 1, uid, 0, ring=2)
    try:
        res = result_buffer(abi, 99)
        ex.publish(1, res.ptr, None)
        ex.collect(1, None)
        assert ex.wait(1) == ([99], 0, 99)
        send = abi.DeviceBuffer(24)
        send.upload(np.array([3, 1, 4], dtype=np.int64))
        recv = abi.DeviceBuffer(24)
        ex.allgather(send.ptr, recv.ptr, 3, None)
        assert list(recv.download(np.int64, 3)) == [3, 1, 4]
    finally:
        ex.close()


def _chain_shard(abi, dev: int, a, b, c):
    """Fused chain + compaction of one shard on device `dev`; returns (selected values, result buffer)."""
    L = abi.lib()
    abi.check(L.twg_set_device(dev))
    n = a.size
    bufs = [abi.DeviceBuffer(4 * n, dev) for _ in range(3)]
    for buf, h in zip(bufs, (a, b, c)):
        buf.upload(h.reshape(-1))
    mask, out, res = abi.DeviceBuffer(n, dev), abi.DeviceBuffer(4 * n, dev), abi.DeviceBuffer(16, dev)
    ws_bytes = L.twg_masked_select_workspace_bytes(n)
    ws = abi.DeviceBuffer(ws_bytes, dev)
    prog = abi.fused_compile(abi.CHAIN_MASK_PROGRAM)
    d4, d2 = abi.IterDesc(), abi.IterDesc()
    abi.check(L.twg_iter_contiguous(ctypes.byref(d4), 4, n))
    abi.check(L.twg_iter_contiguous(ctypes.byref(d2), 2, n))
    ptrs = (ctypes.c_void_p * 4)(mask.ptr, bufs[0].ptr, bufs[1].ptr, bufs[2].ptr)
    abi.check(L.twg_fused_launch(prog, ctypes.byref(d4), ptrs, None))
    abi.check(L.twg_masked_select_f32(ctypes.byref(d2), bufs[0].ptr, mask.ptr, out.ptr, res.ptr, ws.ptr, ws_bytes, None))
    return out, res, mask, (bufs, ws)


def test_two_gpu_shards_concatenate_to_the_single_gpu_result(abi):
    """Configuration 5 on a reduced batch (4 slabs of [1024,1024]): shards on devices 0 and 1,
    counts exchanged with peer stores between the two GPUs, segments placed at the exchanged
    offsets == the one-GPU result == the CPU oracle, bit for bit."""
    if abi.device_count() < 2:
        pytest.skip("needs two GPUs")
    from torch_webgpu.sharding import PeerStoreExchange, shard_range
    L = abi.lib()
    rng = np.random.default_rng(4)
    a, b, c = (rng.standard_normal((4, 1024, 1024)).astype(np.float32) for _ in range(3))
    a[1, ::5] = 0.0
    # one GPU
    out1, res1, mask1, keep1 = _chain_shard(abi, 0, a, b, c)
    k1 = int(res1.download(np.int64, 2)[0])
    single = out1.download(np.float32, k1)
    gpu_mask = mask1.download(np.uint8, a.size).astype(bool).reshape(a.shape)
    ref = oracle.masked_select(a.reshape(-1), gpu_mask.reshape(-1))
    assert_bit_equal(single, ref, "single-GPU chain vs oracle (given the GPU's mask)")
    y_ref, m_ref = oracle.chain_mask(a, b, c, want_y=True)
    flipped = gpu_mask != m_ref
    assert flipped.sum() <= 4 and np.all(np.abs(y_ref[flipped]) < 1e-6)
    # two GPUs
    xs = []
    for r in range(2):
        abi.check(L.twg_set_device(r))
        xs.append(PeerStoreExchange(abi, r, 2, ring=4))
    try:
        for r, x in enumerate(xs):
            abi.check(L.twg_set_device(r))
            x.connect_local(xs)
        shards = []
        for r in range(2):
            lo, hi = shard_range(4, r, 2)
            shards.append(_chain_shard(abi, r, a[lo:hi], b[lo:hi], c[lo:hi]))
        # every publish is enqueued (each on its own device) before any collect
        for r, x in enumerate(xs):
            abi.check(L.twg_set_device(r))
            x.publish(1, shards[r][1].ptr, None)
        for r, x in enumerate(xs):
            abi.check(L.twg_set_device(r))
            x.collect(1, None)
        combined = np.empty(k1, np.float32)
        seen_total = set()
        for r, x in enumerate(xs):
            abi.check(L.twg_set_device(r))
            counts, offset, total = x.wait(1, timeout_ms=10000)
            seen_total.add(total)
            combined[offset:offset + counts[r]] = shards[r][0].download(np.float32, counts[r])
        assert seen_total == {k1}
        assert_bit_equal(combined, single, "two-GPU shards vs the single-GPU result")
    finally:
        for r, x in enumerate(xs):
            abi.check(L.twg_set_device(r))
            x.close()
        abi.check(L.twg_set_device(0))
