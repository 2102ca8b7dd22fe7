"""Batch sharding of the op path over several GPUs (one process per GPU).

Every op on the path is elementwise over independent elements, and masked_select over a
batch-major tensor is the order-preserving concatenation of the per-shard results.  So a batch is
cut into contiguous blocks of its leading dimension, each rank runs the kernels on its block with
no data-path communication, and the only exchange is one int64 per rank - the number of elements
its masked_select produced - from which every rank derives the offset of its segment in the
global (concatenated) result.  The reference has no multi-device support
(`webgpu_device_count = 1`, csrc/core/webgpu_device_guard.h:9).

Three transports for that exchange:

* `PeerStoreExchange` - the library's own kernels store the counts into every peer's mailbox
  over NVLink and the host polls pinned memory (twg_exchange_*): no collective launch per step.
* `NcclExchange` - ncclAllGather through the C ABI (twg_comm_*, twg_allgather_i64).
* `allgather_counts` - torch.distributed, for hosts that already run a process group (and for
  the gloo tests on CPU).

`Rendezvous` is the host-side channel the first two need once, at start-up, to pass the NCCL
unique id and the mailbox handles around: a key-value store reached through the same
MASTER_ADDR / MASTER_PORT environment a torchrun launch provides.
"""
from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world_size: int) -> tuple[int, int]:
    """Half-open range [lo, hi) of the leading dimension owned by `rank`.

    Blocks are contiguous and as even as possible; the first `total % world_size` ranks get one
    extra item, so any world size works, including ones larger than the batch.
    """
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} is outside a world of {world_size}")
    base, extra = divmod(int(total), world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo, hi


def exclusive_offsets(counts: Sequence[int]) -> list[int]:
    """Global output offset of each rank's segment: the exclusive prefix sum of the counts."""
    out, acc = [], 0
    for c in counts:
        out.append(acc)
        acc += int(c)
    return out


def allgather_counts(local_count: int, device: torch.device | str = "cpu", group=None) -> list[int]:
    """All-gather one int64 per rank.  With the NCCL backend `device` must be the rank's CUDA
    device (8 bytes per rank cross NVLink); with gloo it is the CPU."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [int(local_count)]
    world = dist.get_world_size(group)
    mine = torch.tensor([int(local_count)], dtype=torch.int64, device=device)
    gathered = torch.empty(world, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    return [int(v) for v in gathered.cpu().tolist()]


def global_segment(local_count: int, device: torch.device | str = "cpu", group=None) -> tuple[int, int, list[int]]:
    """(offset of this rank's segment, total selected elements, all counts)."""
    counts = allgather_counts(local_count, device, group)
    rank = dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0
    offsets = exclusive_offsets(counts)
    return offsets[rank], sum(counts), counts


# ---------------------------------------------------------------------------------------------
# host-side channel for start-up data
# ---------------------------------------------------------------------------------------------
class Rendezvous:
    """Key-value channel between the ranks of one job, used only at start-up (and for
    host-side barriers outside timed regions).  `store` is any torch.distributed Store."""

    def __init__(self, store, rank: int, world: int):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self._round = 0

    @classmethod
    def from_env(cls) -> "Rendezvous":
        """RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT as torchrun exports them.  Under torchrun
        the launcher already serves the store on that port and the ranks connect as clients."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        if world == 1:
            return cls(None, 0, 1)
        store, rank, world = next(iter(dist.rendezvous("env://", rank=rank, world_size=world)))
        return cls(store, rank, world)

    def share(self, payload: bytes) -> list[bytes]:
        """Every rank contributes `payload`; every rank gets all of them in rank order."""
        if self.world == 1:
            return [bytes(payload)]
        self._round += 1
        self.store.set(f"twg/share/{self._round}/{self.rank}", bytes(payload))
        return [bytes(self.store.get(f"twg/share/{self._round}/{r}")) for r in range(self.world)]

    def broadcast(self, payload: bytes | None, root: int = 0) -> bytes:
        if self.world == 1:
            return bytes(payload or b"")
        self._round += 1
        key = f"twg/bcast/{self._round}"
        if self.rank == root:
            self.store.set(key, bytes(payload or b""))
        return bytes(self.store.get(key))

    def barrier(self) -> None:
        """Host-side barrier (milliseconds; not for timed regions)."""
        self.share(b"")


# ---------------------------------------------------------------------------------------------
# the count exchange through the C ABI
# ---------------------------------------------------------------------------------------------
class PeerStoreExchange:
    """twg_exchange_*: counts travel as plain stores into every peer's mailbox.

    `ring` bounds how far a rank may run ahead: sequence number s may be published only after
    wait(s - ring // 2) has returned on this rank.
    """

    kind = "peer stores"

    def __init__(self, abi, rank: int, world: int, ring: int = 8):
        self.abi, self.rank, self.world, self.ring = abi, int(rank), int(world), int(ring)
        handle = ctypes.c_void_p()
        abi.check(abi.lib().twg_exchange_create(self.rank, self.world, self.ring, ctypes.byref(handle)))
        self.handle = handle
        self._counts = (ctypes.c_int64 * self.world)()
        self._status = (ctypes.c_int64 * self.world)()
        self._offset, self._total = ctypes.c_int64(), ctypes.c_int64()

    def export_handle(self) -> bytes:
        buf = ctypes.create_string_buffer(64)
        self.abi.check(self.abi.lib().twg_exchange_handle(self.handle, buf))
        return buf.raw

    def connect(self, handles: Sequence[bytes]) -> None:
        """handles[r] = export_handle() of rank r (other processes)."""
        for r, h in enumerate(handles):
            if r != self.rank:
                self.abi.check(self.abi.lib().twg_exchange_connect_ipc(self.handle, r, ctypes.c_char_p(h)))

    def connect_local(self, peers: Sequence["PeerStoreExchange"]) -> None:
        """All ranks live in this process (one object per device)."""
        for r, p in enumerate(peers):
            self.abi.check(self.abi.lib().twg_exchange_connect_local(self.handle, r, p.handle))

    def publish(self, seq: int, result_ptr: int, stream) -> None:
        self.abi.check(self.abi.lib().twg_exchange_publish(self.handle, seq, result_ptr, stream))

    def masked_select_publish(self, seq: int, desc, src_ptr: int, mask_ptr: int, out_ptr: int, result_ptr: int,
                              ws_ptr: int, ws_bytes: int, stream) -> None:
        """masked_select whose last chunk publishes this rank's count itself (one launch less)."""
        self.abi.check(self.abi.lib().twg_masked_select_f32_publish(
            ctypes.byref(desc), src_ptr, mask_ptr, out_ptr, result_ptr, ws_ptr, ws_bytes, self.handle, seq, stream))

    def select_bits_publish(self, seq: int, src_ptr: int, bits_ptr: int, n: int, out_ptr: int, result_ptr: int,
                            ws_ptr: int, ws_bytes: int, stream) -> None:
        """The compaction by a bit mask (twg_masked_select_bits_f32) publishing its count the same way."""
        self.abi.check(self.abi.lib().twg_masked_select_bits_f32_publish(
            src_ptr, bits_ptr, n, out_ptr, result_ptr, ws_ptr, ws_bytes, self.handle, seq, stream))

    def fused_select_publish(self, seq: int, program, src_index: int, n: int, in_ptrs, out_ptr: int, result_ptr: int,
                             ws_ptr: int, ws_bytes: int, stream) -> None:
        """Predicate bits + that compaction as one call (twg_fused_select_f32)."""
        self.abi.check(self.abi.lib().twg_fused_select_f32_publish(
            program, src_index, n, in_ptrs, out_ptr, result_ptr, ws_ptr, ws_bytes, self.handle, seq, stream))

    def collect(self, seq: int, stream) -> None:
        self.abi.check(self.abi.lib().twg_exchange_collect(self.handle, seq, stream))

    def wait(self, seq: int, timeout_ms: int = 20000) -> tuple[list[int], int, int]:
        """(counts of every rank, this rank's offset, total); raises on a device status."""
        self.abi.check(self.abi.lib().twg_exchange_wait(self.handle, seq, self._counts, self._status,
                                                        ctypes.byref(self._offset), ctypes.byref(self._total), timeout_ms))
        return list(self._counts), int(self._offset.value), int(self._total.value)

    def set_timeout_ns(self, ns: int) -> None:
        self.abi.check(self.abi.lib().twg_exchange_set_timeout_ns(self.handle, ns))

    def close(self) -> None:
        if self.handle:
            self.abi.check(self.abi.lib().twg_exchange_destroy(self.handle))
            self.handle = None


class NcclExchange:
    """twg_comm_* / twg_allgather_i64: the same exchange as one ncclAllGather per step followed by
    a 16-byte-per-rank copy to pinned memory; the host waits on an event."""

    kind = "ncclAllGather"

    def __init__(self, abi, rank: int, world: int, unique_id: bytes, device: int, ring: int = 8):
        self.abi, self.rank, self.world, self.ring = abi, int(rank), int(world), int(ring)
        L = abi.lib()
        comm = ctypes.c_void_p()
        abi.check(L.twg_comm_init_rank(ctypes.c_char_p(unique_id), self.rank, self.world, ctypes.byref(comm)))
        self.comm = comm
        self.dev = [abi.DeviceBuffer(16 * self.world, device) for _ in range(self.ring)]
        self.host = []
        for _ in range(self.ring):
            p = ctypes.c_void_p()
            abi.check(L.twg_host_alloc_pinned(ctypes.byref(p), 16 * self.world))
            self.host.append(p)
        self.events = []
        for _ in range(self.ring):
            e = ctypes.c_void_p()
            abi.check(L.twg_event_create(ctypes.byref(e)))
            self.events.append(e)
        self._pending: dict[int, int] = {}

    @staticmethod
    def make_unique_id(abi) -> bytes:
        buf = ctypes.create_string_buffer(128)
        abi.check(abi.lib().twg_comm_unique_id(buf))
        return buf.raw

    def allgather(self, send_ptr: int, recv_ptr: int, n: int, stream) -> None:
        self.abi.check(self.abi.lib().twg_allgather_i64(self.comm, send_ptr, recv_ptr, n, stream))

    def publish(self, seq: int, result_ptr: int, stream) -> None:
        self._pending[seq] = result_ptr

    def masked_select_publish(self, seq: int, desc, src_ptr: int, mask_ptr: int, out_ptr: int, result_ptr: int,
                              ws_ptr: int, ws_bytes: int, stream) -> None:
        self.abi.check(self.abi.lib().twg_masked_select_f32(ctypes.byref(desc), src_ptr, mask_ptr, out_ptr, result_ptr,
                                                            ws_ptr, ws_bytes, stream))
        self.publish(seq, result_ptr, stream)

    def select_bits_publish(self, seq: int, src_ptr: int, bits_ptr: int, n: int, out_ptr: int, result_ptr: int,
                            ws_ptr: int, ws_bytes: int, stream) -> None:
        self.abi.check(self.abi.lib().twg_masked_select_bits_f32(src_ptr, bits_ptr, n, out_ptr, result_ptr, ws_ptr, ws_bytes,
                                                                stream))
        self.publish(seq, result_ptr, stream)

    def fused_select_publish(self, seq: int, program, src_index: int, n: int, in_ptrs, out_ptr: int, result_ptr: int,
                             ws_ptr: int, ws_bytes: int, stream) -> None:
        self.abi.check(self.abi.lib().twg_fused_select_f32(program, src_index, n, in_ptrs, out_ptr, result_ptr, ws_ptr,
                                                           ws_bytes, stream))
        self.publish(seq, result_ptr, stream)

    def collect(self, seq: int, stream) -> None:
        L, slot = self.abi.lib(), seq % self.ring
        self.allgather(self._pending.pop(seq), self.dev[slot].ptr, 2, stream)
        self.abi.check(L.twg_memcpy_d2h(self.host[slot], self.dev[slot].ptr, 16 * self.world, stream, 0))
        self.abi.check(L.twg_event_record(self.events[slot], stream))

    def wait(self, seq: int, timeout_ms: int = 20000) -> tuple[list[int], int, int]:
        slot = seq % self.ring
        self.abi.check(self.abi.lib().twg_event_sync(self.events[slot]))
        flat = (ctypes.c_int64 * (2 * self.world)).from_address(self.host[slot].value)
        counts, status = list(flat[0::2]), list(flat[1::2])
        if any(status):
            raise self.abi.TwgError(int(min(status)), f"masked_select reported device status {status}")
        return counts, sum(counts[:self.rank]), sum(counts)

    def close(self) -> None:
        L = self.abi.lib()
        if self.comm:
            self.abi.check(L.twg_comm_destroy(self.comm))
            self.comm = None
        for p in self.host:
            L.twg_host_free_pinned(p)
        for e in self.events:
            L.twg_event_destroy(e)
        self.host, self.events, self.dev = [], [], []
