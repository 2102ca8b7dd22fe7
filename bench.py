#!/usr/bin/env python
"""Benchmark of the data-parallel op path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the reference's torch.compile configuration): a batch of 64 f32 [4096,4096] tensors
a, b, c ~ N(0,1); one step computes  y = relu(silu(a + b) + c),  m = (y == 0) & (a != 0)  and
masked_select(a, m)  over the whole batch.  The batch is cut by its leading dimension over the N
ranks (one process per GPU); the only exchange is one int64 count (and a status) per rank.
Total work is fixed, so scaling is "strong".  Inputs are synthetic: every [4096,4096] slab is
drawn with its own seed so that a rank can build its shard without generating the others.

One JSON line is printed by rank 0.  `value` is whole-job Gelem/s with the inputs resident in HBM;
`e2e` is the same metric through the public PyTorch API with pinned HOST buffers, upload of a, b, c
and read-back of the selected values inside the timed region.  `roofline` describes the dominant
kernel (the fused pointwise chain, which hands its mask to the compaction as one bit per element:
12.125 algorithmic bytes per element; 13 with --mask bytes); `ops` lists achieved GB/s of every
single op of the other configurations.  `--impl reference` times the CPU implementation of
the same path on the host cores instead.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO / "torch-webgpu_b200"))
sys.path.insert(0, str(REPO))

import numpy as np  # noqa: E402
import torch  # noqa: E402

BATCH, ROWS, COLS = 64, 4096, 4096   # --batch changes the first (a diagnostic, not the benchmark)
SLAB = ROWS * COLS
SEED = 4
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0   # the round figure for B200 HBM3e; every fraction is also reported against it
# Algorithmic bytes per element of the step's dominant kernel, the fused chain: read a, b, c
# (3 x 4 B) and write the mask - one bit per element (the default, --mask bits) or a bool tensor
# (--mask bytes).
CHAIN_BYTES_PER_ELEM = {"bits": 12.125, "bytes": 13.0}
# DRAM bytes that kernel moves per element (dram__bytes_read.sum + dram__bytes_write.sum of one ncu
# capture on 2^27 elements).  Constants taken from those captures, not measurements of this run:
# the traffic of a streaming kernel is proportional to its element count, so it is scaled to the
# elements of a launch.
CHAIN_DRAM_BYTES_PER_ELEM = {"bits": 12.07, "bytes": 12.89}
CHAIN_KERNEL = {"bits": "predicate_bits_kernel<AotChainMaskQuick> (fused chain, mask as bits: 12.125 B/elem)",
                "bytes": "pw_contig_kernel<AotChainMask> (fused chain, bool mask: 13 B/elem)"}


def slab_seed(tensor_id: int, batch_index: int) -> int:
    return SEED * 1_000_003 + tensor_id * BATCH + batch_index


def fill_shard(dst: torch.Tensor, tensor_id: int, lo: int, hi: int) -> None:
    """dst[i - lo] = N(0,1) slab i of tensor `tensor_id`, each slab from its own generator."""
    def one(i: int) -> None:
        g = torch.Generator().manual_seed(slab_seed(tensor_id, i))
        torch.randn(ROWS, COLS, generator=g, out=dst[i - lo])
    with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
        list(ex.map(one, range(lo, hi)))


def measured_peak() -> tuple[float, str]:
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clock and throttle-reason samples taken while the timed region runs (read-only NVML
    queries from a background thread every few milliseconds)."""
    REASONS = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40, "sw_power_cap": 0x4}

    def __init__(self, cuda_index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.stop_flag = False
        self.thread = None
        self.handle = None
        try:
            import pynvml
            self.nvml = pynvml
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(cuda_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.handle = None

    def _run(self) -> None:
        nv = self.nvml
        while not self.stop_flag:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                query = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                bits = int(query(self.handle))
                for name, bit in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self) -> None:
        if self.handle is None:
            return
        import threading
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=2)
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.samples:
            out["sm_mhz"] = statistics.median(self.samples)
        return out


# ---------------------------------------------------------------------------------------------
# CPU implementation of the path (oracle port) - cpu_baseline leg and the reference arm
# ---------------------------------------------------------------------------------------------
def cpu_chain_step(oracle, a: np.ndarray, b: np.ndarray, c: np.ndarray) -> int:
    m = oracle.chain_mask(a, b, c)
    return int(oracle.masked_select(a.reshape(-1), m.reshape(-1)).size)


def cpu_sample(nslabs: int) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    bufs = [torch.empty(nslabs, ROWS, COLS) for _ in range(3)]
    for t, buf in enumerate(bufs):
        fill_shard(buf, t, 0, nslabs)
    return tuple(x.numpy() for x in bufs)


def run_cpu_baseline(target_seconds: float = 12.0) -> dict:
    from oracle import oracle
    oracle.build()
    oracle.set_num_threads(os.cpu_count() or 1)
    a, b, c = cpu_sample(1)
    cpu_chain_step(oracle, a, b, c)  # warm-up
    t0 = time.perf_counter()
    cpu_chain_step(oracle, a, b, c)
    per_slab = max(time.perf_counter() - t0, 1e-4)
    nslabs = int(max(1, min(16, target_seconds / per_slab / 3)))
    if nslabs > 1:
        a, b, c = cpu_sample(nslabs)
    times = []
    for _ in range(3):
        t0 = time.perf_counter()
        cpu_chain_step(oracle, a, b, c)
        times.append(time.perf_counter() - t0)
    best = min(times)
    out = {"value": nslabs * SLAB / best / 1e9, "unit": "Gelem/s", "cores": oracle.num_threads(), "kind": "port",
           "sample": f"{nslabs} of {BATCH} [4096,4096] slabs of the chain (seeded like the GPU run), best of 3, "
                     f"C restatement with OpenMP on {oracle.num_threads()} threads"}
    # the same sample through the PyTorch CPU kernels the reference's fallback ops execute
    torch.set_num_threads(os.cpu_count() or 1)
    ta, tb, tc = (torch.from_numpy(x) for x in (a, b, c))
    def aten():
        y = torch.relu(torch.nn.functional.silu(ta + tb) + tc)
        m = torch.bitwise_and(torch.eq(y, 0), torch.ne(ta, 0))
        return torch.masked_select(ta, m)
    aten()
    t0 = time.perf_counter()
    aten()
    out["aten_cpu_gelem_s"] = nslabs * SLAB / (time.perf_counter() - t0) / 1e9
    out["cpu_model"] = cpu_model()
    out["ops_aten_cpu_gbs"] = aten_cpu_ops()
    return out


def cpu_model() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def aten_cpu_ops() -> dict:
    """The single ops on the host through PyTorch's CPU kernels (what the reference's fallback ops
    run): algorithmic GB/s on one [4096,4096] slab, best of 3 after a warm-up, all host threads."""
    g = torch.Generator().manual_seed(0)
    n = ROWS * COLS
    x, y = torch.randn(ROWS, COLS, generator=g), torch.randn(ROWS, COLS, generator=g)
    m1, m2 = x > 0, y > 0
    cases = {
        "add": (12 * n, lambda: torch.add(x, y)),
        "relu": (8 * n, lambda: torch.relu(x)),
        "silu": (8 * n, lambda: torch.nn.functional.silu(x)),
        "gelu_erf": (8 * n, lambda: torch.nn.functional.gelu(x)),
        "eq_tensor": (9 * n, lambda: torch.eq(x, y)),
        "ne_scalar": (5 * n, lambda: torch.ne(x, 0)),
        "bitwise_and_bool": (3 * n, lambda: torch.bitwise_and(m1, m2)),
        "masked_select_p0.5": (5 * n + 4 * int(m1.sum()), lambda: torch.masked_select(x, m1)),
    }
    out = {}
    for name, (nbytes, fn) in cases.items():
        fn()
        best = float("inf")
        for _ in range(3):
            t0 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t0)
        out[name] = round(nbytes / best / 1e9, 2)
    return out


def run_reference_arm(args) -> None:
    """The path on the host cores: the C restatement of the reference's CPU-side algorithm
    (its fallback ops are PyTorch CPU kernels; its shaders cannot run here)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    oracle.build()
    oracle.set_num_threads(os.cpu_count() or 1)
    nslabs = 2
    a, b, c = cpu_sample(nslabs)
    for _ in range(max(args.warmup, 1)):
        cpu_chain_step(oracle, a, b, c)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_chain_step(oracle, a, b, c)
    dt = time.perf_counter() - t0
    value = args.steps * nslabs * SLAB / dt / 1e9
    sample = (f"each step = {nslabs} of {BATCH} [4096,4096] slabs of the chain on the host cores, C restatement with "
              f"OpenMP on {oracle.num_threads()} threads (faster than the PyTorch CPU kernels the reference's fallback ops run)")
    line = {
        "impl": "reference", "metric": "Gelem/s of the compiled chain + masked_select", "value": value, "unit": "Gelem/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(args.gpus, 0), elements_per_step_timed=nslabs * SLAB,
                       note=f"each timed step processes {nslabs} of the {BATCH} slabs (a bounded sample of the workload); "
                            "the rate is per element and comparable, the step time is not"),
        "cpu_baseline": {"value": value, "unit": "Gelem/s", "cores": oracle.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "Gelem/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int, depth: int, mask: str = "bits") -> dict:
    calls = ("twg_fused_predicate_bits (the mask m as one bit per element) + twg_masked_select_bits_f32_publish" if mask == "bits"
             else "twg_fused_launch (m as a bool tensor) + twg_masked_select_f32_publish")
    cfg = {"workload": "cfg5: y=relu(silu(a+b)+c); m=(y==0)&(a!=0); masked_select(a,m) over 64 x f32[4096,4096]; "
                       f"`value` = C ABI calls {calls} + twg_exchange_collect per step, "
                       "`public_api` / `e2e` = the same through torch.compile(backend=webgpu_backend)",
           "global_batch": BATCH, "elements_per_step": BATCH * SLAB, "parallelism": f"batch-sharded x{n_gpus}",
           "l2": "inputs (>= 1.5 GiB per rank) are larger than the 126 MB L2; no flush needed"}
    if depth:
        cfg["pipelining"] = (f"every step ends with its counts on the host; the host collects the counts of step i while the "
                             f"stream already runs up to {depth - 1} later steps ({depth} sets of output buffers)")
    return cfg


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class Events:
    def __init__(self, abi, n: int):
        self.abi = abi
        self.ev = []
        for _ in range(n):
            e = ctypes.c_void_p()
            abi.check(abi.lib().twg_event_create(ctypes.byref(e)))
            self.ev.append(e)

    def record(self, i: int, stream) -> None:
        self.abi.check(self.abi.lib().twg_event_record(self.ev[i], stream))

    def elapsed(self, i: int, j: int) -> float:
        ms = ctypes.c_float()
        self.abi.check(self.abi.lib().twg_event_elapsed_ms(self.ev[i], self.ev[j], ctypes.byref(ms)))
        return float(ms.value)

    def sync(self, i: int) -> None:
        self.abi.check(self.abi.lib().twg_event_sync(self.ev[i]))


class Timing(float):
    """Median milliseconds of single calls (an event on either side of each call); the fastest
    sample rides along as .min_ms, and .batch_ms is the average over the same number of calls
    issued back to back between ONE pair of events - for kernels of a few tens of microseconds the
    two differ by the front-end gap that an event record in front of every launch exposes."""
    min_ms: float = 0.0
    batch_ms: float = 0.0


def time_op(abi, stream, fn, iters: int = 20, warmup: int = 3) -> Timing:
    """Median device time (ms) of fn() on `stream`, CUDA events around each call."""
    ev = Events(abi, 2 * iters)
    for _ in range(warmup):
        fn()
    for i in range(iters):
        ev.record(2 * i, stream)
        fn()
        ev.record(2 * i + 1, stream)
    abi.check(abi.lib().twg_stream_sync(stream))
    samples = [ev.elapsed(2 * i, 2 * i + 1) for i in range(iters)]
    t = Timing(statistics.median(samples))
    t.min_ms = min(samples)
    ev.record(0, stream)
    for _ in range(iters):
        fn()
    ev.record(1, stream)
    abi.check(abi.lib().twg_stream_sync(stream))
    t.batch_ms = ev.elapsed(0, 1) / iters
    return t


def per_op_table(abi, stream, peak: float) -> dict:
    """Achieved algorithmic GB/s of every single op at the sizes of configurations 1-4."""
    L = abi.lib()
    table: dict = {}

    def put(name, nbytes, ms, note=None):
        gbs = nbytes / ms / 1e6
        table[name] = {"ms": round(ms, 4), "gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 3),
                       "frac_of_nominal_8000": round(gbs / NOMINAL_HBM_GBS, 3)}
        if isinstance(ms, Timing):
            table[name]["min_ms"] = round(ms.min_ms, 4)
            table[name]["ms_back_to_back"] = round(ms.batch_ms, 4)
            table[name]["frac_of_peak_back_to_back"] = round(nbytes / ms.batch_ms / 1e6 / peak, 3)
        if note:
            table[name]["note"] = note

    def dense_desc(nt, n):
        d = abi.IterDesc()
        abi.check(L.twg_iter_contiguous(ctypes.byref(d), nt, n))
        return d

    # configuration 1: add [4096,4096], rotating over 4 buffer sets (> L2), and [16384,16384]
    n1 = 4096 * 4096
    g = torch.Generator().manual_seed(0)
    a1, b1 = torch.randn(n1, generator=g).numpy(), torch.randn(n1, generator=g).numpy()
    sets = []
    for _ in range(4):
        da, db, do = abi.DeviceBuffer(4 * n1), abi.DeviceBuffer(4 * n1), abi.DeviceBuffer(4 * n1)
        da.upload(a1, stream); db.upload(b1, stream)
        sets.append((da, db, do))
    d3 = dense_desc(3, n1)
    turn = [0]
    def add_small():
        da, db, do = sets[turn[0] % 4]
        turn[0] += 1
        abi.check(L.twg_binary_f32(0, ctypes.byref(d3), da.ptr, db.ptr, 1.0, do.ptr, stream))
    put("add_4096x4096", 12 * n1, time_op(abi, stream, add_small, iters=40), "4 rotating buffer sets (768 MiB)")
    del sets

    # configuration 2: activations on 2^28 elements
    n2 = 1 << 28
    g = torch.Generator().manual_seed(1)
    x = (torch.rand(n2, generator=g) * 16 - 8).numpy()
    dx, dy, dz = abi.DeviceBuffer(4 * n2), abi.DeviceBuffer(4 * n2), abi.DeviceBuffer(4 * n2)
    dx.upload(x, stream)
    abi.check(L.twg_memcpy_d2d(dy.ptr, dx.ptr, 4 * n2, stream))
    d2 = dense_desc(2, n2)
    d3 = dense_desc(3, n2)
    put("add_16384x16384", 12 * n2, time_op(abi, stream, lambda: abi.check(
        L.twg_binary_f32(0, ctypes.byref(d3), dx.ptr, dy.ptr, 1.0, dz.ptr, stream))))
    for name, op in (("relu", 1), ("silu", 3), ("gelu_erf", 4), ("gelu_tanh", 2)):
        put(f"{name}_2^28", 8 * n2, time_op(abi, stream, lambda op=op: abi.check(
            L.twg_unary_f32(op, ctypes.byref(d2), dx.ptr, dz.ptr, stream))))
    # true transpose: input viewed as [16384,16384].t(), dense output
    r = 16384
    dt = abi.make_desc((r, r), [((r, r), (r, 1)), ((r, r), (1, r))])
    # (output in the buffer next to the input: with a 64 KiB row pitch the throughput of a transpose
    # depends on how far apart the two operands lie - 1 GiB here, 2 GiB costs about 5 %)
    for name, op in (("relu", 1), ("silu", 3), ("gelu_erf", 4)):
        put(f"{name}_transposed_into_dense", 8 * n2, time_op(abi, stream, lambda op=op: abi.check(
            L.twg_unary_f32(op, ctypes.byref(dt), dx.ptr, dy.ptr, stream)), iters=10), "2-D tile kernel")
    ds = abi.make_desc((r, r // 2), [((r, r // 2), (r // 2, 1)), ((r, r // 2), (r, 2))])
    put("relu_stride2_slice", 8 * (n2 // 2), time_op(abi, stream, lambda: abi.check(
        L.twg_unary_f32(1, ctypes.byref(ds), dx.ptr, dz.ptr, stream)), iters=10),
        "strided index path; the stride-2 read drags in whole sectors (real traffic ~12 B/elem)")

    # configuration 3: comparisons and masks on [8192,8192]
    n3 = 8192 * 8192
    g = torch.Generator().manual_seed(2)
    p = torch.randint(-2, 3, (n3,), generator=g).float().numpy()
    q = torch.randint(-2, 3, (n3,), generator=g).float().numpy()
    dx.upload(p, stream); dy.upload(q, stream)
    m1, m2, m3 = abi.DeviceBuffer(n3), abi.DeviceBuffer(n3), abi.DeviceBuffer(n3)
    d2 = dense_desc(2, n3)
    d3 = dense_desc(3, n3)
    put("eq_tensor_8192x8192", 9 * n3, time_op(abi, stream, lambda: abi.check(
        L.twg_compare_f32(0, ctypes.byref(d3), dx.ptr, dy.ptr, 0.0, m1.ptr, stream)), iters=40))
    put("ne_scalar_8192x8192", 5 * n3, time_op(abi, stream, lambda: abi.check(
        L.twg_compare_f32(1, ctypes.byref(d2), dx.ptr, None, 0.0, m2.ptr, stream)), iters=40))
    put("bitwise_and_bool_8192x8192", 3 * n3, time_op(abi, stream, lambda: abi.check(
        L.twg_bitwise_and(ctypes.byref(d3), 1, 1, m1.ptr, m2.ptr, m3.ptr, stream)), iters=40),
        "192 MiB footprint: partly L2-resident")
    del m1, m2, m3

    # configuration 4: masked_select on [16384,16384]
    g = torch.Generator().manual_seed(3)
    src = torch.randn(n2, generator=g).numpy()
    dx.upload(src, stream)
    dm = abi.DeviceBuffer(n2)
    res = abi.DeviceBuffer(16)
    ws_bytes = L.twg_masked_select_workspace_bytes(n2)
    ws = abi.DeviceBuffer(ws_bytes)
    dsel = dense_desc(2, n2)
    for prob in (0.01, 0.5, 0.99):
        mask = (torch.rand(n2, generator=g) < prob).numpy().view(np.uint8)
        dm.upload(mask, stream)
        run = lambda: abi.check(L.twg_masked_select_f32(ctypes.byref(dsel), dx.ptr, dm.ptr, dz.ptr, res.ptr, ws.ptr, ws_bytes, stream))
        ms = time_op(abi, stream, run, iters=10)
        k = int(res.download(np.int64, 2, stream)[0])
        put(f"masked_select_p{prob}", 5 * n2 + 4 * k, ms, f"k={k}; includes the workspace clear")
    rowmask = (torch.rand(r, generator=g) < 0.5).numpy().view(np.uint8)
    dm.upload(rowmask, stream)
    drow = abi.make_desc((r, r), [((r, r), (r, 1)), ((r, 1), (1, 1))])
    run = lambda: abi.check(L.twg_masked_select_f32(ctypes.byref(drow), dx.ptr, dm.ptr, dz.ptr, res.ptr, ws.ptr, ws_bytes, stream))
    ms = time_op(abi, stream, run, iters=10)
    k = int(res.download(np.int64, 2, stream)[0])
    put("masked_select_rowmask_16384x1", 4 * n2 + r + 4 * k, ms, f"k={k}; broadcast mask through the strided path")

    # the chain's mask kernel: the ahead-of-time instantiation beside the same chain with a constant
    # changed in the last place, which no ahead-of-time program matches and NVRTC compiles at run time
    g = torch.Generator().manual_seed(4)
    for buf in (dx, dy):
        buf.upload(torch.randn(n2, generator=g).numpy(), stream)
    dc0 = abi.DeviceBuffer(4 * n2)
    dc0.upload(torch.randn(n2, generator=g).numpy(), stream)
    d4 = dense_desc(4, n2)
    chain_ptrs = (ctypes.c_void_p * 4)(dm.ptr, dx.ptr, dy.ptr, dc0.ptr)
    jit_prog = [list(i) for i in abi.CHAIN_MASK_PROGRAM]
    jit_prog[3][3] = float(np.nextafter(np.float32(1.0), np.float32(2.0)))   # alpha of the first add
    for name, prog in (("chain_mask_aot_2^28", abi.CHAIN_MASK_PROGRAM), ("chain_mask_nvrtc_2^28", [tuple(i) for i in jit_prog])):
        handle = abi.fused_compile(prog)
        kind = abi.fused_kind(handle)
        put(name, 13 * n2, time_op(abi, stream, lambda: abi.check(
            L.twg_fused_launch(handle, ctypes.byref(d4), chain_ptrs, stream))), f"kernel kind: {kind}")
        abi.check(L.twg_fused_release(handle))
    del dc0

    # predicate + select: byte mask kernel then masked_select, against the form that keeps the mask as bits
    g = torch.Generator().manual_seed(4)
    for buf in (dx, dy):
        buf.upload(torch.randn(n2, generator=g).numpy(), stream)
    dc = abi.DeviceBuffer(4 * n2)
    dc.upload(torch.randn(n2, generator=g).numpy(), stream)
    fws_bytes = L.twg_fused_select_workspace_bytes(n2)
    fws = abi.DeviceBuffer(fws_bytes)
    F = abi
    positive = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_CONST_F32, 0, 0, 0.0), (F.F_GT, 0, 1, 0.0), (F.F_OUTPUT, 2, 0, 0.0)]
    for name, prog, nin in (("chain", abi.CHAIN_MASK_PROGRAM, 3), ("positive", positive, 1)):
        handle = abi.fused_compile(prog)
        ins = [dx, dy, dc][:nin]
        dmask = dense_desc(1 + nin, n2)
        mask_ptrs = (ctypes.c_void_p * (1 + nin))(dm.ptr, *[i.ptr for i in ins])
        in_ptrs = (ctypes.c_void_p * nin)(*[i.ptr for i in ins])

        def two_launches():
            abi.check(L.twg_fused_launch(handle, ctypes.byref(dmask), mask_ptrs, stream))
            abi.check(L.twg_masked_select_f32(ctypes.byref(dsel), dx.ptr, dm.ptr, dz.ptr, res.ptr, ws.ptr, ws_bytes, stream))

        def bit_mask():
            abi.check(L.twg_fused_select_f32(handle, 0, n2, in_ptrs, dz.ptr, res.ptr, fws.ptr, fws_bytes, stream))

        ms2 = time_op(abi, stream, two_launches, iters=10)
        k2 = int(res.download(np.int64, 2, stream)[0])
        ms1 = time_op(abi, stream, bit_mask, iters=10)
        k1, status = (int(v) for v in res.download(np.int64, 2, stream))
        if k1 != k2 or status != 0:
            raise RuntimeError(f"fused select kept {k1} elements (status {status}), the two-launch form {k2}")
        put(f"select_{name}_two_launches", (4 * nin + 1) * n2 + 5 * n2 + 4 * k2, ms2, f"k={k2}; mask written and read back")
        put(f"select_{name}_bit_mask", 4 * nin * n2 + n2 // 4 + 4 * n2 + 4 * k1, ms1, f"k={k1}; mask written and read back as bits")
        abi.check(L.twg_fused_release(handle))
    return table


def run_case(args) -> None:
    """One kernel on a small case (a few GB at most, still larger than L2), sized for a profiler
    capture.  Prints its own JSON line; not the benchmark."""
    from torch_webgpu import abi
    L = abi.lib()
    n = args.case_elems
    stream = None
    peak, _ = measured_peak()
    rng = np.random.default_rng(11)

    def host(count):
        return (rng.random(count, dtype=np.float32) * 4 - 2).astype(np.float32)

    def dense(nt, count):
        d = abi.IterDesc()
        abi.check(L.twg_iter_contiguous(ctypes.byref(d), nt, count))
        return d

    bufs = []
    if args.case == "chain":
        ins = [abi.DeviceBuffer(4 * n) for _ in range(3)]
        for b_ in ins:
            b_.upload(host(n))
        m = abi.DeviceBuffer(n)
        prog = abi.fused_compile(abi.CHAIN_MASK_PROGRAM)
        d = dense(4, n)
        ptrs = (ctypes.c_void_p * 4)(m.ptr, ins[0].ptr, ins[1].ptr, ins[2].ptr)
        fn = lambda: abi.check(L.twg_fused_launch(prog, ctypes.byref(d), ptrs, stream))
        nbytes = 13 * n
        bufs = ins + [m]
    elif args.case in ("relu", "silu", "gelu_erf"):
        x, y = abi.DeviceBuffer(4 * n), abi.DeviceBuffer(4 * n)
        x.upload(host(n))
        d = dense(2, n)
        op = abi.UNARY[args.case]
        fn = lambda: abi.check(L.twg_unary_f32(op, ctypes.byref(d), x.ptr, y.ptr, stream))
        nbytes = 8 * n
        bufs = [x, y]
    elif args.case == "add":
        x, y, z = abi.DeviceBuffer(4 * n), abi.DeviceBuffer(4 * n), abi.DeviceBuffer(4 * n)
        x.upload(host(n)); y.upload(host(n))
        d = dense(3, n)
        fn = lambda: abi.check(L.twg_binary_f32(0, ctypes.byref(d), x.ptr, y.ptr, 1.0, z.ptr, stream))
        nbytes = 12 * n
        bufs = [x, y, z]
    elif args.case in ("relu_transposed", "silu_transposed", "gelu_erf_transposed"):
        r = int(round(n ** 0.5))
        n = r * r
        x, y = abi.DeviceBuffer(4 * n), abi.DeviceBuffer(4 * n)
        x.upload(host(n))
        d = abi.make_desc((r, r), [((r, r), (r, 1)), ((r, r), (1, r))])
        op = abi.UNARY[args.case[:-len("_transposed")]]
        fn = lambda: abi.check(L.twg_unary_f32(op, ctypes.byref(d), x.ptr, y.ptr, stream))
        nbytes = 8 * n
        bufs = [x, y]
    elif args.case in ("masked_select", "masked_select_rowmask", "masked_select_transposed", "masked_select_colmask",
                       "masked_select_slice"):
        x, out = abi.DeviceBuffer(4 * n), abi.DeviceBuffer(4 * n)
        x.upload(host(n))
        res = abi.DeviceBuffer(16)
        wsb = L.twg_masked_select_workspace_bytes(n)
        ws = abi.DeviceBuffer(wsb)
        if args.case == "masked_select":
            mk = abi.DeviceBuffer(n)
            mk.upload((rng.random(n) < args.case_density).astype(np.uint8))
            d = dense(2, n)
        elif args.case == "masked_select_colmask":
            r = int(round(n ** 0.5))
            n = r * r
            mk = abi.DeviceBuffer(r)
            mk.upload((rng.random(r) < args.case_density).astype(np.uint8))
            d = abi.make_desc((r, r), [((r, r), (r, 1)), ((1, r), (1, 1))])   # one mask byte per column
        elif args.case == "masked_select_slice":
            r = int(round(n ** 0.5))
            n = r * (r // 2)
            mk = abi.DeviceBuffer(r * r)
            mk.upload((rng.random(r * r) < args.case_density).astype(np.uint8))
            d = abi.make_desc((r, r // 2), [((r, r // 2), (r, 2)), ((r, r // 2), (r, 2))])   # x[:, ::2], m[:, ::2]
        elif args.case == "masked_select_transposed":
            r = int(round(n ** 0.5))
            n = r * r
            mk = abi.DeviceBuffer(n)
            mk.upload((rng.random(n) < args.case_density).astype(np.uint8))
            d = abi.make_desc((r, r), [((r, r), (1, r)), ((r, r), (1, r))])   # src.t() and mask.t()
        else:
            r = int(round(n ** 0.5))
            n = r * r
            mk = abi.DeviceBuffer(r)
            mk.upload((rng.random(r) < args.case_density).astype(np.uint8))
            d = abi.make_desc((r, r), [((r, r), (r, 1)), ((r, 1), (1, 1))])
        fn = lambda: abi.check(L.twg_masked_select_f32(ctypes.byref(d), x.ptr, mk.ptr, out.ptr, res.ptr, ws.ptr, wsb, stream))
        fn()
        k = int(res.download(np.int64, 2)[0])
        nbytes = (4 if args.case in ("masked_select_rowmask", "masked_select_colmask") else 5) * n + 4 * k
        bufs = [x, out, res, ws, mk]
    elif args.case == "fused_select":
        ins = [abi.DeviceBuffer(4 * n) for _ in range(3)]
        for b_ in ins:
            b_.upload(host(n))
        out, res = abi.DeviceBuffer(4 * n), abi.DeviceBuffer(16)
        wsb = L.twg_fused_select_workspace_bytes(n)
        ws = abi.DeviceBuffer(wsb)
        prog = abi.fused_compile(abi.CHAIN_MASK_PROGRAM)
        in_ptrs = (ctypes.c_void_p * 3)(*[i.ptr for i in ins])
        fn = lambda: abi.check(L.twg_fused_select_f32(prog, 0, n, in_ptrs, out.ptr, res.ptr, ws.ptr, wsb, stream))
        fn()
        k = int(res.download(np.int64, 2)[0])
        nbytes = 12 * n + n // 4 + 4 * n + 4 * k
        bufs = ins + [out, res, ws]
    else:
        raise SystemExit(f"unknown case {args.case}")
    ms = time_op(abi, stream, fn, iters=max(args.steps, 1), warmup=max(args.warmup, 0))
    print(json.dumps({"case": args.case, "elements": n, "ms": ms, "ms_back_to_back": ms.batch_ms, "algorithmic_bytes": nbytes,
                      "gbs": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / peak,
                      "frac_of_peak_back_to_back": nbytes / ms.batch_ms / 1e6 / peak, "path": abi.last_path()}), flush=True)
    del bufs


def pin_to_core_block(local_rank: int, local_world: int) -> list[int]:
    """With several ranks on one host, give each its own block of the allowed cores so that the
    ranks' issuing threads and their helper threads do not migrate over each other."""
    try:
        allowed = sorted(os.sched_getaffinity(0))
        per = len(allowed) // max(local_world, 1)
        if local_world > 1 and per >= 2:
            mine = allowed[local_rank * per:(local_rank + 1) * per]
            os.sched_setaffinity(0, mine)
            return mine
        return allowed
    except (AttributeError, OSError):
        return []


def verify_slab(oracle, a, b, c, gpu_mask, gpu_selected, what: str) -> None:
    """One [4096,4096] slab of the timed run against the CPU oracle.  The mask may differ from the
    oracle's only where the value under relu is within rounding of zero (silu is allowed 2 ulp);
    given the mask, the selected values and their order must be bit-identical."""
    y_ref, m_ref = oracle.chain_mask(a, b, c, want_y=True)
    gpu_mask = gpu_mask.reshape(m_ref.shape).astype(bool)
    flipped = gpu_mask != m_ref
    if flipped.sum() > max(4, m_ref.size // 1_000_000) or not np.all(np.abs(y_ref[flipped]) < 1e-6):
        raise RuntimeError(f"bench verification failed ({what}): {int(flipped.sum())} mask elements differ from the oracle")
    ref_sel = oracle.masked_select(a.reshape(-1), gpu_mask.reshape(-1))
    if ref_sel.size != gpu_selected.size or not np.array_equal(ref_sel.view(np.uint32), gpu_selected.view(np.uint32)):
        raise RuntimeError(f"bench verification failed ({what}): the selected values differ from the oracle "
                           f"({gpu_selected.size} on the GPU, {ref_sel.size} expected)")


def run_gpu_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU fallback (use --impl reference for the CPU arm)")

    import torch_webgpu  # noqa: F401  (registers the webgpu device and the compile backend)
    from torch_webgpu import abi, webgpu_backend
    from torch_webgpu.sharding import NcclExchange, PeerStoreExchange, Rendezvous, shard_range

    cores = pin_to_core_block(local_rank, local_world)
    rdv = Rendezvous.from_env()
    torch.webgpu.set_device(local_rank)
    L = abi.lib()
    abi.check(L.twg_set_device(local_rank))
    stream = ctypes.c_void_p(torch.webgpu.current_stream_handle(local_rank))   # the backend's compute stream
    side = ctypes.c_void_p()
    abi.check(L.twg_get_stream(local_rank, 2, ctypes.byref(side)))             # collects the counts behind it
    peak, peak_kind = measured_peak()

    lo, hi = shard_range(BATCH, rank, world)
    nb = hi - lo
    n = nb * SLAB
    DEPTH = 2 if world == 1 else 4      # steps the host may run ahead of the counts it has seen
    RING = 2 * DEPTH                    # mailbox slots (see twg_exchange_publish's reuse rule)

    # ---- the ranks' communicator and count exchange, all through the C ABI ---------------------
    nccl = None
    exchange_note = None
    if world > 1:
        uid = rdv.broadcast(NcclExchange.make_unique_id(abi) if rank == 0 else None)
        nccl = NcclExchange(abi, rank, world, uid, local_rank, ring=RING)
    d_token = abi.DeviceBuffer(8 * (world + 1), local_rank, stream)

    def barrier() -> None:
        """Every rank's stream has drained and every rank has arrived (device-side meeting point:
        the ranks leave within microseconds of each other)."""
        abi.check(L.twg_stream_sync(side))
        abi.check(L.twg_stream_sync(stream))
        if nccl is not None:
            nccl.allgather(d_token.ptr, d_token.ptr + 8, 1, stream)
            abi.check(L.twg_stream_sync(stream))

    xchg = None
    if args.exchange in ("auto", "peer"):
        px, handle, ok = None, b"", 1
        try:
            px = PeerStoreExchange(abi, rank, world, ring=RING)
            handle = px.export_handle() if world > 1 else b""
        except abi.TwgError as exc:
            ok, exchange_note = 0, str(exc)
        handles = rdv.share(handle)
        if ok and world > 1:
            try:
                px.connect(handles)
            except abi.TwgError as exc:
                ok, exchange_note = 0, str(exc)
        oks = rdv.share(bytes([ok]) + (exchange_note or "").encode()[:200])
        if all(o[:1] == b"\x01" for o in oks):
            xchg = px
        else:
            exchange_note = next(o[1:].decode(errors="replace") for o in oks if o[:1] != b"\x01")
            if args.exchange == "peer":
                raise SystemExit(f"bench.py: --exchange peer is not possible here: {exchange_note}")
    if xchg is None:
        if nccl is None:
            raise SystemExit("bench.py: --exchange nccl needs more than one rank")
        xchg = nccl

    # ---- synthetic inputs in pinned host memory --------------------------------------------
    host = [torch.empty(nb, ROWS, COLS, pin_memory=True) for _ in range(3)]
    for t, buf in enumerate(host):
        fill_shard(buf, t, lo, hi)

    # ---- leg 1: inputs resident in HBM, C ABI calls ----------------------------------------
    dev_in = [abi.DeviceBuffer(4 * n, local_rank, stream) for _ in range(3)]
    for buf, h in zip(dev_in, host):
        abi.check(L.twg_memcpy_h2d(buf.ptr, h.data_ptr(), 4 * n, stream))
    bits_mode = args.mask == "bits"
    d_mask = None if bits_mode else abi.DeviceBuffer(n, local_rank, stream)
    # DEPTH sets of everything a step writes: the host picks up the counts of step i while the GPU
    # already runs the steps after it, so the stream never waits for the host or for another rank.
    ws_bytes = L.twg_masked_select_workspace_bytes(n)
    d_bits = abi.DeviceBuffer(L.twg_predicate_bits_bytes(n), local_rank, stream) if bits_mode else None
    d_out = [abi.DeviceBuffer(4 * n, local_rank, stream) for _ in range(DEPTH)]
    d_ws = [abi.DeviceBuffer(ws_bytes, local_rank, stream) for _ in range(DEPTH)]
    d_res = [abi.DeviceBuffer(16, local_rank, stream) for _ in range(DEPTH)]   # [count, status] of this rank
    compacted = Events(abi, DEPTH)
    program = abi.fused_compile(abi.CHAIN_MASK_PROGRAM)
    assert abi.fused_kind(program) == "aot"
    desc4 = abi.IterDesc()
    abi.check(L.twg_iter_contiguous(ctypes.byref(desc4), 4, n))
    desc2 = abi.IterDesc()
    abi.check(L.twg_iter_contiguous(ctypes.byref(desc2), 2, n))
    ptrs = (ctypes.c_void_p * 4)(0 if bits_mode else d_mask.ptr, dev_in[0].ptr, dev_in[1].ptr, dev_in[2].ptr)
    in_ptrs = (ctypes.c_void_p * 3)(dev_in[0].ptr, dev_in[1].ptr, dev_in[2].ptr)

    steps, warmup = args.steps, args.warmup
    ev = Events(abi, 2 + 2 * steps)
    counts_seen: list[tuple[int, int, int]] = []   # (this rank's count, its global offset, total) per collected step
    host_s = [0.0, 0.0, 0.0]   # seconds spent issuing steps / waiting for counts / handling them
    seq_next = [1]

    def launch(i: int | None) -> int:
        """Everything one step puts on the GPU: fused chain and compaction (which also publishes this
        rank's count to every rank) on the compute stream, and on a second stream the kernel that
        gathers all ranks' counts for the host.  Events 2+2i / 3+2i bracket the fused chain."""
        t_issue = time.perf_counter()
        seq = seq_next[0]
        seq_next[0] += 1
        slot = seq % DEPTH
        if i is not None:
            ev.record(2 + 2 * i, stream)
        if bits_mode:
            abi.check(L.twg_fused_predicate_bits(program, n, in_ptrs, d_bits.ptr, stream))
        else:
            abi.check(L.twg_fused_launch(program, ctypes.byref(desc4), ptrs, stream))
        if i is not None:
            ev.record(3 + 2 * i, stream)
        # compaction; its last chunk stores this rank's count into every rank's mailbox
        if bits_mode:
            xchg.select_bits_publish(seq, dev_in[0].ptr, d_bits.ptr, n, d_out[slot].ptr, d_res[slot].ptr, d_ws[slot].ptr,
                                     ws_bytes, stream)
        else:
            xchg.masked_select_publish(seq, desc2, dev_in[0].ptr, d_mask.ptr, d_out[slot].ptr, d_res[slot].ptr,
                                       d_ws[slot].ptr, ws_bytes, stream)
        compacted.record(slot, stream)
        abi.check(L.twg_event_wait(compacted.ev[slot], side))
        xchg.collect(seq, side)
        host_s[0] += time.perf_counter() - t_issue
        return seq

    def collect(seq: int) -> None:
        """The step's host sync: its counts are needed on the host (output shape, global offset)."""
        t_wait = time.perf_counter()
        counts, offset, total = xchg.wait(seq)
        t_got = time.perf_counter()
        counts_seen.append((counts[rank], offset, total))
        host_s[1] += t_got - t_wait
        host_s[2] += time.perf_counter() - t_got

    def run_steps(count: int, timed: bool) -> None:
        pending: list[int] = []
        for i in range(count):
            pending.append(launch(i if timed else None))
            if len(pending) >= DEPTH:
                collect(pending.pop(0))
        while pending:
            collect(pending.pop(0))

    # the clock sampler attaches to NVML before the ranks meet, so that nothing but the record of
    # the first event lies between the barrier and the timed region
    sampler = ClockSampler(local_rank)
    run_steps(max(warmup, 1), False)
    if rank == 0:
        sampler.start()
    L.twg_reset_launch_count()
    counts_seen.clear()
    barrier()
    host_s[0] = host_s[1] = host_s[2] = 0.0
    ev.record(0, stream)
    run_steps(steps, True)
    ev.record(1, stream)
    ev.sync(1)
    launches = int(L.twg_launch_count())
    barrier()
    clocks = sampler.stop() if rank == 0 else {}
    ms_total = ev.elapsed(0, 1)
    fused_samples = [ev.elapsed(2 + 2 * i, 3 + 2 * i) for i in range(steps)]
    intervals = [ev.elapsed(2 + 2 * i, 4 + 2 * i) for i in range(steps - 1)]
    mine = {"ms_total": ms_total, "fused_ms": statistics.mean(fused_samples),
            "first_kernel_ms": ev.elapsed(0, 2), "tail_ms": ev.elapsed(2 + 2 * (steps - 1), 1),
            "step_ms_median": statistics.median(intervals) if intervals else ms_total,
            "step_ms_p90": sorted(intervals)[int(0.9 * (len(intervals) - 1))] if intervals else ms_total,
            "step_ms_max": max(intervals) if intervals else ms_total,
            "host_us": [round(x / steps * 1e6, 1) for x in host_s],
            "count": counts_seen[-1][0], "offset": counts_seen[-1][1], "total": counts_seen[-1][2],
            "same_every_step": len(set(counts_seen)) == 1}
    per_rank = [json.loads(x) for x in rdv.share(json.dumps(mine).encode())]
    ms_total = max(r["ms_total"] for r in per_rank)
    fused_ms_max = max(r["fused_ms"] for r in per_rank)
    ms_per_step = ms_total / steps
    value = BATCH * SLAB / (ms_per_step * 1e-3) / 1e9
    total_k = per_rank[0]["total"]
    # every rank saw the same total, the offsets are the exclusive prefix sums of the counts, and
    # no step produced a different count from the others (the inputs never change)
    acc = 0
    for r in per_rank:
        if r["total"] != total_k or r["offset"] != acc or not r["same_every_step"]:
            raise RuntimeError(f"bench: inconsistent counts across ranks or steps: {per_rank}")
        acc += r["count"]
    if acc != total_k:
        raise RuntimeError(f"bench: the ranks' counts add up to {acc}, the exchanged total is {total_k}")

    # ---- verification, not timed: this rank's first and last slab against the CPU oracle --------
    verified = None
    if not args.no_verify:
        from oracle import oracle
        oracle.build()
        oracle.set_num_threads(max(1, len(cores) or (os.cpu_count() or 1)))
        last_slot = (seq_next[0] - 1) % DEPTH
        k_mine = counts_seen[-1][0]
        for which in sorted({0, nb - 1}):
            if bits_mode:   # bit i of byte j is element 8 j + i
                packed = d_bits.download(np.uint8, SLAB // 8, stream, offset_bytes=which * (SLAB // 8))
                gmask = np.unpackbits(packed, bitorder="little")
            else:
                gmask = d_mask.download(np.uint8, SLAB, stream, offset_bytes=which * SLAB)
            kept = int(np.count_nonzero(gmask))
            seg_lo = 0 if which == 0 else k_mine - kept      # first slab: head of the output; last slab: its tail
            if nb == 1 and kept != k_mine:
                raise RuntimeError(f"bench verification failed: the mask keeps {kept} elements, the kernel counted {k_mine}")
            gsel = d_out[last_slot].download(np.float32, kept, stream, offset_bytes=4 * seg_lo)
            verify_slab(oracle, host[0][which].numpy(), host[1][which].numpy(), host[2][which].numpy(), gmask, gsel,
                        f"rank {rank}, slab {lo + which}")
        verified = all(x == b"ok" for x in rdv.share(b"ok"))

    # ---- per-op table (single GPU only) -----------------------------------------------------
    del d_out, d_mask, d_ws, d_bits
    for b_ in dev_in:
        b_.free()
    ops = per_op_table(abi, stream, peak) if world == 1 and not args.no_ops else None
    abi.check(L.twg_empty_cache(local_rank))

    # ---- the public API: torch.compile(chain, backend=webgpu_backend) -------------------------
    def chain(a, b, c):
        y = torch.relu(torch.nn.functional.silu(a + b) + c)
        m = torch.bitwise_and(torch.eq(y, 0), torch.ne(a, 0))
        return torch.masked_select(a, m)

    # With this dynamo flag masked_select stays inside the compiled graph, and the backend hands the
    # mask over as bits (webgpu::run_fused_select); without it dynamo cuts the graph in front of
    # masked_select and the mask has to be a bool tensor.
    torch._dynamo.config.capture_dynamic_output_shape_ops = bits_mode
    compiled = torch.compile(chain, backend=webgpu_backend)
    dev_name = f"webgpu:{local_rank}"
    d_cnt = abi.DeviceBuffer(16, local_rank, stream)
    h_cnt = (ctypes.c_int64 * 2)()

    def exchange_count(k: int) -> tuple[int, int]:
        """The count a rank's masked_select returned, told to every rank: (global offset, total)."""
        seq = seq_next[0]
        seq_next[0] += 1
        h_cnt[0], h_cnt[1] = k, 0
        abi.check(L.twg_memcpy_h2d(d_cnt.ptr, ctypes.addressof(h_cnt), 16, stream))
        xchg.publish(seq, d_cnt.ptr, stream)
        xchg.collect(seq, stream)
        _counts, offset, total = xchg.wait(seq)
        return offset, total

    # (a) inputs resident on the device: what a drop-in user of the backend gets per step
    resident = [h.to(dev_name) for h in host]
    api_steps = max(1, min(steps, 10))
    for _ in range(3):
        sel = compiled(*resident)     # kept across the next call, as in the timed loop: warms both result buffers
    barrier()
    ev3 = Events(abi, 2 + api_steps)
    ev3.record(0, stream)
    for i in range(api_steps):
        sel = compiled(*resident)     # ends with the count read-back that sizes the result
        api_total = exchange_count(sel.numel())[1]
        ev3.record(2 + i, stream)
    ev3.record(1, stream)
    ev3.sync(1)
    api_each = [ev3.elapsed(2 + i - 1 if i else 0, 2 + i) for i in range(api_steps)]
    if api_total != total_k:
        raise RuntimeError(f"bench: the public API selected {api_total} elements, the C ABI leg {total_k}")
    api_ms = max(float(x) for x in rdv.share(repr(ev3.elapsed(0, 1) / api_steps).encode()))
    public_api = {"value": BATCH * SLAB / (api_ms * 1e-3) / 1e9, "unit": "Gelem/s", "ms_per_step": api_ms, "steps": api_steps,
                  "ms_per_step_median_rank0": statistics.median(api_each), "ms_each_rank0": [round(x, 3) for x in api_each],
                  "api": "torch.compile(chain, backend=webgpu_backend)(a, b, c) on device-resident webgpu tensors"
                         + (", torch._dynamo.config.capture_dynamic_output_shape_ops=True (one graph, mask as bits)" if bits_mode
                            else " (graph break in front of masked_select, mask as a bool tensor)")
                         + "; every call ends with the blocking count read-back of masked_select"}
    del resident, sel
    abi.check(L.twg_empty_cache(local_rank))

    # (b) end to end with host buffers: upload of a, b, c and read-back of the result every step
    h_sel = [torch.empty(n, pin_memory=True) for _ in range(2)]   # the read-back of step i runs under step i+1's uploads
    e2e_steps = max(1, min(steps, 8))
    d2h_bytes = [0]
    side2 = torch.Stream(device=dev_name)
    in_flight: list = []    # (event after the read-back, the tensor it reads) of the previous step

    def retire() -> None:
        while in_flight:
            copied, _keep = in_flight.pop()
            copied.synchronize()

    def e2e_step(i: int) -> None:
        da, db, dc = (h.to(dev_name, non_blocking=True) for h in host)
        sel = compiled(da, db, dc)                  # ends with the count read-back: the step's host sync
        k = sel.numel()
        ready = torch.Event(device=dev_name)
        ready.record()
        with side2:                                 # PCIe is full duplex: read back on a second stream
            side2.wait_event(ready)
            h_sel[i & 1][:k].copy_(sel, non_blocking=True)
            copied = torch.Event(device=dev_name)
            copied.record()
        retire()                                    # the previous step's result is now complete on the host
        in_flight.append((copied, sel))
        d2h_bytes[0] = 4 * k + 16
        exchange_count(k)

    e2e_step(0)  # warm the allocator
    retire()
    barrier()
    ev2 = Events(abi, 2)
    ev2.record(0, stream)
    t_host = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    retire()                                        # every result has landed in host memory
    ev2.record(1, stream)
    ev2.sync(1)
    host_ms = (time.perf_counter() - t_host) * 1e3
    barrier()
    # the last read-back runs on the second stream, which the events on the main stream do not see:
    # the host clock around the loop (it ends after retire()) bounds it, so take the larger
    e2e_mine = max(ev2.elapsed(0, 1), host_ms) / e2e_steps
    # the same uploads and nothing else: what the host side of PCIe delivers to this many GPUs at once
    staging = [abi.DeviceBuffer(4 * n, local_rank, stream) for _ in range(3)]
    for _ in range(2):
        for buf, h in zip(staging, host):
            abi.check(L.twg_memcpy_h2d(buf.ptr, h.data_ptr(), 4 * n, stream))
    barrier()
    ev4 = Events(abi, 2)
    ev4.record(0, stream)
    for _ in range(4):
        for buf, h in zip(staging, host):
            abi.check(L.twg_memcpy_h2d(buf.ptr, h.data_ptr(), 4 * n, stream))
    ev4.record(1, stream)
    ev4.sync(1)
    h2d_only_ms = ev4.elapsed(0, 1) / 4
    del staging
    shared = [json.loads(x) for x in rdv.share(json.dumps([e2e_mine, h2d_only_ms, 3 * 4 * n, d2h_bytes[0]]).encode())]
    e2e_ms = max(s[0] for s in shared)
    h2d_total, d2h_total = sum(s[2] for s in shared), sum(s[3] for s in shared)
    e2e = {"value": BATCH * SLAB / (e2e_ms * 1e-3) / 1e9, "unit": "Gelem/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
           "h2d_bytes_per_step": int(h2d_total), "d2h_bytes_per_step": int(d2h_total),
           "h2d_gbs_achieved": round(h2d_total / e2e_ms / 1e6, 1),
           "h2d_only_gbs": round(h2d_total / max(s[1] for s in shared) / 1e6, 1),
           "api": "x.to('webgpu') from pinned tensors, torch.compile(backend=webgpu_backend) chain, pinned read-back "
                  "on a second torch.Stream so that it overlaps the next step's uploads; h2d_only_gbs is the same "
                  "uploads with nothing else running, all ranks at once"}

    if rank == 0:
        achieved = CHAIN_BYTES_PER_ELEM[args.mask] * n / (fused_ms_max * 1e-3) / 1e9
        traffic = CHAIN_DRAM_BYTES_PER_ELEM[args.mask] * n
        line = {
            "metric": "Gelem/s of the compiled chain + masked_select", "value": value, "unit": "Gelem/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(world, DEPTH, args.mask),
            "selected_elements": total_k, "verified": verified,
            "roofline": {"bound": "hbm", "kernel": CHAIN_KERNEL[args.mask],
                         "achieved": achieved, "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                         "frac": achieved / peak, "frac_of_nominal_8000": achieved / NOMINAL_HBM_GBS, "traffic": traffic,
                         "ms_per_launch": fused_ms_max, "algorithmic_bytes_per_launch": CHAIN_BYTES_PER_ELEM[args.mask] * n},
            "e2e": e2e, "public_api": public_api, "gpu_launches": launches, "clocks": clocks,
            "step_ms_median": max(r["step_ms_median"] for r in per_rank),
            "step_timing": {"per_rank_ms_total": [round(r["ms_total"], 4) for r in per_rank],
                            "step_ms_median": [round(r["step_ms_median"], 4) for r in per_rank],
                            "step_ms_p90": [round(r["step_ms_p90"], 4) for r in per_rank],
                            "step_ms_max": [round(r["step_ms_max"], 4) for r in per_rank],
                            "first_kernel_ms": [round(r["first_kernel_ms"], 4) for r in per_rank],
                            "last_step_and_drain_ms": [round(r["tail_ms"], 4) for r in per_rank],
                            "host_us_per_step_issue_wait_handle": [r["host_us"] for r in per_rank]},
            "count_exchange": xchg.kind, "cores_per_rank": len(cores),
        }
        if exchange_note:
            line["count_exchange_note"] = exchange_note[:300]
        if ops is not None:
            line["ops"] = ops
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = run_cpu_baseline()
        print(json.dumps(line), flush=True)
    barrier()
    if xchg is not nccl:
        xchg.close()
    if nccl is not None:
        nccl.close()
    rdv.barrier()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-ops", action="store_true", help="skip the per-op GB/s table")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="how the ranks exchange their counts: the library's peer-store kernels, ncclAllGather through "
                         "the C ABI, or (auto) peer stores when every rank can map every other rank's mailbox")
    ap.add_argument("--mask", default="bits", choices=["bits", "bytes"],
                    help="how the chain hands its mask to masked_select in the `value` leg: one bit per element in scratch "
                         "memory (what the compile backend does), or a bool tensor")
    ap.add_argument("--no-verify", action="store_true", help="skip the oracle check of each rank's first and last slab")
    ap.add_argument("--batch", type=int, default=64,
                    help="slabs in the batch (64 is the benchmark; smaller values are for diagnosing overheads)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--case", default=None, help="run one kernel on a small case (for ncu captures) and exit")
    ap.add_argument("--case-elems", type=int, default=1 << 27)
    ap.add_argument("--case-density", type=float, default=0.5)
    args = ap.parse_args()
    global BATCH
    BATCH = args.batch
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
