"""Host-side checks that need no GPU: the C ABI library loads and exports everything
include/twg.h declares, descriptor and program logic, the PyTorch device flow up to the first
allocation, the compile backend's partitioning, and the multi-rank sharding logic on gloo."""
from __future__ import annotations

import ctypes
import os
import re
import socket
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def abi():
    from torch_webgpu import abi as _abi
    return _abi


def header_symbols() -> set[str]:
    text = (REPO / "include" / "twg.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(twg_[a-z0-9_]+)\s*\(", text))


def test_library_exports_every_declared_symbol(abi):
    lib = abi.lib()
    names = header_symbols()
    assert len(names) > 40
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, f"declared in twg.h but not exported by libtwg.so: {missing}"
    assert names == set(abi.SIGNATURES), "the ctypes binding and the header disagree"
    assert b"sm_100a" in lib.twg_version()


def test_iteration_descriptor_coalescing(abi):
    L = abi.lib()
    d = abi.IterDesc()
    abi.check(L.twg_iter_contiguous(ctypes.byref(d), 3, 1000))
    assert (d.ndim, d.numel, d.shape[0], d.strides[2][0]) == (1, 1000, 1000, 1)
    # dense [4,6,5] seen by a dense and a broadcast operand: only the dense pair of dims merges
    d = abi.make_desc((4, 6, 5), [((4, 6, 5), (30, 5, 1)), ((4, 1, 5), (5, 5, 1))])
    abi.check(L.twg_iter_coalesce(ctypes.byref(d)))
    assert d.ndim == 3
    d = abi.make_desc((4, 6, 5), [((4, 6, 5), (30, 5, 1)), ((4, 6, 5), (30, 5, 1))])
    abi.check(L.twg_iter_coalesce(ctypes.byref(d)))
    assert (d.ndim, d.shape[0], d.strides[0][0], d.strides[1][0]) == (1, 120, 1, 1)
    # size-1 dimensions vanish; a transposed pair does not merge
    d = abi.make_desc((1, 7, 1, 3), [((1, 7, 1, 3), (21, 3, 3, 1)), ((1, 7, 1, 3), (21, 1, 7, 7))])
    abi.check(L.twg_iter_coalesce(ctypes.byref(d)))
    assert (d.ndim, list(d.shape)[:2]) == (2, [3, 7])
    assert (list(d.strides[0])[:2], list(d.strides[1])[:2]) == ([1, 3], [7, 1])
    d = abi.make_desc((), [((), ()), ((), ())])
    abi.check(L.twg_iter_coalesce(ctypes.byref(d)))
    assert (d.ndim, d.numel) == (0, 1)
    bad = abi.IterDesc()
    bad.ndim, bad.ntensors, bad.numel = 9, 1, 1
    assert L.twg_iter_coalesce(ctypes.byref(bad)) == abi.TWG_ERR_INVALID
    assert b"dimensions" in L.twg_last_error()
    bad.ndim, bad.numel = 1, 7
    bad.shape[0] = 5
    assert L.twg_iter_coalesce(ctypes.byref(bad)) == abi.TWG_ERR_INVALID


def test_fused_program_analysis_and_ahead_of_time_match(abi):
    h = abi.fused_compile(abi.CHAIN_MASK_PROGRAM)
    assert abi.fused_kind(h) == "aot"
    assert abi.fused_compile(abi.CHAIN_MASK_PROGRAM) == h  # cached by content
    add_relu = [(abi.F_INPUT_F32, 0, 0, 0.0), (abi.F_INPUT_F32, 1, 0, 0.0), (abi.F_ADD, 0, 1, 1.0),
                (abi.F_RELU, 2, 0, 0.0), (abi.F_OUTPUT, 3, 0, 0.0)]
    assert abi.fused_kind(abi.fused_compile(add_relu)) == "aot"
    src = ctypes.c_char_p()
    abi.check(abi.lib().twg_fused_source(h, ctypes.byref(src)))
    text = src.value.decode()
    assert "f_silu" in text and "twg_fused_dense" in text and "kOutByteMask = 1u" in text
    for bad in (
        [(abi.F_INPUT_F32, 0, 0, 0.0), (abi.F_AND, 0, 0, 0.0), (abi.F_OUTPUT, 1, 0, 0.0)],   # f32 into and
        [(abi.F_INPUT_F32, 0, 0, 0.0), (abi.F_RELU, 3, 0, 0.0), (abi.F_OUTPUT, 1, 0, 0.0)],  # forward reference
        [(abi.F_INPUT_F32, 0, 0, 0.0), (abi.F_RELU, 0, 0, 0.0)],                             # no output
        [(abi.F_INPUT_F32, 1, 0, 0.0), (abi.F_OUTPUT, 0, 0, 0.0)],                           # slot 0 missing
        [(99, 0, 0, 0.0)],
    ):
        with pytest.raises(abi.TwgError) as e:
            abi.fused_compile(bad)
        assert e.value.code == abi.TWG_ERR_INVALID


def test_bit_mask_sizes_and_argument_checks_need_no_gpu(abi):
    """Sizes of the predicate's bit mask and of the fused select's workspace, and the argument
    checks of the entry points around them (every call below returns before touching a device)."""
    L = abi.lib()
    assert [L.twg_predicate_bits_bytes(n) for n in (-5, 0, 1, 128, 129, 1 << 20)] == [0, 0, 16, 16, 32, 1 << 17]
    for n in (0, 1, 4097, (1 << 22) + 3):
        ms = L.twg_masked_select_workspace_bytes(n)
        assert L.twg_fused_select_workspace_bytes(n) == (ms + 255) // 256 * 256 + L.twg_predicate_bits_bytes(n)
    chain = abi.fused_compile(abi.CHAIN_MASK_PROGRAM)
    add_relu = abi.fused_compile([(abi.F_INPUT_F32, 0, 0, 0.0), (abi.F_INPUT_F32, 1, 0, 0.0), (abi.F_ADD, 0, 1, 1.0),
                                  (abi.F_RELU, 2, 0, 0.0), (abi.F_OUTPUT, 3, 0, 0.0)])
    three = (ctypes.c_void_p * 3)(256, 512, 768)          # never dereferenced: the calls fail before any launch
    assert L.twg_fused_predicate_bits(None, 8, three, 1024, None) == abi.TWG_ERR_INVALID
    assert L.twg_fused_predicate_bits(chain, -1, three, 1024, None) == abi.TWG_ERR_INVALID
    assert L.twg_fused_predicate_bits(chain, 8, three, 1028, None) == abi.TWG_ERR_INVALID          # bits misaligned
    assert b"16-byte aligned" in L.twg_last_error()
    assert L.twg_fused_predicate_bits(add_relu, 8, three, 1024, None) == abi.TWG_ERR_UNSUPPORTED    # f32 output, no predicate
    assert b"not a predicate" in L.twg_last_error()
    misaligned = (ctypes.c_void_p * 3)(256, 516, 768)
    assert L.twg_fused_predicate_bits(chain, 8, misaligned, 1024, None) == abi.TWG_ERR_UNSUPPORTED  # caller falls back
    assert L.twg_masked_select_bits_f32(256, 1024, 8, 2048, None, 4096, 4096, None) == abi.TWG_ERR_INVALID   # no result words
    assert L.twg_masked_select_bits_f32(256, 1024, 8, 2048, 8192, 4096, 16, None) == abi.TWG_ERR_INVALID     # workspace too small
    assert b"smaller than" in L.twg_last_error()
    assert L.twg_masked_select_bits_f32(260, 1024, 8, 2048, 8192, 4096, 4096, None) == abi.TWG_ERR_INVALID   # src misaligned
    assert L.twg_fused_select_f32(chain, 3, 8, three, 2048, 8192, 4096, 1 << 20, None) == abi.TWG_ERR_INVALID  # src_input
    assert L.twg_fused_select_f32(add_relu, 0, 8, three, 2048, 8192, 4096, 1 << 20, None) == abi.TWG_ERR_UNSUPPORTED
    assert L.twg_fused_select_f32(chain, 0, 8, three, 2048, 8192, 4096, 64, None) == abi.TWG_ERR_INVALID      # workspace too small
    assert L.twg_fused_select_f32(chain, 0, 8, three, 2048, 8192, 4100, 1 << 20, None) == abi.TWG_ERR_INVALID  # workspace misaligned


def test_nvrtc_builds_generated_source_without_a_gpu(abi):
    prog = [(abi.F_INPUT_F32, 0, 0, 0.0), (abi.F_INPUT_BOOL, 1, 0, 0.0), (abi.F_GELU_TANH, 0, 0, 0.0),
            (abi.F_CONST_F32, 0, 0, 0.25), (abi.F_LE, 2, 3, 0.0), (abi.F_AND, 4, 1, 0.0), (abi.F_OUTPUT, 5, 0, 0.0),
            (abi.F_OUTPUT, 2, 1, 0.0)]
    try:
        h = abi.fused_compile(prog)
    except abi.TwgError as e:
        if e.code == abi.TWG_ERR_UNSUPPORTED:
            pytest.skip(f"NVRTC is not installed here: {e}")
        raise
    assert abi.fused_kind(h) == "nvrtc"
    # a predicate (one bool output over f32 inputs) also gets the kernel that writes it as bits
    pred = [(abi.F_INPUT_F32, 0, 0, 0.0), (abi.F_INPUT_F32, 1, 0, 0.0), (abi.F_MUL, 0, 1, 0.0),
            (abi.F_CONST_F32, 0, 0, 0.25), (abi.F_GT, 2, 3, 0.0), (abi.F_OUTPUT, 4, 0, 0.0)]
    assert abi.fused_kind(abi.fused_compile(pred)) == "nvrtc"
    src = ctypes.c_char_p()
    abi.check(abi.lib().twg_fused_source(abi.fused_compile(pred), ctypes.byref(src)))
    assert b"twg_fused_bits" in src.value


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour of a machine without a GPU")
def test_no_gpu_means_clean_errors_not_crashes(abi):
    assert abi.device_count() == 0
    with pytest.raises(abi.TwgError) as e:
        abi.DeviceBuffer(1024)
    assert "no CUDA device" in str(e.value)
    import torch_webgpu  # noqa: F401
    assert torch.webgpu.is_available() is False
    with pytest.raises(RuntimeError, match="no CUDA device"):
        torch.empty(4, device="webgpu")


def test_import_registers_the_device_flow():
    import torch_webgpu
    from torch_webgpu import webgpu_backend
    assert torch._C._get_privateuse1_backend_name() == "webgpu"
    assert torch.webgpu.is_initialized() is True and torch.webgpu.current_device() == 0
    assert hasattr(torch.Tensor, "webgpu") and hasattr(torch.Tensor, "is_webgpu")
    assert "webgpu_backend" in torch._dynamo.list_backends(None)
    assert callable(webgpu_backend)
    table = torch._C._dispatch_dump_table
    for op in ("aten::add.out", "aten::relu", "aten::gelu.out", "aten::silu", "aten::eq.Tensor_out", "aten::eq.Scalar",
               "aten::ne.Scalar", "aten::bitwise_and.Tensor", "aten::masked_select", "aten::copy_", "aten::_copy_from",
               "aten::empty.memory_format", "aten::empty_strided", "aten::as_strided", "aten::view",
               "webgpu::fused_add_relu", "webgpu::create_buffer", "webgpu::write_buffer", "webgpu::run_fused"):
        line = [l for l in table(op).splitlines() if l.startswith("PrivateUse1:")]
        assert line and "fallback" not in line[0].lower(), f"{op} has no PrivateUse1 kernel: {line}"
    assert torch_webgpu._C.version().startswith("twg")


def test_compile_backend_partitions_the_chain_into_one_ahead_of_time_program(abi):
    import torch_webgpu  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    from torch.fx.experimental.proxy_tensor import make_fx
    from torch_webgpu.compiler import webgpu_compiler as wc

    def chain(a, b, c):
        y = torch.relu(torch.nn.functional.silu(a + b) + c)
        m = torch.bitwise_and(torch.eq(y, 0), torch.ne(a, 0))
        return m, a.view(-1)

    with FakeTensorMode() as mode:
        args = [torch.empty(4, 8, 8, device="webgpu") for _ in range(3)]
        gm = make_fx(chain)(*args)
    groups = wc.partition(gm.graph)
    assert len(groups) == 1 and len(groups[0]) == 7
    prog, inputs, outs = wc.build_program(groups[0])
    assert [tuple(i) for i in prog.instrs] == [tuple(i) for i in abi.CHAIN_MASK_PROGRAM]
    assert len(inputs) == 3 and len(outs) == 1 and prog.out_dtypes() == [11]
    handle = torch.ops.webgpu.compile_fused(*prog.columns())
    assert torch.ops.webgpu.fused_kind(handle) == 0

    # a mask that feeds only masked_select(a, mask) is recognised as a fused select on input 0 ...
    def select_only(a, b, c):
        y = torch.relu(torch.nn.functional.silu(a + b) + c)
        return torch.masked_select(a, torch.bitwise_and(torch.eq(y, 0), torch.ne(a, 0)))

    with FakeTensorMode(shape_env=torch.fx.experimental.symbolic_shapes.ShapeEnv()):
        gm_sel = make_fx(select_only)(*[torch.empty(4, 8, 8, device="webgpu") for _ in range(3)])
    (grp,) = wc.partition(gm_sel.graph)
    prog_s, inputs_s, outs_s = wc.build_program(grp)
    sel_node, src_index = wc.select_pattern(grp, inputs_s, outs_s)
    assert sel_node.target is torch.ops.aten.masked_select.default and src_index == 0
    # ... but not when the mask is also returned
    assert wc.select_pattern(groups[0], inputs, outs) is None

    # a consumer in the middle splits the run; different iteration shapes do not fuse
    def split(a, b):
        t = torch.relu(a + b)
        s = t.sum()            # reads a value of the open group
        u = torch.nn.functional.silu(t) * 2.0
        v = (a[:, :1] + 1.0) * 3.0
        return s, u, v

    with FakeTensorMode():
        gm2 = make_fx(split)(torch.empty(6, 5, device="webgpu"), torch.empty(6, 5, device="webgpu"))
    shapes = [tuple(g[0].meta["val"].shape) for g in wc.partition(gm2.graph)]
    assert shapes == [(6, 5), (6, 5), (6, 1)]


def test_shard_ranges_and_offsets():
    from torch_webgpu.sharding import exclusive_offsets, shard_range
    for total in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    assert exclusive_offsets([3, 0, 5]) == [0, 3, 3]
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist
    from oracle import oracle
    from torch_webgpu.sharding import global_segment, shard_range
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the same batch on every rank (seeded); each rank handles its block with the CPU oracle
        rng = np.random.default_rng(7)
        a, b, c = (rng.standard_normal((6, 33, 17)).astype(np.float32) for _ in range(3))
        a[::2, ::3] = 0.0
        lo, hi = shard_range(a.shape[0], rank, world)
        m = oracle.chain_mask(a[lo:hi], b[lo:hi], c[lo:hi])
        sel = oracle.masked_select(a[lo:hi], m)
        offset, total, counts = global_segment(sel.size)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), sel=sel, offset=offset, total=total, counts=np.array(counts))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_reproduces_the_single_rank_result(tmp_path):
    """world_size 2 on gloo: concatenating the shards at the gathered offsets equals one rank."""
    import torch.multiprocessing as mp
    from oracle import oracle
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    rng = np.random.default_rng(7)
    a, b, c = (rng.standard_normal((6, 33, 17)).astype(np.float32) for _ in range(3))
    a[::2, ::3] = 0.0
    ref = oracle.masked_select(a, oracle.chain_mask(a, b, c))
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(2)]
    assert int(parts[0]["total"]) == int(parts[1]["total"]) == ref.size
    assert int(parts[0]["offset"]) == 0 and int(parts[1]["offset"]) == parts[0]["sel"].size
    out = np.empty(ref.size, np.float32)
    for p in parts:
        out[int(p["offset"]): int(p["offset"]) + p["sel"].size] = p["sel"]
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))


def test_tracing_switch_and_ranges_without_a_profiler(abi):
    """NVTX ranges are off by default, can be switched on and off, and a traced call behaves like an
    untraced one (here: a call that fails its argument check, so no GPU is needed)."""
    L = abi.lib()
    assert L.twg_get_tracing() == (1 if os.environ.get("TWG_NVTX", "0") not in ("", "0") else 0)
    abi.check(L.twg_set_tracing(1))
    assert L.twg_get_tracing() == 1
    assert L.twg_unary_f32(1, None, None, None, None) == abi.TWG_ERR_INVALID
    assert b"descriptor" in L.twg_last_error()
    abi.check(L.twg_set_tracing(0))
    assert L.twg_get_tracing() == 0
    assert L.twg_unary_f32(1, None, None, None, None) == abi.TWG_ERR_INVALID


def _share_main(rank: int, world: int, port: int, out_dir: str) -> None:
    from torch_webgpu.sharding import Rendezvous
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    os.environ.pop("TORCHELASTIC_USE_AGENT_STORE", None)
    rdv = Rendezvous.from_env()
    got = rdv.share(f"handle-of-{rank}".encode() * (rank + 1))
    uid = rdv.broadcast(b"\x07" * 128 if rank == 0 else None)
    rdv.barrier()
    with open(os.path.join(out_dir, f"share{rank}.txt"), "w") as f:
        f.write(repr((rdv.rank, rdv.world, got, uid)))


def test_rendezvous_channel_passes_startup_data_between_two_ranks(tmp_path):
    """The host-side channel that carries the NCCL unique id and the mailbox handles at start-up."""
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_share_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    expect = [b"handle-of-0", b"handle-of-1" * 2]
    for r in range(2):
        rank, world, got, uid = eval((tmp_path / f"share{r}.txt").read_text())
        assert (rank, world, got, uid) == (r, 2, expect, b"\x07" * 128)
    from torch_webgpu.sharding import Rendezvous
    solo = Rendezvous(None, 0, 1)
    assert solo.share(b"x") == [b"x"] and solo.broadcast(b"y") == b"y"


def test_communicator_entry_points_fail_cleanly_on_the_host(abi):
    """Bad arguments and a missing NCCL library come back as status codes with a message - no
    crash, no exception from the C side, nothing touches a GPU."""
    import subprocess
    import sys
    L = abi.lib()
    comm = ctypes.c_void_p(123)
    assert L.twg_comm_init_rank(ctypes.c_char_p(b"\0" * 128), 0, 2, ctypes.byref(comm)) == abi.TWG_ERR_INVALID
    assert comm.value is None and b"all zeros" in L.twg_last_error()
    assert L.twg_comm_init_rank(ctypes.c_char_p(b"\1" * 128), 2, 2, ctypes.byref(comm)) == abi.TWG_ERR_INVALID
    assert L.twg_comm_init_rank(None, 0, 1, ctypes.byref(comm)) == abi.TWG_ERR_INVALID
    assert L.twg_allgather_i64(None, None, None, 1, None) == abi.TWG_ERR_INVALID
    assert L.twg_comm_destroy(None) == abi.TWG_OK
    x = ctypes.c_void_p()
    assert L.twg_exchange_create(0, 17, 8, ctypes.byref(x)) == abi.TWG_ERR_INVALID       # too many ranks
    assert L.twg_exchange_create(3, 2, 8, ctypes.byref(x)) == abi.TWG_ERR_INVALID        # rank outside the world
    assert L.twg_exchange_create(0, 2, 3, ctypes.byref(x)) == abi.TWG_ERR_INVALID        # odd ring
    assert L.twg_exchange_publish(None, 1, None, None) == abi.TWG_ERR_INVALID
    assert L.twg_exchange_wait(None, 1, None, None, None, None, 0) == abi.TWG_ERR_INVALID
    assert L.twg_exchange_destroy(None) == abi.TWG_OK
    # a library path that does not exist: TWG_ERR_UNSUPPORTED from every NCCL entry point (own
    # process, because the path is only honoured before the first NCCL call)
    code = (
        "import ctypes, sys\n"
        f"sys.path.insert(0, {str(REPO / 'torch-webgpu_b200')!r})\n"
        "from torch_webgpu import abi\n"
        "L = abi.lib()\n"
        "assert L.twg_comm_set_nccl_path(b'/nonexistent/libnccl.so.2') == 0\n"
        "buf = ctypes.create_string_buffer(128)\n"
        "rc = L.twg_comm_unique_id(buf)\n"
        "assert rc == abi.TWG_ERR_UNSUPPORTED, rc\n"
        "assert b'/nonexistent/libnccl.so.2' in L.twg_last_error()\n"
        "comm = ctypes.c_void_p()\n"
        "assert L.twg_comm_init_rank(ctypes.c_char_p(b'\\x01' * 128), 0, 1, ctypes.byref(comm)) == abi.TWG_ERR_UNSUPPORTED\n"
        "print('ok')\n")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stderr
