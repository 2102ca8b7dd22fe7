"""Parity of the CUDA path with the CPU oracle, driven through the C ABI (ctypes -> libtwg.so).

Every case uploads seeded inputs, makes ONE library call and compares the download with
oracle/twg_oracle.c on the same inputs: bit-exact for add / mul / relu / abs / comparisons /
bitwise_and / masked_select / copies, max(2 ulp, 1e-6 relative) for silu, the same plus a 2e-6
absolute floor for GELU.  The golden PyTorch-ATen fixtures are checked as well.
"""
from __future__ import annotations

import numpy as np
import pytest

from oracle import oracle
from util import CVT_NAMES, assert_bit_equal, assert_close_ulp, cvt_case

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 2, 3, 4, 5, 63, 64, 65, 1023, 4095, 4096, 4097, 100003]


@pytest.fixture(scope="module")
def abi():
    from torch_webgpu import abi as _abi
    assert _abi.device_count() >= 1, "no CUDA device visible"
    return _abi


def rnd(n, seed, lo=-8.0, hi=8.0):
    rng = np.random.default_rng(seed)
    return (rng.random(n, dtype=np.float32) * (hi - lo) + lo).astype(np.float32)


def small_ints(n, seed):
    return np.random.default_rng(seed).integers(-2, 3, n).astype(np.float32)


def b(a):
    return a.view(np.bool_)


# ------------------------------------------------------------------------------------------
# golden fixtures (PyTorch CPU ATen outputs, reference-test known answers)
# ------------------------------------------------------------------------------------------
def test_known_answers_of_the_reference_tests(abi, golden):
    out = abi.binary("add", golden["kat_add_a"], golden["kat_add_b"])
    assert np.allclose(out, golden["kat_add_expected_handwritten"])          # tests/ops/test_add.py:10
    assert_bit_equal(out, golden["kat_add_out"], "add")
    out = abi.binary("fused_add_relu", golden["kat_add_a"], golden["kat_add_b"])
    assert np.allclose(out, golden["kat_fused_add_relu_expected_handwritten"])  # tests/test_dev.py:18
    for i in range(4):
        x = golden[f"kat_act{i}_x"]
        assert np.allclose(abi.unary("gelu_tanh", x), golden[f"kat_act{i}_gelu"], atol=1e-3)  # test_gelu.py:14
        assert np.allclose(abi.unary("silu", x), golden[f"kat_act{i}_silu"], atol=1e-6)       # test_silu.py:13
        assert_close_ulp(abi.unary("gelu_erf", x), golden[f"kat_act{i}_gelu"], abs_floor=2e-6, what="gelu")
        assert_close_ulp(abi.unary("silu", x), golden[f"kat_act{i}_silu"], what="silu")
        assert_bit_equal(abi.unary("relu", x), golden[f"kat_act{i}_relu"], "relu")


def test_edge_values_against_aten(abi, golden):
    x, y = golden["edge_x"], golden["edge_y"]
    assert_bit_equal(abi.binary("add", x, y), golden["edge_add"], "edge add", any_nan=True)
    assert_bit_equal(abi.binary("add", x, y, alpha=2.5), golden["edge_add_alpha"], "edge add alpha", any_nan=True)
    assert_bit_equal(abi.unary("relu", x), golden["edge_relu"], "edge relu")  # relu passes NaN through untouched
    assert_bit_equal(abi.compare("eq", x, y), b(golden["edge_eq"]), "edge eq")
    assert_bit_equal(abi.compare("ne", x, 0.0), b(golden["edge_ne0"]), "edge ne0")
    assert_bit_equal(abi.compare("eq", x, 0.0), b(golden["edge_eq0"]), "edge eq0")
    keep = (np.abs(x) <= 1e4) | np.isnan(x)
    assert_close_ulp(abi.unary("silu", x[keep]), golden["edge_silu"][keep], what="edge silu")


def test_random_cases_against_aten(abi, golden):
    x, y = golden["rnd_x"], golden["rnd_y"]
    assert_bit_equal(abi.binary("add", x, y), golden["rnd_add"], "add")
    assert_bit_equal(abi.binary("add", x, y, alpha=-0.75), golden["rnd_add_alpha"], "add alpha")
    assert_bit_equal(abi.binary("mul", x, y), golden["rnd_mul"], "mul")
    assert_bit_equal(abi.unary("relu", x), golden["rnd_relu"], "relu")
    assert_bit_equal(abi.unary("abs", x), golden["rnd_abs"], "abs")
    assert_close_ulp(abi.unary("silu", x), golden["rnd_silu"], what="silu")
    assert_close_ulp(abi.unary("gelu_erf", x), golden["rnd_gelu"], abs_floor=2e-6, what="gelu erf")
    assert_close_ulp(abi.unary("gelu_tanh", x), golden["rnd_gelu_tanh"], abs_floor=2e-6, what="gelu tanh")
    p, q = golden["rnd_p"], golden["rnd_q"]
    m1, m2 = abi.compare("eq", p, q), abi.compare("ne", p, 0.0)
    assert_bit_equal(m1, b(golden["rnd_eq"]), "eq")
    assert_bit_equal(m2, b(golden["rnd_ne0"]), "ne")
    assert_bit_equal(abi.bitwise_and(m1, m2), b(golden["rnd_and"]), "and")
    assert_bit_equal(abi.bitwise_and(golden["rnd_i1"], golden["rnd_i2"]), golden["rnd_and_i32"], "and i32")
    s = golden["lay_s"]
    assert_bit_equal(abi.unary("relu", s.T), golden["lay_relu_t"], "relu transposed")
    assert_bit_equal(abi.binary("add", s, golden["lay_row"]), golden["lay_add_row"], "add row")
    assert_bit_equal(abi.binary("add", s, golden["lay_col"], alpha=3.0), golden["lay_add_col"], "add col")
    assert_bit_equal(abi.binary("add", golden["lay_row"], golden["lay_col"]), golden["lay_add_outer"], "add outer")
    src = golden["ms_src"]
    for tag in ("001", "05", "099"):
        mk = b(golden[f"ms_mask_{tag}"])
        assert_bit_equal(abi.masked_select(src, mk), golden[f"ms_out_{tag}"], f"masked_select {tag}")
        assert_bit_equal(abi.masked_select(src.T, mk.T), golden[f"ms_out_t_{tag}"], f"masked_select T {tag}")
    assert_bit_equal(abi.masked_select(src, b(golden["ms_mask_row"])), golden["ms_out_row"], "row mask")
    assert_bit_equal(abi.masked_select(src, b(golden["ms_mask_col"])), golden["ms_out_col"], "col mask")
    assert_bit_equal(abi.masked_select(src[:, :1], b(golden["ms_mask_col"])), golden["ms_out_bsrc"], "bcast self")


@pytest.mark.parametrize("src", CVT_NAMES)
def test_conversions(abi, golden, src):
    for dst in CVT_NAMES:
        x, want = cvt_case(golden, src, dst)
        assert_bit_equal(abi.convert(x, src, dst), want, f"{src} -> {dst} vs ATen")
        assert_bit_equal(abi.convert(x, src, dst, pad=1), want, f"{src} -> {dst} misaligned")


def test_conversions_large_and_strided(abi):
    n = 1 << 20
    x = rnd(n + 3, 101, -1000, 1000)
    for dst in ("float16", "bf16", "int32", "float64", "bool", "uint8"):
        src = np.abs(x) % 250 if dst == "uint8" else x
        assert_bit_equal(abi.convert(src, "float32", dst), oracle.convert(src, "float32", dst), f"f32 -> {dst}")
    h = oracle.convert(x, "float32", "float16")
    assert_bit_equal(abi.convert(h, "float16", "float32"), oracle.convert(h, "float16", "float32"), "f16 -> f32")
    i = np.random.default_rng(102).integers(-2**40, 2**40, n).astype(np.int64)
    assert_bit_equal(abi.convert(i, "int64", "float32"), oracle.convert(i, "int64", "float32"), "i64 -> f32")
    assert_bit_equal(abi.convert(i, "int64", "int16"), oracle.convert(i, "int64", "int16"), "i64 -> i16 wraps")
    m = x.reshape(-1)[: 512 * 300].reshape(512, 300)
    assert_bit_equal(abi.convert(m.T, "float32", "bf16"), oracle.convert(np.ascontiguousarray(m.T), "float32", "bf16"), "transposed")
    assert_bit_equal(abi.convert(m[:, ::3], "float32", "int64"), oracle.convert(np.ascontiguousarray(m[:, ::3]), "float32", "int64"), "slice")


def test_scalar_right_operands(abi):
    for n in (1, 7, 4097, 100003):
        x = rnd(n, 110 + n)
        s_arr = np.full(n, 2.5, np.float32)
        for pad in (0, 1):
            assert_bit_equal(abi.binary_scalar("add", x, 2.5, pad=pad), oracle.binary("add", x, s_arr), f"x + 2.5 n={n}")
            assert_bit_equal(abi.binary_scalar("add", x, 2.5, alpha=-0.75, pad=pad), oracle.binary("add", x, s_arr, -0.75), "x - 0.75*2.5")
            assert_bit_equal(abi.binary_scalar("mul", x, 2.5, pad=pad), oracle.binary("mul", x, s_arr), "x * 2.5")
            assert_bit_equal(abi.binary_scalar("div", x, 2.5, pad=pad), oracle.binary("div", x, s_arr), "x / 2.5")
        if n >= 4096:
            assert abi.last_path() == "strided32"   # pad = 1 is misaligned
            abi.binary_scalar("mul", x, 2.5)
            assert abi.last_path() == "dense"
    m = rnd(96 * 160, 111).reshape(96, 160)
    assert_bit_equal(abi.binary_scalar("mul", m.T, -3.0), oracle.binary("mul", np.ascontiguousarray(m.T), np.full((160, 96), -3.0, np.float32)), "transposed * scalar")


def test_sub_div_where_masked_fill(abi, golden):
    x, y, e, er = golden["rnd_x"], golden["rnd_y"], golden["edge_x"], golden["edge_y"]
    assert_bit_equal(abi.binary("add", x, y, alpha=-1.0), golden["rnd_sub"], "sub")
    assert_bit_equal(abi.binary("add", x, y, alpha=-1.75), golden["rnd_sub_alpha"], "sub alpha")
    assert_bit_equal(abi.binary("div", x, y), golden["rnd_div"], "div")
    assert_bit_equal(abi.binary("div", e, er), golden["edge_div"], "div edge", any_nan=True)
    assert_bit_equal(abi.binary("add", e, er, alpha=-1.0), golden["edge_sub"], "sub edge", any_nan=True)
    m1, m2 = b(golden["rnd_eq"]), b(golden["rnd_ne0"])
    assert_bit_equal(abi.where(m2, x, y), golden["rnd_where"], "where")
    assert_bit_equal(abi.masked_fill(x, m1, -3.5), golden["rnd_masked_fill"], "masked_fill")
    s, col, wc = golden["lay_s"], golden["lay_col"], b(golden["lay_where_cond"])
    assert_bit_equal(abi.where(wc, s, col), golden["lay_where"], "where broadcast")
    assert_bit_equal(abi.masked_fill(s.T, wc.T, 2.0), golden["lay_masked_fill_t"], "masked_fill transposed")
    # every size and alignment on the dense path, and a true transpose, against the oracle
    for n in (1, 5, 4097, 100003):
        for pad in (0, 3):
            u, v = rnd(n, 95), rnd(n, 96)
            c = np.random.default_rng(97).random(n) < 0.4
            assert_bit_equal(abi.where(c, u, v, pad=pad), oracle.where(c, u, v), f"where n={n} pad={pad}")
            assert_bit_equal(abi.masked_fill(u, c, 7.25, pad=pad), oracle.masked_fill(u, c, 7.25), f"masked_fill n={n}")
            assert_bit_equal(abi.binary("div", u, v, pad=pad), oracle.binary("div", u, v), f"div n={n} pad={pad}")
    u, v = rnd(96 * 160, 98).reshape(96, 160), rnd(96 * 160, 99).reshape(160, 96)
    c = np.random.default_rng(100).random((96, 160)) < 0.5
    assert_bit_equal(abi.where(c, u, v.T), oracle.where(c, u, np.ascontiguousarray(v.T)), "where with a transposed operand")
    assert_bit_equal(abi.binary("div", u, v.T), oracle.binary("div", u, np.ascontiguousarray(v.T)), "div transposed")


# ------------------------------------------------------------------------------------------
# dense path: every size around the vector / chunk boundaries, aligned and misaligned
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("pad", [0, 1, 3])
def test_dense_ops_all_sizes(abi, n, pad):
    x, y = rnd(n, 10 + n), rnd(n, 20 + n)
    assert_bit_equal(abi.binary("add", x, y, pad=pad), oracle.binary("add", x, y), "add")
    assert abi.last_path() == ("none" if n == 0 else "dense" if pad == 0 else "strided32")
    assert_bit_equal(abi.binary("add", x, y, alpha=0.3, pad=pad), oracle.binary("add", x, y, 0.3), "add alpha")
    assert_bit_equal(abi.unary("relu", x, pad=pad), oracle.unary("relu", x), "relu")
    assert_close_ulp(abi.unary("silu", x, pad=pad), oracle.unary("silu", x), what="silu")
    assert_close_ulp(abi.unary("gelu_erf", x, pad=pad), oracle.unary("gelu_erf", x), abs_floor=2e-6, what="gelu")
    p, q = small_ints(n, 30 + n), small_ints(n, 40 + n)
    m1, m2 = abi.compare("eq", p, q, pad=pad), abi.compare("ne", p, 0.0, pad=pad)
    assert_bit_equal(m1, oracle.compare("eq", p, q), "eq")
    assert_bit_equal(m2, oracle.compare("ne", p, 0.0), "ne")
    assert_bit_equal(abi.bitwise_and(m1, m2, pad=pad), oracle.bitwise_and(m1, m2), "and bool")


@pytest.mark.parametrize("op", ["lt", "le", "gt", "ge", "eq", "ne"])
def test_all_comparisons(abi, op):
    p, q = small_ints(5001, 1), small_ints(5001, 2)
    p[::97] = np.nan
    assert_bit_equal(abi.compare(op, p, q), oracle.compare(op, p, q), op)
    assert_bit_equal(abi.compare(op, p, 1.0), oracle.compare(op, p, 1.0), op + " scalar")


@pytest.mark.parametrize("dtype", [np.uint8, np.int16, np.int32, np.int64])
def test_integer_bitwise_and(abi, dtype):
    rng = np.random.default_rng(3)
    info = np.iinfo(dtype)
    a = rng.integers(info.min, info.max, 10007, dtype=dtype)
    c = rng.integers(info.min, info.max, 10007, dtype=dtype)
    assert_bit_equal(abi.bitwise_and(a, c), a & c, "and int")
    a2, c2 = a[:9999].reshape(99, 101), c[:9999].reshape(99, 101)
    assert_bit_equal(abi.bitwise_and(a2.T, c2.T), a2.T & c2.T, "and int transposed")
    assert_bit_equal(abi.bitwise_and(a2[:, ::3], c2[:, ::3]), a2[:, ::3] & c2[:, ::3], "and int sliced")


# ------------------------------------------------------------------------------------------
# strided / broadcast / permuted layouts
# ------------------------------------------------------------------------------------------
def test_true_transpose_uses_the_tile_kernel(abi):
    for rows, cols in [(33, 65), (128, 96), (1000, 1031), (17, 4096)]:
        x = rnd(rows * cols, rows).reshape(rows, cols)
        got = abi.unary("relu", x.T)  # output dense in the transposed logical shape
        assert abi.last_path() == "tile", (rows, cols)
        assert_bit_equal(got, oracle.unary("relu", x.T), "relu transpose")
        got = abi.unary("silu", x.T)
        assert_close_ulp(got, oracle.unary("silu", x.T), what="silu transpose")
        y = rnd(rows * cols, cols).reshape(cols, rows)
        assert_bit_equal(abi.binary("add", x.T, y), oracle.binary("add", x.T, y), "add transposed + dense")
        assert abi.last_path() == "tile"
        p, q = small_ints(rows * cols, 5).reshape(rows, cols), small_ints(rows * cols, 6).reshape(cols, rows)
        assert_bit_equal(abi.compare("eq", p.T, q), oracle.compare("eq", p.T, q), "eq transposed")
        m = (p > 0)
        assert_bit_equal(abi.bitwise_and(m.T, (q < 1)), oracle.bitwise_and(m.T, (q < 1)), "and transposed")
        assert_bit_equal(abi.copy(x.T), np.ascontiguousarray(x.T), "copy transposed")
        assert abi.last_path() == "tile"


def test_transposes_with_vector_tiles(abi):
    """Shapes whose strides allow 128-bit accesses in interior tiles (multiples of 4), with scalar
    edge tiles around them, operands of both orientations, and a misaligned case that must not."""
    for rows, cols in [(256, 192), (260, 200), (64, 64), (68, 1028)]:
        x = rnd(rows * cols, rows + 1).reshape(rows, cols)
        y = rnd(rows * cols, cols + 2).reshape(cols, rows)
        for pad in (0, 1):
            assert_bit_equal(abi.unary("relu", x.T, pad=pad), oracle.unary("relu", x.T), f"relu T {rows}x{cols} pad={pad}")
            assert abi.last_path() == "tile"
            assert_bit_equal(abi.binary("add", x.T, y, alpha=0.5, pad=pad), oracle.binary("add", x.T, y, 0.5), "add T + dense")
            assert_bit_equal(abi.binary("mul", y, x.T, pad=pad), oracle.binary("mul", y, x.T), "dense * T")
        assert_close_ulp(abi.unary("gelu_erf", x.T), oracle.unary("gelu_erf", x.T), abs_floor=2e-6, what="gelu T")
        out_like = np.empty((cols, rows), np.float32).T   # logical [rows, cols], dense along dimension 0
        assert_bit_equal(abi.unary("relu", x, out_like=out_like), oracle.unary("relu", x), "relu into transposed out")
        assert abi.last_path() == "tile"
        c = np.random.default_rng(rows).random((cols, rows)) < 0.5
        assert_bit_equal(abi.where(c, x.T, y), oracle.where(c, np.ascontiguousarray(x.T), y), "where with a transposed operand")


def test_transposed_output_layout(abi):
    x = rnd(96 * 80, 7).reshape(96, 80)
    out_like = np.empty((80, 96), np.float32).T  # logical [96,80], dense along dimension 0
    got = abi.unary("relu", x, out_like=out_like)
    assert abi.last_path() == "tile"
    assert_bit_equal(got, oracle.unary("relu", x), "relu into transposed out")


def test_slices_broadcasts_and_many_dims(abi):
    x = rnd(64 * 130, 8).reshape(64, 130)
    assert_bit_equal(abi.unary("relu", x[:, ::2]), oracle.unary("relu", x[:, ::2]), "stride-2 slice")
    assert abi.last_path() == "strided32"
    assert_bit_equal(abi.unary("relu", x[3:, 5:77]), oracle.unary("relu", x[3:, 5:77]), "offset window")
    row, col = rnd(64, 9).reshape(64, 1), rnd(130, 10).reshape(1, 130)
    assert_bit_equal(abi.binary("add", x, row), oracle.binary("add", x, row), "row broadcast")
    assert_bit_equal(abi.binary("add", x, col, alpha=2.0), oracle.binary("add", x, col, 2.0), "col broadcast")
    assert_bit_equal(abi.binary("add", row, col), oracle.binary("add", row, col), "outer broadcast")
    scalar = rnd(1, 11).reshape(1, 1)
    assert_bit_equal(abi.binary("mul", x, scalar), oracle.binary("mul", x, scalar), "scalar broadcast")
    # negative strides take the 64-bit index path
    assert_bit_equal(abi.unary("relu", x[::-1, ::-1]), oracle.unary("relu", x[::-1, ::-1]), "flipped")
    assert abi.last_path() == "strided64"
    assert_bit_equal(abi.copy(x[::-1, ::3]), np.ascontiguousarray(x[::-1, ::3]), "copy flipped slice")
    for ndim in range(1, 9):
        shape = [3, 2, 4, 2, 3, 2, 2, 3][:ndim]
        base = rnd(int(np.prod(shape)), 100 + ndim).reshape(shape)
        perm = list(reversed(range(ndim)))
        v = base.transpose(perm)
        assert_bit_equal(abi.unary("relu", v), oracle.unary("relu", v), f"permuted {ndim}-d")
        w = rnd(int(np.prod(shape)), 200 + ndim).reshape(v.shape)
        assert_bit_equal(abi.binary("add", v, w[..., ::1]), oracle.binary("add", v, w), f"permuted add {ndim}-d")
        assert_bit_equal(abi.copy(v), np.ascontiguousarray(v), f"permuted copy {ndim}-d")
    with pytest.raises(abi.TwgError):
        abi.unary("relu", np.zeros((1,) * 9, np.float32))


def test_copy_every_element_size(abi):
    rng = np.random.default_rng(12)
    for dtype in (np.uint8, np.uint16, np.float32, np.float64, np.complex128):
        a = rng.integers(0, 255, 50 * 70 * np.dtype(dtype).itemsize, dtype=np.uint8).view(dtype).reshape(50, 70)
        for v in (a.T, a[:, ::2], a[::3, 1:], a):
            assert_bit_equal(abi.copy(v).view(np.uint8), np.ascontiguousarray(v).view(np.uint8), f"copy {dtype}")


def test_byte_operands_far_apart_use_64bit_offsets(abi):
    # a bool view whose rows are 2^30 bytes apart: offsets no longer fit 32 bits
    big = np.zeros(3 << 30, np.uint8)
    rng = np.random.default_rng(13)
    view = big.reshape(3, 1 << 30)[:, :40]
    view[...] = rng.integers(0, 2, (3, 40))
    other = rng.integers(0, 2, (3, 40)).astype(np.uint8)
    got = abi.bitwise_and(view.view(np.bool_), other.view(np.bool_))
    assert abi.last_path() == "strided64"
    assert_bit_equal(got, (view & other).view(np.bool_), "far-apart rows")


# ------------------------------------------------------------------------------------------
# masked_select
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [0, 1, 5, 4095, 4096, 4097, 3 * 4096 + 17, 1 << 20, (1 << 22) + 3])
@pytest.mark.parametrize("p", [0.0, 0.01, 0.5, 0.99, 1.0])
def test_masked_select_dense(abi, n, p):
    x = rnd(n, 50 + n)
    mask = np.random.default_rng(60 + n).random(n) < p
    got = abi.masked_select(x, mask)
    assert_bit_equal(got, oracle.masked_select(x, mask), f"masked_select n={n} p={p}")
    if n:
        assert abi.last_path() == "dense"


def test_masked_select_mixed_density(abi):
    """Chunks on either side of the sparse / dense decision inside one call, and a sparse row mask."""
    n = (1 << 22) + 4099
    x = rnd(n, 71)
    rng = np.random.default_rng(72)
    mask = np.zeros(n, np.bool_)
    third = n // 3
    mask[:third] = rng.random(third) < 0.9
    mask[third:2 * third] = rng.random(third) < 0.002
    mask[2 * third:] = rng.random(n - 2 * third) < 0.06
    mask[n - 1] = True
    assert_bit_equal(abi.masked_select(x, mask), oracle.masked_select(x, mask), "mixed density")
    rows, cols = 2048, 1024
    y = rnd(rows * cols, 73).reshape(rows, cols)
    rowmask = (rng.random((rows, 1)) < 0.01)
    assert_bit_equal(abi.masked_select(y, rowmask), oracle.masked_select(y, rowmask), "sparse row mask")
    assert abi.last_path() == "dense"


@pytest.mark.parametrize("pad", [0, 1, 2, 3])
def test_masked_select_runs_of_full_and_empty_spans(abi, pad):
    """Whole 512-element spans selected or empty, at every output alignment: the straight-copy path
    of full spans, its hand-over to and from staged spans, skipped spans, and output runs that start
    and end inside a 16-byte vector."""
    n = 37 * 4096 + 300
    x = rnd(n, 74)
    rng = np.random.default_rng(75 + pad)
    mask = np.zeros(n, np.bool_)
    for s0 in range(0, n, 512):
        kind = rng.integers(0, 5)
        if kind == 0:
            mask[s0:s0 + 512] = True
        elif kind == 1:
            mask[s0:s0 + 512] = rng.random(min(512, n - s0)) < 0.5
        elif kind == 2:
            mask[s0 + rng.integers(0, 8)] = True          # a lone element: shifts the alignment of what follows
        elif kind == 3:
            mask[s0:s0 + 512] = rng.random(min(512, n - s0)) < 0.97
    assert_bit_equal(abi.masked_select(x, mask, pad=pad), oracle.masked_select(x, mask), f"span runs pad={pad}")
    ones = np.ones(n, np.bool_)
    assert_bit_equal(abi.masked_select(x, ones, pad=pad), x, f"all true pad={pad}")
    ones[0] = False                                          # every full span now starts one element off a vector
    assert_bit_equal(abi.masked_select(x, ones, pad=pad), x[1:], f"all true but the first, pad={pad}")
    rows, cols = 300, 1536                                   # row mask: selected rows are three full spans each
    y = rnd(rows * cols, 76).reshape(rows, cols)
    rowmask = rng.random((rows, 1)) < 0.5
    assert_bit_equal(abi.masked_select(y, rowmask, pad=pad), oracle.masked_select(y, rowmask), f"row mask pad={pad}")


@pytest.mark.parametrize("p", [0.0, 0.01, 0.3, 0.5, 0.99, 1.0])
def test_masked_select_large_inputs(abi, p):
    """About ten million elements: chunks of the longest kind, several per CTA slot, a partial last one."""
    n = 320 * 32768 + 12345
    x = rnd(n, 77)
    mask = np.random.default_rng(78).random(n) < p
    assert_bit_equal(abi.masked_select(x, mask), oracle.masked_select(x, mask), f"large n p={p}")
    assert abi.last_path() == "dense"


def test_masked_select_large_mixed_density_and_row_mask(abi):
    n = 310 * 32768 + 4099
    x = rnd(n, 79)
    rng = np.random.default_rng(80)
    mask = np.zeros(n, np.bool_)
    for c0 in range(0, n, 32768):               # every chunk gets its own density, some are sparse, some full
        kind = rng.integers(0, 6)
        seg = slice(c0, min(c0 + 32768, n))
        width = seg.stop - seg.start
        if kind == 0:
            mask[seg] = True
        elif kind == 1:
            mask[seg] = rng.random(width) < 0.002
        elif kind == 2:
            mask[seg] = rng.random(width) < 0.05
        elif kind == 3:
            mask[seg] = rng.random(width) < 0.6
        elif kind == 4:
            mask[seg] = np.repeat(rng.random((width + 511) // 512) < 0.5, 512)[:width]   # whole spans on or off
    assert_bit_equal(abi.masked_select(x, mask), oracle.masked_select(x, mask), "large mixed density")
    assert_bit_equal(abi.masked_select(x, mask, pad=1), oracle.masked_select(x, mask), "large mixed density, misaligned (strided path)")
    rows, cols = 5000, 2048
    y = rnd(rows * cols, 81).reshape(rows, cols)
    for density in (0.5, 0.02):
        rowmask = rng.random((rows, 1)) < density
        assert_bit_equal(abi.masked_select(y, rowmask), oracle.masked_select(y, rowmask), f"large row mask {density}")
        assert abi.last_path() == "dense"
    rows, cols = 7001, 1500                     # rows that are not a multiple of 32 elements long
    y = rnd(rows * cols, 82).reshape(rows, cols)
    rowmask = rng.random((rows, 1)) < 0.5
    assert_bit_equal(abi.masked_select(y, rowmask), oracle.masked_select(y, rowmask), "large row mask, odd row length")


@pytest.mark.parametrize("pad", [1, 2, 3])
def test_masked_select_misaligned(abi, pad):
    n = 5 * 4096 + 123
    x = rnd(n, 70)
    mask = np.random.default_rng(71).random(n) < 0.4
    assert_bit_equal(abi.masked_select(x, mask, pad=pad), oracle.masked_select(x, mask), "misaligned")
    assert abi.last_path() == "strided32"


def test_masked_select_broadcast_and_strided(abi):
    rng = np.random.default_rng(72)
    x = rnd(300 * 517, 73).reshape(300, 517)
    full = rng.random((300, 517)) < 0.5
    rowm = rng.random((300, 1)) < 0.5
    colm = rng.random((1, 517)) < 0.5
    assert_bit_equal(abi.masked_select(x, rowm), oracle.masked_select(x, rowm), "row mask")
    assert_bit_equal(abi.masked_select(x, colm), oracle.masked_select(x, colm), "col mask")
    assert_bit_equal(abi.masked_select(x.T, full.T), oracle.masked_select(x.T, full.T), "both transposed")
    assert_bit_equal(abi.masked_select(x.T, np.ascontiguousarray(full.T)), oracle.masked_select(x.T, full.T), "self transposed")
    assert_bit_equal(abi.masked_select(x[:, :1], colm), oracle.masked_select(x[:, :1], colm), "self broadcast")
    assert_bit_equal(abi.masked_select(x[::2, ::3], full[::2, ::3]), oracle.masked_select(x[::2, ::3], full[::2, ::3]), "sliced")
    x4 = rnd(6 * 5 * 7 * 9, 74).reshape(6, 5, 7, 9)
    m4 = rng.random((6, 1, 7, 1)) < 0.5
    assert_bit_equal(abi.masked_select(x4, m4), oracle.masked_select(x4, m4), "4-d broadcast mask")
    with pytest.raises(RuntimeError):
        abi.masked_select(x, np.ones(x.shape, np.uint8))


def test_masked_select_nonzero_bytes_count_as_true(abi):
    x = rnd(9000, 75)
    raw = np.random.default_rng(76).integers(0, 256, 9000).astype(np.uint8)
    raw[::3] = 0
    got = abi.masked_select(x, raw.view(np.bool_))
    assert_bit_equal(got, x[raw != 0], "non 0/1 mask bytes")


def test_masked_select_bounded_wait_reports_timeout(abi):
    """The look-back wait must run out and report, never hang: tile 0 withholds its count."""
    n = 64 * 4096
    x = rnd(n, 77)
    mask = np.random.default_rng(78).random(n) < 0.5
    try:
        abi.check(abi.lib().twg_masked_select_set_poll_budget(-200))
        _, status = abi.masked_select(x, mask, return_status=True)
        assert status == abi.TWG_ERR_TIMEOUT
        with pytest.raises(abi.TwgError):
            abi.masked_select(x, mask)
    finally:
        abi.check(abi.lib().twg_masked_select_set_poll_budget(0))
    # the context is still usable and the next call is correct
    assert_bit_equal(abi.masked_select(x, mask), oracle.masked_select(x, mask), "after timeout")


def test_masked_select_workspace_is_validated(abi):
    import ctypes
    x = abi.DeviceArray(rnd(10000, 79))
    m = abi.DeviceArray(np.ones(10000, np.uint8))
    d = abi.make_desc((10000,), [x, m])
    out, res, ws = abi.DeviceBuffer(40000), abi.DeviceBuffer(16), abi.DeviceBuffer(256)
    rc = abi.lib().twg_masked_select_f32(ctypes.byref(d), x.ptr, m.ptr, out.ptr, res.ptr, ws.ptr, 8, None)
    assert rc == abi.TWG_ERR_INVALID
    assert b"workspace" in abi.lib().twg_last_error()


# ------------------------------------------------------------------------------------------
# fused programs
# ------------------------------------------------------------------------------------------
def test_fused_chain_ahead_of_time_kernel(abi, golden):
    a, bb, c = golden["chain_a"], golden["chain_b"], golden["chain_c"]
    (m,), kind = abi.fused(abi.CHAIN_MASK_PROGRAM, [a, bb, c], [np.bool_])
    assert kind == "aot"
    assert_bit_equal(m, oracle.chain_mask(a, bb, c), "chain mask vs oracle")
    assert_bit_equal(m, b(golden["chain_m"]), "chain mask vs ATen")
    assert_bit_equal(abi.masked_select(a, m), golden["chain_sel"], "chain select")
    n = 1 << 20
    a, bb, c = rnd(n, 80, -3, 3), rnd(n, 81, -3, 3), rnd(n, 82, -3, 3)
    a[::5] = 0.0
    (m,), _ = abi.fused(abi.CHAIN_MASK_PROGRAM, [a, bb, c], [np.bool_])
    y_ref, m_ref = oracle.chain_mask(a, bb, c, want_y=True)
    # silu may differ by an ulp, which can flip relu's "exactly zero" only next to zero
    diff = m != m_ref
    assert diff.sum() <= 4
    assert np.all(np.abs(y_ref[diff]) < 1e-6)


def test_fused_program_compiled_at_run_time(abi):
    F = abi
    prog = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_INPUT_F32, 1, 0, 0.0), (F.F_GELU_ERF, 0, 0, 0.0), (F.F_MUL, 2, 1, 0.0),
            (F.F_CONST_F32, 0, 0, 0.5), (F.F_GT, 3, 4, 0.0), (F.F_ABS, 3, 0, 0.0), (F.F_OUTPUT, 6, 0, 0.0),
            (F.F_OUTPUT, 5, 1, 0.0)]
    for shape_x, shape_y in [((100003,), (100003,)), ((257, 130), (257, 1)), ((64, 96), (96, 64))]:
        x = rnd(int(np.prod(shape_x)), 83).reshape(shape_x)
        y = rnd(int(np.prod(shape_y)), 84).reshape(shape_y)
        if shape_y == (96, 64):
            y = y.T
        (val, flag), kind = abi.fused(prog, [x, y], [np.float32, np.bool_])
        assert kind == "nvrtc"
        g = oracle.unary("gelu_erf", x)
        ref = oracle.binary("mul", g, np.broadcast_to(y, x.shape).copy())
        # the product is computed from this build's gelu, so compare against what it implies
        got_g = abi.unary("gelu_erf", x)
        exact = oracle.unary("abs", oracle.binary("mul", got_g, np.broadcast_to(y, x.shape).copy()))
        assert_bit_equal(val, exact, "fused abs(gelu*y)")
        assert_close_ulp(val, np.abs(ref), abs_floor=2e-5, what="fused vs oracle")
        assert_bit_equal(flag, oracle.compare("gt", oracle.binary("mul", got_g, np.broadcast_to(y, x.shape).copy()), 0.5), "fused flag")


@pytest.mark.parametrize("n", [1, 5, 127, 128, 129, 4095, 7680, 7681, 8193, 100003, (1 << 22) + 7, (1 << 24) + 513])
def test_fused_select_equals_mask_then_masked_select(abi, n):
    a, bb, c = rnd(n, 85, -3, 3), rnd(n, 86, -3, 3), rnd(n, 87, -3, 3)
    a[::5] = 0.0
    (m,), _ = abi.fused(abi.CHAIN_MASK_PROGRAM, [a, bb, c], [np.bool_])
    sel, kind = abi.fused_select(abi.CHAIN_MASK_PROGRAM, [a, bb, c], 0)
    assert kind == "aot"
    assert_bit_equal(sel, abi.masked_select(a, m), "fused select vs mask + masked_select")
    assert_bit_equal(sel, oracle.masked_select(a, m), "fused select vs oracle on the same mask")


@pytest.mark.parametrize("n", [1, 31, 128, 1000, 8192 * 3 + 77, (1 << 21) + 5])
def test_predicate_bits_equal_the_bool_mask(abi, n):
    """First half of the fused select: the same predicate as bits (ahead-of-time and NVRTC kernels,
    1 / 2 / 3 inputs, i.e. 4 / 2 / 1 rounds per warp)."""
    F = abi
    a, bb, c = rnd(n, 185, -3, 3), rnd(n, 186, -3, 3), rnd(n, 187, -3, 3)
    a[::5] = 0.0
    positive = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_CONST_F32, 0, 0, 0.0), (F.F_GT, 0, 1, 0.0), (F.F_OUTPUT, 2, 0, 0.0)]
    product = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_INPUT_F32, 1, 0, 0.0), (F.F_MUL, 0, 1, 0.0), (F.F_CONST_F32, 0, 0, 0.25),
               (F.F_GT, 2, 3, 0.0), (F.F_OUTPUT, 4, 0, 0.0)]
    for prog, ins in ((abi.CHAIN_MASK_PROGRAM, [a, bb, c]), (positive, [bb]), (product, [bb, c])):
        try:
            got = abi.predicate_bits(prog, ins)
        except abi.TwgError as e:
            if e.code == abi.TWG_ERR_UNSUPPORTED and prog is not abi.CHAIN_MASK_PROGRAM:
                pytest.skip(f"NVRTC is not installed here: {e}")
            raise
        (m,), _ = abi.fused(prog, ins, [np.bool_])
        assert np.array_equal(got, m), f"predicate bits differ from the bool mask ({len(ins)} inputs, n={n})"


@pytest.mark.parametrize("spread", [4.0, 30.0, 95.0])
def test_bits_of_the_chain_equal_the_exact_chain_near_its_decision_boundary(abi, spread):
    """The ahead-of-time bits kernel decides the cfg-5 predicate from a fast silu wherever that is
    provably the exact chain's decision; here c = -silu(a + b) (1 + d) with |d| from 1e-8 to 1e-2,
    a + b across +-2 spread, so that many elements lie inside, at the edge of and just outside the
    band that is sent to the exact evaluation."""
    n = 1 << 22
    rng = np.random.default_rng(int(spread) + 300)
    a = ((rng.random(n, dtype=np.float32) * 2 - 1) * np.float32(spread)).astype(np.float32)
    bb = ((rng.random(n, dtype=np.float32) * 2 - 1) * np.float32(spread)).astype(np.float32)
    s = oracle.unary("silu", oracle.binary("add", a, bb)).astype(np.float64)
    d = 10.0 ** rng.uniform(-8, -2, n) * rng.choice([-1.0, 1.0], n)
    c = (-s * (1.0 + d)).astype(np.float32)
    got, _ = abi.predicate_bits(abi.CHAIN_MASK_PROGRAM, [a, bb, c]), None
    (m,), _ = abi.fused(abi.CHAIN_MASK_PROGRAM, [a, bb, c], [np.bool_])
    assert 0.1 < m.mean() < 0.9
    assert np.array_equal(got, m), f"{int((got != m).sum())} decisions differ from the exact chain"


@pytest.mark.parametrize("n,density", [(0, 0.5), (1, 1.0), (127, 0.5), (4096, 0.0), (4096, 1.0), (100003, 0.03),
                                       (100003, 0.5), ((1 << 22) + 9, 0.97), ((1 << 23), 1.0), ((1 << 23) + 1, 0.002)])
def test_masked_select_by_bits_matches_the_oracle(abi, n, density):
    """Second half: compaction of dense src by a bit mask (sparse, dense and full-span chunk paths)."""
    src = rnd(n, 201, -5, 5)
    mask = np.random.default_rng(202).random(n) < density
    assert_bit_equal(abi.masked_select_bits(src, mask), oracle.masked_select(src, mask), f"n={n} p={density}")


def test_fused_programs_are_reference_counted(abi):
    F = abi
    L = abi.lib()
    prog = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_CONST_F32, 0, 0, 1.25), (F.F_MUL, 0, 1, 0.0), (F.F_ABS, 2, 0, 0.0),
            (F.F_OUTPUT, 3, 0, 0.0)]
    x = rnd(5000, 93)
    h1 = abi.fused_compile(prog)
    h2 = abi.fused_compile(prog)                      # same program: same handle, second reference
    assert h1 == h2 and abi.fused_kind(h1) == "nvrtc"
    (y,), _ = abi.fused(prog, [x], [np.float32])      # third reference, launches the kernel
    assert_bit_equal(y, np.abs(x * np.float32(1.25)), "abs(1.25 x)")
    assert L.twg_fused_release(h1) == abi.TWG_OK
    assert L.twg_fused_release(h1) == abi.TWG_OK
    assert abi.fused_kind(h1) == "nvrtc"              # still alive: one reference left
    assert L.twg_fused_release(h1) == abi.TWG_OK      # last one: module unloaded, program freed
    assert L.twg_fused_release(h1) == abi.TWG_ERR_INVALID
    assert b"not a live program handle" in L.twg_last_error()
    (y2,), kind = abi.fused(prog, [x], [np.float32])  # compiling again after the release works
    assert kind == "nvrtc"
    assert_bit_equal(y2, y, "after recompilation")


def test_nvrtc_results_are_cached_on_disk(abi, tmp_path):
    """With a cache directory set, a program NVRTC has compiled once is loaded from its file the
    next time (here: after its last handle was released, which frees the in-memory copy)."""
    F = abi
    L = abi.lib()
    import ctypes
    prog = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_CONST_F32, 0, 0, 0.8125), (F.F_MUL, 0, 1, 0.0), (F.F_RELU, 2, 0, 0.0),
            (F.F_OUTPUT, 3, 0, 0.0)]
    x = rnd(7000, 94)
    hits, misses = ctypes.c_int64(), ctypes.c_int64()
    abi.check(L.twg_fused_set_cache_dir(str(tmp_path).encode()))
    try:
        abi.check(L.twg_fused_cache_stats(ctypes.byref(hits), ctypes.byref(misses)))
        h0, m0 = hits.value, misses.value
        (y1,), kind = abi.fused(prog, [x], [np.float32])
        assert kind == "nvrtc"
        abi.check(L.twg_fused_cache_stats(ctypes.byref(hits), ctypes.byref(misses)))
        assert (hits.value, misses.value) == (h0, m0 + 1)
        files = list(tmp_path.glob("twg_*.cubin"))
        assert len(files) == 1 and files[0].stat().st_size > 1000 and not list(tmp_path.glob("*.tmp.*"))
        handle = abi.fused_compile(prog)                     # same process: the in-memory cache, no file access
        abi.check(L.twg_fused_cache_stats(ctypes.byref(hits), ctypes.byref(misses)))
        assert (hits.value, misses.value) == (h0, m0 + 1)
        abi.check(L.twg_fused_release(handle))
        abi.check(L.twg_fused_release(handle))               # abi.fused's reference: the program is gone now
        (y2,), kind = abi.fused(prog, [x], [np.float32])     # compiled "again": served from the file
        abi.check(L.twg_fused_cache_stats(ctypes.byref(hits), ctypes.byref(misses)))
        assert kind == "nvrtc" and (hits.value, misses.value) == (h0 + 1, m0 + 1)
        assert_bit_equal(y2, y1, "cubin from the disk cache")
        assert_bit_equal(y1, np.maximum(x * np.float32(0.8125), 0), "relu(0.8125 x)")
        files[0].write_bytes(files[0].read_bytes()[:100])    # a damaged file is ignored and rewritten
        handle = abi.fused_compile(prog)
        abi.check(L.twg_fused_release(handle))
        abi.check(L.twg_fused_release(handle))
        (y3,), _ = abi.fused(prog, [x], [np.float32])
        abi.check(L.twg_fused_cache_stats(ctypes.byref(hits), ctypes.byref(misses)))
        assert (hits.value, misses.value) == (h0 + 1, m0 + 2) and files[0].stat().st_size > 1000
        assert_bit_equal(y3, y1, "after the damaged file")
    finally:
        abi.check(L.twg_fused_set_cache_dir(None))


def test_fused_select_on_the_decision_boundary_of_the_chain(abi):
    """Inputs placed on and next to the boundary silu(a + b) + c == 0, huge and non-finite values:
    the fused select (whose bits kernel decides most elements from a fast silu) must select exactly
    what the exact chain's mask says."""
    n = 1 << 18
    rng = np.random.default_rng(91)
    a = (rng.random(n, dtype=np.float32) * 8 - 4).astype(np.float32)
    bb = (rng.random(n, dtype=np.float32) * 8 - 4).astype(np.float32)
    k = np.arange(n) % 8
    a[k == 7] *= np.float32(11.0)                                 # a + b out to +-88: the whole range of exp
    bb[k == 7] *= np.float32(11.0)
    s = oracle.unary("silu", oracle.binary("add", a, bb))
    c = (-s).astype(np.float32)                                   # silu(a + b) + c is within a few ulp of zero
    wide = k == 7
    c[wide] = (c[wide].view(np.int32) + rng.integers(-60, 61, int(wide.sum())).astype(np.int32)).view(np.float32)
    for step, sel in ((1, k == 1), (2, k == 2), (40, k == 3), (400, k == 4)):
        c[sel] = (c[sel].view(np.int32) + step).view(np.float32)  # a few ulp to a few hundred ulp away
    for step, sel in ((1, k == 5), (300, k == 6)):
        c[sel] = (c[sel].view(np.int32) - step).view(np.float32)
    far = rng.random(n) < 0.02                                    # and some values far outside the fast range
    a[far] = rng.choice(np.array([100.0, -100.0, 3e38, -3e38, np.inf, -np.inf, np.nan, 1e-42, -1e-42, 0.0], np.float32), int(far.sum()))
    c[rng.random(n) < 0.01] = np.float32(0.0)
    (m,), _ = abi.fused(abi.CHAIN_MASK_PROGRAM, [a, bb, c], [np.bool_])
    sel, kind = abi.fused_select(abi.CHAIN_MASK_PROGRAM, [a, bb, c], 0)
    assert kind == "aot"
    assert 0.2 < m.mean() < 0.8
    assert_bit_equal(sel, oracle.masked_select(a, m), "fused select on the boundary vs the exact chain's mask")


def test_fill_every_width_and_layout(abi):
    rng = np.random.default_rng(92)
    for dtype, value in ((np.uint8, 7), (np.int16, -3), (np.float32, -0.0), (np.float32, np.nan), (np.int64, -(1 << 40)),
                         (np.float64, 2.5)):
        for n in (1, 3, 15, 16, 17, 4099, 100003):
            base = rng.integers(0, 100, n).astype(dtype)
            for pad in (0, 1, 3):
                got = abi.fill(base, value, pad=pad)
                assert_bit_equal(got.view(np.uint8), np.full(n, value, dtype).view(np.uint8), f"fill {dtype.__name__} n={n} pad={pad}")
        grid = rng.integers(0, 100, (33, 47)).astype(dtype)
        got = abi.fill(grid[::2, 1::3], value).reshape(33, 47)       # only the view's elements change
        ref = grid.copy()
        ref[::2, 1::3] = value
        assert_bit_equal(got.view(np.uint8), ref.view(np.uint8), f"strided fill {dtype.__name__}")
        assert abi.last_path() in ("strided32", "dense")
    d = abi.IterDesc()
    abi.check(abi.lib().twg_iter_contiguous(__import__("ctypes").byref(d), 1, 4))
    assert abi.lib().twg_fill(__import__("ctypes").byref(d), 3, 0, 1, None) == abi.TWG_ERR_INVALID


def test_fused_select_with_a_predicate_compiled_at_run_time(abi):
    F = abi
    # keep y where x * y > 0.25 (selected source is the second input)
    prog = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_INPUT_F32, 1, 0, 0.0), (F.F_MUL, 0, 1, 0.0), (F.F_CONST_F32, 0, 0, 0.25),
            (F.F_GT, 2, 3, 0.0), (F.F_OUTPUT, 4, 0, 0.0)]
    for n in (3, 70001, 1 << 21):
        x, y = rnd(n, 88), rnd(n, 89)
        sel, kind = abi.fused_select(prog, [x, y], 1)
        assert kind == "nvrtc"
        m = oracle.compare("gt", oracle.binary("mul", x, y), 0.25)
        assert_bit_equal(sel, oracle.masked_select(y, m), f"fused select n={n}")
    # all kept / none kept
    x = np.full(50000, 2.0, np.float32)
    sel, _ = abi.fused_select(prog, [x, x], 0)
    assert_bit_equal(sel, x, "all kept")
    sel, _ = abi.fused_select(prog, [x, -x], 0)
    assert sel.size == 0


def test_fused_select_bounded_wait_reports_timeout(abi):
    """Same look-back, same rule: chunk 0 withholds its count, the wait runs out and says so."""
    n = 64 * 8192
    a, bb, c = rnd(n, 91, -3, 3), rnd(n, 92, -3, 3), rnd(n, 93, -3, 3)
    a[::3] = 0.0
    try:
        abi.check(abi.lib().twg_masked_select_set_poll_budget(-200))
        with pytest.raises(abi.TwgError) as err:
            abi.fused_select(abi.CHAIN_MASK_PROGRAM, [a, bb, c], 0)
        assert err.value.code == abi.TWG_ERR_TIMEOUT
    finally:
        abi.check(abi.lib().twg_masked_select_set_poll_budget(0))
    (m,), _ = abi.fused(abi.CHAIN_MASK_PROGRAM, [a, bb, c], [np.bool_])
    sel, _ = abi.fused_select(abi.CHAIN_MASK_PROGRAM, [a, bb, c], 0)
    assert_bit_equal(sel, oracle.masked_select(a, m), "after timeout")


def test_fused_select_rejects_programs_that_are_not_one_predicate(abi):
    F = abi
    two_outputs = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_CONST_F32, 0, 0, 0.0), (F.F_GT, 0, 1, 0.0), (F.F_RELU, 0, 0, 0.0),
                   (F.F_OUTPUT, 2, 0, 0.0), (F.F_OUTPUT, 3, 1, 0.0)]
    x = rnd(1000, 90)
    with pytest.raises(abi.TwgError):
        abi.fused_select(two_outputs, [x], 0)
    float_output = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_RELU, 0, 0, 0.0), (F.F_OUTPUT, 1, 0, 0.0)]
    with pytest.raises(abi.TwgError):
        abi.fused_select(float_output, [x], 0)
    pred = [(F.F_INPUT_F32, 0, 0, 0.0), (F.F_CONST_F32, 0, 0, 0.0), (F.F_GT, 0, 1, 0.0), (F.F_OUTPUT, 2, 0, 0.0)]
    with pytest.raises(abi.TwgError):
        abi.fused_select(pred, [x], 3)


def test_fused_rejects_malformed_programs(abi):
    F = abi
    with pytest.raises(abi.TwgError):
        abi.fused_compile([(F.F_INPUT_F32, 0, 0, 0.0), (F.F_AND, 0, 0, 0.0), (F.F_OUTPUT, 1, 0, 0.0)])
    with pytest.raises(abi.TwgError):
        abi.fused_compile([(F.F_INPUT_F32, 0, 0, 0.0), (F.F_RELU, 5, 0, 0.0), (F.F_OUTPUT, 1, 0, 0.0)])
    with pytest.raises(abi.TwgError):
        abi.fused_compile([(F.F_INPUT_F32, 0, 0, 0.0), (F.F_RELU, 0, 0, 0.0)])


# ------------------------------------------------------------------------------------------
# allocator, copies, events
# ------------------------------------------------------------------------------------------
def test_allocator_caches_splits_trims_and_reports(abi):
    import ctypes
    L = abi.lib()

    def stats():
        s = abi.MemStats()
        abi.check(L.twg_memory_stats(0, ctypes.byref(s)))
        return s

    abi.check(L.twg_empty_cache(0))
    s0 = stats()
    a = abi.DeviceBuffer(64 << 20)
    s1 = stats()
    assert s1.num_device_mallocs == s0.num_device_mallocs + 1
    assert s1.allocated_bytes - s0.allocated_bytes == 64 << 20
    ptr = a.ptr
    a.free()
    a2 = abi.DeviceBuffer(64 << 20)          # served from the cache, same block
    s2 = stats()
    assert a2.ptr == ptr and s2.num_device_mallocs == s1.num_device_mallocs
    assert s2.num_cache_hits == s1.num_cache_hits + 1
    abi.check(L.twg_trim(a2.ptr, 8 << 20))   # give 56 MiB back
    s3 = stats()
    assert s2.allocated_bytes - s3.allocated_bytes == 56 << 20
    tail = abi.DeviceBuffer(40 << 20)        # fits in the returned tail: no new cudaMalloc
    assert stats().num_device_mallocs == s2.num_device_mallocs
    assert tail.ptr == ptr + (8 << 20)
    small = [abi.DeviceBuffer(1000) for _ in range(100)]  # carved from one 2 MiB segment
    assert stats().num_device_mallocs <= s2.num_device_mallocs + 1
    assert all(sm.ptr % 512 == 0 for sm in small)
    for sm in small:
        sm.free()
    tail.free(); a2.free()
    abi.check(L.twg_empty_cache(0))
    s4 = stats()
    assert s4.reserved_bytes <= s0.reserved_bytes
    assert abi.DeviceBuffer(0).ptr == 0
    assert L.twg_free(12345) == abi.TWG_ERR_INVALID


def test_guard_words_report_a_write_past_the_end(abi):
    """With guard words on, bytes behind a block's requested size carry a pattern; a write that runs
    a few bytes over (still inside the block: nothing faults) is found by the check."""
    import ctypes
    L = abi.lib()
    bad, first = ctypes.c_int64(), ctypes.c_void_p()
    abi.check(L.twg_set_guard_words(1))
    try:
        a = abi.DeviceBuffer(1000)
        b = abi.DeviceBuffer(3 << 20)
        abi.check(L.twg_memset(a.ptr, 0, 1000, None))                 # exactly what was asked for
        x = rnd(1 << 18, 95)
        assert_bit_equal(abi.unary("relu", x), oracle.unary("relu", x), "relu with guarded blocks")
        abi.check(L.twg_check_guard_words(0, ctypes.byref(bad), ctypes.byref(first)))
        assert bad.value == 0 and first.value is None
        abi.check(L.twg_memset(b.ptr + (3 << 20) - 8, 0, 12, None))   # four bytes too many
        abi.check(L.twg_check_guard_words(0, ctypes.byref(bad), ctypes.byref(first)))
        assert bad.value == 1 and first.value == b.ptr
        abi.check(L.twg_trim(a.ptr, 100))                             # guarded blocks keep their tail
        size = ctypes.c_size_t()
        abi.check(L.twg_block_size(a.ptr, ctypes.byref(size), None))
        assert size.value >= 1000 + 512
        del a, b
    finally:
        abi.check(L.twg_set_guard_words(0))
    c = abi.DeviceBuffer(1000)                                         # blocks made afterwards are plain again
    abi.check(L.twg_check_guard_words(0, ctypes.byref(bad), ctypes.byref(first)))
    assert bad.value == 0


def test_allocator_budget_injects_out_of_memory(abi):
    L = abi.lib()
    import ctypes
    abi.check(L.twg_empty_cache(0))
    s = abi.MemStats()
    abi.check(L.twg_memory_stats(0, ctypes.byref(s)))
    abi.check(L.twg_set_memory_budget(0, s.reserved_bytes + (32 << 20)))
    try:
        with pytest.raises(abi.TwgError) as e:
            abi.DeviceBuffer(256 << 20)
        assert e.value.code == abi.TWG_ERR_OOM
        ok = abi.DeviceBuffer(4 << 20)       # still serviceable below the cap
        ok.free()
    finally:
        abi.check(L.twg_set_memory_budget(0, 0))
    abi.DeviceBuffer(256 << 20).free()


def test_blocks_used_on_a_second_stream_wait_for_it(abi):
    import ctypes
    L = abi.lib()
    s2 = ctypes.c_void_p()
    abi.check(L.twg_get_stream(0, 2, ctypes.byref(s2)))
    buf = abi.DeviceBuffer(48 << 20)
    ptr = buf.ptr
    abi.check(L.twg_record_stream(buf.ptr, s2))
    abi.check(L.twg_memset(buf.ptr, 1, 48 << 20, s2))
    buf.free()                                # deferred behind an event on the second stream
    abi.check(L.twg_stream_sync(s2))
    again = abi.DeviceBuffer(48 << 20)        # after the event completed the block is reusable
    assert again.ptr == ptr
    again.free()


@pytest.mark.parametrize("nbytes", [1, 4097, (16 << 20) - 1, (16 << 20) + 5, (40 << 20) + 3])
def test_pageable_and_pinned_round_trips(abi, nbytes):
    import ctypes
    L = abi.lib()
    host = np.random.default_rng(nbytes % 1000).integers(0, 256, nbytes, dtype=np.uint8)
    dev = abi.DeviceBuffer(nbytes)
    dev.upload(host)
    assert np.array_equal(dev.download(np.uint8, nbytes), host)
    pinned = ctypes.c_void_p()
    abi.check(L.twg_host_alloc_pinned(ctypes.byref(pinned), nbytes))
    try:
        view = np.ctypeslib.as_array(ctypes.cast(pinned, ctypes.POINTER(ctypes.c_uint8)), shape=(nbytes,))
        view[:] = host[::-1]
        abi.check(L.twg_memcpy_h2d(dev.ptr, pinned, nbytes, None))
        abi.check(L.twg_stream_sync(None))
        view[:] = 0
        abi.check(L.twg_memcpy_d2h(pinned, dev.ptr, nbytes, None, 1))
        assert np.array_equal(view, host[::-1])
    finally:
        abi.check(L.twg_host_free_pinned(pinned))


def test_events_and_launch_accounting(abi):
    import ctypes
    L = abi.lib()
    e0, e1 = ctypes.c_void_p(), ctypes.c_void_p()
    abi.check(L.twg_event_create(ctypes.byref(e0)))
    abi.check(L.twg_event_create(ctypes.byref(e1)))
    x = rnd(1 << 20, 90)
    L.twg_reset_launch_count()
    abi.check(L.twg_event_record(e0, None))
    abi.unary("relu", x)
    abi.check(L.twg_event_record(e1, None))
    abi.check(L.twg_event_sync(e1))
    ms = ctypes.c_float()
    abi.check(L.twg_event_elapsed_ms(e0, e1, ctypes.byref(ms)))
    assert ms.value > 0
    assert L.twg_launch_count() == 1
    done = ctypes.c_int()
    abi.check(L.twg_event_query(e1, ctypes.byref(done)))
    assert done.value == 1
    abi.check(L.twg_event_destroy(e0)); abi.check(L.twg_event_destroy(e1))
