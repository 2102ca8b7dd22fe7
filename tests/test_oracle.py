"""Pin the CPU oracle (oracle/twg_oracle.c) before anything is compared against it.

Two anchors: the known-answer vectors of the reference's own tests, and outputs of the PyTorch
CPU ATen kernels (the reference's implementation of its fallback ops and the expected values of
all its tests) committed under tests/golden/.  Bit-exact for add / mul / relu / abs / comparisons /
bitwise_and / masked_select / copies; silu within max(2 ulp, 1e-6 rel); erf-GELU additionally
within 2e-6 absolute.
"""
from __future__ import annotations

import numpy as np
import pytest

from oracle import oracle
from util import CVT_NAMES, assert_bit_equal, assert_close_ulp, cvt_case


def b(a):  # golden bool arrays are stored as uint8
    return a.view(np.bool_)


def test_kat_add_reference_test_vector(golden):
    # tests/ops/test_add.py:6-10 (allclose against hand-written values)
    out = oracle.binary("add", golden["kat_add_a"], golden["kat_add_b"])
    assert np.allclose(out, golden["kat_add_expected_handwritten"])
    assert_bit_equal(out, golden["kat_add_out"], "add KAT")


def test_kat_fused_add_relu_reference_test_vector(golden):
    # tests/test_dev.py:8-9,18
    out = oracle.binary("fused_add_relu", golden["kat_add_a"], golden["kat_add_b"])
    assert np.allclose(out, golden["kat_fused_add_relu_expected_handwritten"])
    assert_bit_equal(out, golden["kat_fused_add_relu_out"], "fused_add_relu KAT")


@pytest.mark.parametrize("i", range(4))
def test_kat_activations_reference_test_vectors(golden, i):
    # tests/ops/test_gelu.py:7,18,29,43 and tests/ops/test_silu.py:6,17,28,42
    x = golden[f"kat_act{i}_x"]
    # the reference's tolerances
    assert np.allclose(oracle.unary("gelu_tanh_shader", x), golden[f"kat_act{i}_gelu"], atol=1e-3)
    assert np.allclose(oracle.unary("silu_shader", x), golden[f"kat_act{i}_silu"], atol=1e-6)
    # this build's tolerances
    assert_close_ulp(oracle.unary("gelu_erf", x), golden[f"kat_act{i}_gelu"], abs_floor=2e-6, what="gelu erf KAT")
    assert_close_ulp(oracle.unary("gelu_tanh", x), golden[f"kat_act{i}_gelu_tanh"], abs_floor=2e-6, what="gelu tanh KAT")
    assert_close_ulp(oracle.unary("silu", x), golden[f"kat_act{i}_silu"], what="silu KAT")
    assert_bit_equal(oracle.unary("relu", x), golden[f"kat_act{i}_relu"], "relu KAT")


def test_edge_values_bit_exact(golden):
    x, y = golden["edge_x"], golden["edge_y"]
    assert_bit_equal(oracle.binary("add", x, y), golden["edge_add"], "edge add")
    assert_bit_equal(oracle.binary("add", x, y, alpha=2.5), golden["edge_add_alpha"], "edge add alpha")
    assert_bit_equal(oracle.unary("relu", x), golden["edge_relu"], "edge relu")
    assert_bit_equal(oracle.compare("eq", x, y), b(golden["edge_eq"]), "edge eq")
    assert_bit_equal(oracle.compare("eq", x, x.copy()), b(golden["edge_eq_self"]), "edge eq self")
    assert_bit_equal(oracle.compare("ne", x, 0.0), b(golden["edge_ne0"]), "edge ne 0")
    assert_bit_equal(oracle.compare("eq", x, 0.0), b(golden["edge_eq0"]), "edge eq 0")


def test_edge_values_silu(golden):
    x = golden["edge_x"]
    keep = np.abs(x) <= 1e4  # the CPU kernel's two code paths disagree on huge inputs
    keep |= np.isnan(x)
    assert_close_ulp(oracle.unary("silu", x[keep]), golden["edge_silu"][keep], what="edge silu")


def test_random_bit_exact_ops(golden):
    x, y = golden["rnd_x"], golden["rnd_y"]
    assert_bit_equal(oracle.binary("add", x, y), golden["rnd_add"], "add")
    assert_bit_equal(oracle.binary("add", x, y, alpha=-0.75), golden["rnd_add_alpha"], "add alpha")
    assert_bit_equal(oracle.binary("mul", x, y), golden["rnd_mul"], "mul")
    assert_bit_equal(oracle.unary("relu", x), golden["rnd_relu"], "relu")
    assert_bit_equal(oracle.unary("abs", x), golden["rnd_abs"], "abs")
    p, q = golden["rnd_p"], golden["rnd_q"]
    m1 = oracle.compare("eq", p, q)
    m2 = oracle.compare("ne", p, 0.0)
    assert_bit_equal(m1, b(golden["rnd_eq"]), "eq")
    assert_bit_equal(m2, b(golden["rnd_ne0"]), "ne")
    assert_bit_equal(oracle.bitwise_and(m1, m2), b(golden["rnd_and"]), "and")
    assert_bit_equal(oracle.bitwise_and(golden["rnd_i1"], golden["rnd_i2"]), golden["rnd_and_i32"], "and i32")


def test_random_activations(golden):
    x = golden["rnd_x"]
    assert_close_ulp(oracle.unary("silu", x), golden["rnd_silu"], what="silu")
    assert_close_ulp(oracle.unary("gelu_erf", x), golden["rnd_gelu"], abs_floor=2e-6, what="gelu erf")
    assert_close_ulp(oracle.unary("gelu_tanh", x), golden["rnd_gelu_tanh"], abs_floor=2e-6, what="gelu tanh")


def test_strided_and_broadcast_layouts(golden):
    s = golden["lay_s"]
    assert_bit_equal(oracle.unary("relu", s.T), golden["lay_relu_t"], "relu transposed")
    assert_close_ulp(oracle.unary("silu", s[:, ::2]), golden["lay_silu_slice"], what="silu slice")
    row, col = golden["lay_row"], golden["lay_col"]
    assert_bit_equal(oracle.binary("add", s, row), golden["lay_add_row"], "add row broadcast")
    assert_bit_equal(oracle.binary("add", s, col, alpha=3.0), golden["lay_add_col"], "add col broadcast")
    assert_bit_equal(oracle.binary("add", row, col), golden["lay_add_outer"], "add outer broadcast")
    assert_bit_equal(oracle.compare("eq", s.T, np.ascontiguousarray(s.T)), b(golden["lay_eq_t"]), "eq transposed")
    assert_bit_equal(oracle.copy(s.T), np.ascontiguousarray(s.T), "strided copy")


@pytest.mark.parametrize("tag", ["001", "05", "099"])
def test_masked_select_full_masks(golden, tag):
    src, mask = golden["ms_src"], b(golden[f"ms_mask_{tag}"])
    assert_bit_equal(oracle.masked_select(src, mask), golden[f"ms_out_{tag}"], "masked_select")
    assert_bit_equal(oracle.masked_select(src.T, mask.T), golden[f"ms_out_t_{tag}"], "masked_select transposed")


def test_masked_select_broadcast_and_edges(golden):
    src = golden["ms_src"]
    assert_bit_equal(oracle.masked_select(src, b(golden["ms_mask_row"])), golden["ms_out_row"], "row mask")
    assert_bit_equal(oracle.masked_select(src, b(golden["ms_mask_col"])), golden["ms_out_col"], "col mask")
    assert_bit_equal(oracle.masked_select(src[:, :1], b(golden["ms_mask_col"])), golden["ms_out_bsrc"], "bcast self")
    assert oracle.masked_select(src, np.zeros(src.shape, np.bool_)).size == 0
    assert_bit_equal(oracle.masked_select(src, np.ones(src.shape, np.bool_)), golden["ms_out_all"], "all")
    assert oracle.masked_select(np.empty((0,), np.float32), np.empty((0,), np.bool_)).size == 0
    with pytest.raises(RuntimeError):
        oracle.masked_select(src, np.ones(src.shape, np.uint8))


def test_chain(golden):
    a, bb, c = golden["chain_a"], golden["chain_b"], golden["chain_c"]
    y, m = oracle.chain_mask(a, bb, c, want_y=True)
    # silu's <= 2 ulp error is amplified where adding c cancels, so y gets an absolute floor
    assert_close_ulp(y, golden["chain_y"], abs_floor=1e-6, what="chain y")
    # on this fixture no pre-relu value is close enough to zero for the mask to flip
    assert_bit_equal(m, b(golden["chain_m"]), "chain mask")
    assert_bit_equal(oracle.masked_select(a, m), golden["chain_sel"], "chain select")


def test_sub_div_where_masked_fill_against_aten(golden):
    """Neighbouring ops of the reference's list (README.md:106-166); ATen CPU is the pin."""
    x, y, e, er = golden["rnd_x"], golden["rnd_y"], golden["edge_x"], golden["edge_y"]
    assert_bit_equal(oracle.sub(x, y), golden["rnd_sub"], "sub")
    assert_bit_equal(oracle.sub(x, y, 1.75), golden["rnd_sub_alpha"], "sub alpha")
    assert_bit_equal(oracle.binary("div", x, y), golden["rnd_div"], "div")
    assert_bit_equal(oracle.binary("div", e, er), golden["edge_div"], "div edge", any_nan=True)
    assert_bit_equal(oracle.sub(e, er), golden["edge_sub"], "sub edge", any_nan=True)
    m1, m2 = golden["rnd_eq"].view(np.bool_), golden["rnd_ne0"].view(np.bool_)
    assert_bit_equal(oracle.where(m2, x, y), golden["rnd_where"], "where")
    assert_bit_equal(oracle.masked_fill(x, m1, -3.5), golden["rnd_masked_fill"], "masked_fill")
    s, col, wc = golden["lay_s"], golden["lay_col"], golden["lay_where_cond"].view(np.bool_)
    assert_bit_equal(oracle.where(wc, s, col), golden["lay_where"], "where broadcast")
    assert_bit_equal(oracle.masked_fill(s.T, wc.T, 2.0), golden["lay_masked_fill_t"], "masked_fill transposed")


@pytest.mark.parametrize("src", CVT_NAMES)
def test_conversions_against_aten(golden, src):
    for dst in CVT_NAMES:
        x, want = cvt_case(golden, src, dst)
        got = oracle.convert(x, src, dst)
        assert_bit_equal(got, want, f"{src} -> {dst}")


def test_more_than_eight_dims_rejected():
    x = np.zeros((1,) * 9, np.float32)
    with pytest.raises(RuntimeError):
        oracle.unary("relu", x)


def test_parallel_masked_select_matches_serial():
    rng = np.random.default_rng(5)
    x = rng.standard_normal(300_000).astype(np.float32)
    m = rng.random(300_000) < 0.37
    assert_bit_equal(oracle.masked_select(x, m), x[m], "parallel masked_select")
