"""Generate tests/golden/aten_golden.npz: inputs and PyTorch CPU ATen outputs for the op path.

PyTorch CPU ATen is the reference's own implementation of eq / ne / bitwise_and / masked_select
(it runs them through at::native::cpu_fallback, csrc/bindings.cpp:27-42) and the oracle every
reference test asserts against for add / gelu / silu.  The known-answer inputs of those tests
(tests/ops/test_add.py:6-9, test_gelu.py:7,18,29,43, test_silu.py:6,17,28,42, tests/test_dev.py:8-9,18)
are included verbatim as `kat_*` entries with the expected values the tests compute.

Run once in an environment with torch installed:  python tests/golden/make_golden.py
The output is committed; tests only read it.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

OUT = Path(__file__).resolve().parent / "aten_golden.npz"


def edge_values() -> torch.Tensor:
    f = np.array(
        [0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 2.0, -2.0, 7.999, -7.999, 20.0, -20.0, 88.0, -88.0, 100.0, -100.0,
         1e-45, -1e-45, 1e-40, -1e-40, 1.17549435e-38, -1.17549435e-38, 3.4028235e38, -3.4028235e38,
         np.inf, -np.inf, np.nan, 1e-8, -1e-8, 3.0, -3.0, 0.1], dtype=np.float32)
    return torch.from_numpy(f)


def main() -> None:
    torch.manual_seed(0)
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(1234)
    d: dict[str, np.ndarray] = {}

    def put(name: str, t: torch.Tensor) -> None:
        a = t.detach().contiguous().numpy()
        d[name] = a.view(np.uint8) if a.dtype == np.bool_ else a

    # ---- known-answer vectors from the reference's tests --------------------------------------
    a = torch.tensor([-1.5, 2.7, 1.0, 2.0]); b = torch.tensor([-1.0, 0.9, 1.1, -2.1])
    put("kat_add_a", a); put("kat_add_b", b)
    put("kat_add_expected_handwritten", torch.tensor([-2.5, 3.6, 2.1, -0.1]))
    put("kat_add_out", a + b)
    put("kat_fused_add_relu_expected_handwritten", torch.tensor([0, 3.6, 2.1, 0]))
    put("kat_fused_add_relu_out", torch.relu(a + b))
    for i, x in enumerate([torch.tensor([-1.0, 0.0, 1.0, 2.0]), torch.tensor([[0.5, -0.5], [1.5, -1.5]]),
                           torch.tensor([2.0]), torch.tensor([0.0])]):
        put(f"kat_act{i}_x", x)
        put(f"kat_act{i}_gelu", F.gelu(x))
        put(f"kat_act{i}_gelu_tanh", F.gelu(x, approximate="tanh"))
        put(f"kat_act{i}_silu", F.silu(x))
        put(f"kat_act{i}_relu", torch.relu(x))

    # ---- edge values ---------------------------------------------------------------------------
    e = edge_values()
    put("edge_x", e)
    er = e.flip(0).contiguous()
    put("edge_y", er)
    put("edge_add", torch.add(e, er))
    put("edge_add_alpha", torch.add(e, er, alpha=2.5))
    put("edge_relu", torch.relu(e))
    put("edge_silu", F.silu(e))
    put("edge_eq", torch.eq(e, er))
    put("edge_eq_self", torch.eq(e, e.clone()))
    put("edge_ne0", torch.ne(e, 0.0))
    put("edge_eq0", torch.eq(e, 0.0))

    # ---- seeded random cases -------------------------------------------------------------------
    n = 1031
    x = torch.rand(n, generator=g) * 16 - 8
    y = torch.randn(n, generator=g)
    put("rnd_x", x); put("rnd_y", y)
    put("rnd_add", x + y)
    put("rnd_add_alpha", torch.add(x, y, alpha=-0.75))
    put("rnd_mul", x * y)
    put("rnd_relu", torch.relu(x))
    put("rnd_abs", torch.abs(x))
    put("rnd_silu", F.silu(x))
    put("rnd_gelu", F.gelu(x))
    put("rnd_gelu_tanh", F.gelu(x, approximate="tanh"))
    p = torch.randint(-2, 3, (n,), generator=g).float()
    q = torch.randint(-2, 3, (n,), generator=g).float()
    put("rnd_p", p); put("rnd_q", q)
    m1 = torch.eq(p, q); m2 = torch.ne(p, 0.0)
    put("rnd_eq", m1); put("rnd_ne0", m2); put("rnd_and", torch.bitwise_and(m1, m2))
    i1 = torch.randint(-2**31, 2**31 - 1, (257,), generator=g, dtype=torch.int64).to(torch.int32)
    i2 = torch.randint(-2**31, 2**31 - 1, (257,), generator=g, dtype=torch.int64).to(torch.int32)
    put("rnd_i1", i1); put("rnd_i2", i2); put("rnd_and_i32", torch.bitwise_and(i1, i2))

    # strided / broadcast layouts
    s2 = torch.randn(37, 53, generator=g)
    put("lay_s", s2)
    put("lay_relu_t", torch.relu(s2.t()))                 # logical [53,37]
    put("lay_silu_slice", F.silu(s2[:, ::2]))             # stride-2 read
    row = torch.randn(37, 1, generator=g); col = torch.randn(1, 53, generator=g)
    put("lay_row", row); put("lay_col", col)
    put("lay_add_row", s2 + row); put("lay_add_col", torch.add(s2, col, alpha=3.0))
    put("lay_add_outer", row + col)
    put("lay_eq_t", torch.eq(s2.t(), s2.t().contiguous()))

    # masked_select
    src = torch.randn(61, 67, generator=g)
    put("ms_src", src)
    for pr in (0.01, 0.5, 0.99):
        mk = torch.rand(61, 67, generator=g) < pr
        tag = str(pr).replace(".", "")
        put(f"ms_mask_{tag}", mk)
        put(f"ms_out_{tag}", torch.masked_select(src, mk))
        put(f"ms_out_t_{tag}", torch.masked_select(src.t(), mk.t()))   # non-contiguous self and mask
    mrow = torch.rand(61, 1, generator=g) < 0.5
    mcol = torch.rand(1, 67, generator=g) < 0.5
    put("ms_mask_row", mrow); put("ms_out_row", torch.masked_select(src, mrow))
    put("ms_mask_col", mcol); put("ms_out_col", torch.masked_select(src, mcol))
    put("ms_out_bsrc", torch.masked_select(src[:, :1], mcol))          # self broadcast against the mask
    put("ms_out_none", torch.masked_select(src, torch.zeros(61, 67, dtype=torch.bool)))
    put("ms_out_all", torch.masked_select(src, torch.ones(61, 67, dtype=torch.bool)))

    # the torch.compile chain of the benchmark
    ca = torch.randn(4099, generator=g); cb = torch.randn(4099, generator=g); cc = torch.randn(4099, generator=g)
    ca[::17] = 0.0
    cy = torch.relu(F.silu(ca + cb) + cc)
    cm = torch.bitwise_and(torch.eq(cy, 0), torch.ne(ca, 0))
    put("chain_a", ca); put("chain_b", cb); put("chain_c", cc)
    put("chain_y", cy); put("chain_m", cm); put("chain_sel", torch.masked_select(ca, cm))

    # ---- neighbouring ops of the reference's list: sub, div, where, masked_fill -----------------
    # (appended after everything else so that the generator draws above stay what they were)
    put("rnd_sub", x - y)
    put("rnd_sub_alpha", torch.sub(x, y, alpha=1.75))
    put("rnd_div", x / y)
    put("edge_div", e / er)
    put("edge_sub", e - er)
    put("rnd_where", torch.where(m2, x, y))
    put("rnd_masked_fill", torch.masked_fill(x, m1, -3.5))
    wc = torch.rand(37, 1, generator=g) < 0.5
    put("lay_where_cond", wc)
    put("lay_where", torch.where(wc, s2, col))             # cond [37,1], a [37,53], b [1,53]
    put("lay_masked_fill_t", torch.masked_fill(s2.t(), wc.t(), 2.0))

    # ---- element-type conversions (copy_ between dtypes): every pair, in-range values ------------
    cv = torch.cat([torch.rand(200, generator=g) * 200 - 100, torch.tensor([0.0, -0.0, 0.5, -0.5, 1.5, 2.5, -2.5, 127.0,
                                                                          -128.0, 1e-3, 65504.0 / 1024])])
    names = {torch.uint8: "uint8", torch.int8: "int8", torch.int16: "int16", torch.int32: "int32", torch.int64: "int64",
             torch.float16: "float16", torch.bfloat16: "bf16", torch.float32: "float32", torch.float64: "float64",
             torch.bool: "bool"}
    def bits(t: torch.Tensor) -> torch.Tensor:
        return t.view(torch.int16) if t.dtype == torch.bfloat16 else t
    for sdt, sname in names.items():
        if sdt == torch.uint8:
            base = cv.abs().to(sdt)          # a negative float -> uint8 cast is undefined in C
        elif sdt == torch.bool:
            base = cv > 0
        else:
            base = cv.to(sdt)
        put(f"cvt_src_{sname}", bits(base))
        for ddt, dname in names.items():
            if ddt == torch.uint8 and sdt not in (torch.uint8, torch.bool):
                src_t = base.abs() if sdt != torch.uint8 else base
                put(f"cvt_src_{sname}_for_uint8", bits(src_t))
                put(f"cvt_{sname}_to_{dname}", bits(src_t.to(ddt)))
            else:
                put(f"cvt_{sname}_to_{dname}", bits(base.to(ddt)))

    np.savez_compressed(OUT, **d)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(d)} arrays, torch {torch.__version__})")


if __name__ == "__main__":
    main()
