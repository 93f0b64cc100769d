"""Pins the numpy oracle to outputs of the reference itself (tests/golden/*.npz)."""
import numpy as np
import pytest

from oracle import oracle_np as O


def same(a, b):
    a = np.asarray(a); b = np.asarray(b)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.dtype.kind == "f":
        assert np.array_equal(a, b, equal_nan=True)
    else:
        assert np.array_equal(a, b)


def test_quantize_dequantize_4bit_cases(golden):
    g = golden("4bit")
    for name, qt, dt, n, k, bs, dq in g["cases"]:
        n, k, bs, dq = int(n), int(k), int(bs), int(dq)
        w = g[name + "_w"]
        packed, absmax, absmax2 = O.quantize_4bit(w, bs, qt, bool(dq))
        same(packed, g[name + "_packed"])
        same(absmax, g[name + "_absmax"])
        if dq:
            same(absmax2, g[name + "_absmax2"])
        deq = O.dequantize_4bit(packed, absmax, (n, k), bs, qt, dt, absmax2)
        same(deq, g[name + "_deq"])


def test_known_answers_4bit(golden):
    g = golden("4bit")
    p, _, _ = O.quantize_4bit(g["kat_fp4_in"], 64, "fp4")
    same(p, g["kat_fp4_packed"])
    codes = [int(p[0]) & 15, int(p[0]) >> 4, int(p[1]) & 15, int(p[1]) >> 4, int(p[2]) & 15, int(p[2]) >> 4]
    assert codes == [7, 0, 0, 6, 14, 9]          # ties go to the first (lower) index
    p, _, _ = O.quantize_4bit(g["kat_nf4_in"], 64, "nf4")
    same(p, g["kat_nf4_packed"])
    assert (int(p[0]) & 15, int(p[0]) >> 4, int(p[1]) & 15) == (15, 0, 7)


@pytest.mark.parametrize("nm", ["zeros", "one", "tiny", "max"])
@pytest.mark.parametrize("qt", ["nf4", "fp4"])
def test_special_inputs(golden, nm, qt):
    g = golden("4bit")
    x = g[f"sp_{nm}_{qt}_in"]
    p, a, _ = O.quantize_4bit(x, 64, qt)
    same(p, g[f"sp_{nm}_{qt}_packed"]); same(a, g[f"sp_{nm}_{qt}_absmax"])
    dt = "float32" if x.dtype == np.float32 else "float16"
    d = O.dequantize_4bit(p, a, x.shape, 64, qt, dt)
    same(d, g[f"sp_{nm}_{qt}_deq"])
    assert np.isfinite(d.astype(np.float32)).all()


def test_flat_path(golden):
    g = golden("4bit")
    v = g["flat_in"]
    p, a, _ = O.quantize_4bit(v.reshape(1, -1), 64, "nf4")
    same(p, g["flat_packed"]); same(a, g["flat_absmax"])
    same(O.dequantize_4bit(p, a, (1, v.size), 64, "nf4", "float16").reshape(-1), g["flat_deq"])
    v3 = g["flat3_in"]
    p, a, _ = O.quantize_4bit(v3.reshape(1, -1), 32, "fp4")
    same(p, g["flat3_packed"]); same(a, g["flat3_absmax"])
    same(O.dequantize_4bit(p, a, (1, v3.size), 32, "fp4", "float16").reshape(v3.shape), g["flat3_deq"])


def test_blockwise(golden):
    g = golden("int8")
    for bs in (256, 4096, 64):
        q, am = O.quantize_blockwise(g[f"bw{bs}_in"], bs)
        same(q, g[f"bw{bs}_q"]); same(am, g[f"bw{bs}_absmax"])
        same(O.dequantize_blockwise(q, am, bs, "float32"), g[f"bw{bs}_deq"])


def test_rowwise_colrow_double_quant(golden):
    g = golden("int8")
    q, s = O.quantize_rowwise(g["kat_row_in"])
    same(q, g["kat_row_q"]); same(s, g["kat_row_s"])
    assert q.tolist() == [[127, 0, 2, 2, 0, -2]]                 # round half to even
    for dt in ("float16", "bfloat16", "float32"):
        q, s = O.quantize_rowwise(g[f"row_{dt}_in"])
        same(q, g[f"row_{dt}_q"]); same(s, g[f"row_{dt}_s"])
        for od in ("float16", "bfloat16", "float32"):
            same(O.dequantize_rowwise(q, s, od), g[f"row_{dt}_deq_{od}"])
    oc, orow, cs, rs = O.double_quant(g["dq_in"])
    same(oc, g["dq_col"]); same(orow, g["dq_row"]); same(cs, g["dq_cs"]); same(rs, g["dq_rs"])
    q, r, c = O.quantize_colrow(g["dq_in"])
    same(q, g["cr_q"]); same(r, g["cr_r"]); same(c, g["cr_c"])
    same(O.dequantize_colrow(q, r, c, "float16"), g["cr_deq"])
    same(O.dequantize_colrow(q, r, c, "bfloat16"), g["cr_deq_bf16"])


def test_fp8(golden):
    g = golden("fp8")
    c, s = O.quantize_fp8_e4m3(g["kat_in"])
    same(c, g["kat_codes"]); same(s, g["kat_scales"])
    assert [f"{v:02x}" for v in c[0]] == "77 77 77 77 77 3f 38 30 08 00 00 f7".split()
    same(O.dequantize_fp8_e4m3(np.arange(256, dtype=np.uint8).reshape(1, 256), np.ones(1, np.float32), "float32"),
         g["decode_all"])
    same(O.dequantize_fp8_e4m3(np.arange(256, dtype=np.uint8).reshape(1, 256), np.array([0.0371], np.float32),
                               "float16"), g["decode_all_f16"])
    c, s = O.quantize_fp8_e4m3(g["edge_in"])
    assert s[0] == 1.0
    same(c, g["edge_codes"])
    for dt in ("float16", "bfloat16", "float32"):
        c, s = O.quantize_fp8_e4m3(g[f"rnd_{dt}_in"])
        same(c, g[f"rnd_{dt}_codes"]); same(s, g[f"rnd_{dt}_scales"])
        same(O.dequantize_fp8_e4m3(c, s, dt if dt != "float32" else "float16"), g[f"rnd_{dt}_deq"])


def rel_err(y, ref):
    y = np.asarray(y, np.float32); ref = np.asarray(ref, np.float32)
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


def test_matmuls_within_tolerance(golden):
    """Oracle matmuls vs the reference's torch CPU GEMM: only accumulation order differs."""
    g = golden("matmul")
    for i in range(int(g["mm4_n"])):
        M, N, K, qt, dq, bias, dt = g[f"mm4_{i}_meta"]
        N, K = int(N), int(K)
        p, a, a2 = O.quantize_4bit(g[f"mm4_{i}_w"], 64, qt, bool(int(dq)))
        b = g[f"mm4_{i}_b"] if int(bias) else None
        y = O.matmul_4bit(g[f"mm4_{i}_x"], p, a, (N, K), 64, qt, dt, a2, b, dt)
        assert rel_err(y, g[f"mm4_{i}_y"]) <= 1e-2
    y = O.matmul_int8(g["i8_Aq"], g["i8_Bq"], g["i8_As"], g["i8_Bs"])
    assert rel_err(y, g["i8_y"]) <= 1e-2
    q, r, c = O.quantize_colrow(g["cr_W"])
    assert rel_err(O.matmul_colrow(g["i8_A"], q, r, c, g["cr_b"]), g["cr_y"]) <= 1e-2
    c8, s8 = O.quantize_fp8_e4m3(g["cr_W"])
    assert rel_err(O.matmul_fp8_e4m3(g["i8_A"], c8, s8, g["cr_b"]), g["f8_y"]) <= 1e-2


def test_half_way_cases_int8(golden):
    """x = s*(j+0.5)/127: the rounding of 127.0/s (reciprocal then multiply) decides the code."""
    g = golden("int8")
    t = g["ties_in"]
    q, s = O.quantize_rowwise(t)
    same(q, g["ties_q"]); same(s, g["ties_s"])
    qb, am = O.quantize_blockwise(t.reshape(-1), 128)
    same(qb, g["ties_bw_q"]); same(am, g["ties_bw_absmax"])
    same(O.dequantize_blockwise(qb, am, 128, "float32"), g["ties_bw_deq"])
    qc, r, c = O.quantize_colrow(t)
    same(qc, g["ties_cr_q"])
    # the reference host's sqrt (torch + MKL vector maths) is one ulp low on ~0.6 % of inputs;
    # the oracle uses the IEEE sqrt, so the fp32 dequantised value may differ in its last bits
    d = O.dequantize_colrow(qc, r, c, "float32"); ref = g["ties_cr_deq"]
    assert np.allclose(d, ref, rtol=4e-7, atol=0)
    assert (d != ref).mean() < 0.02
    oc, orow, _, _ = O.double_quant(t)
    same(oc, g["ties_dq_col"]); same(orow, g["ties_dq_row"])
