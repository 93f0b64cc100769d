"""GPU parity, 8-bit family: blockwise / row-wise / col+row int8, LLM.int8 statistics and
FP8 E4M3 — against stored outputs of the reference and against the oracle.  Bit-exact."""
import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from oracle import oracle_np as O
from gpu_util import to_cuda, to_np

pytestmark = pytest.mark.gpu


def test_blockwise_golden_and_ties(golden):
    g = golden("int8")
    for bs in (256, 4096, 64):
        q, st = bnb.quantize_blockwise(to_cuda(g[f"bw{bs}_in"], "float32"), blocksize=bs)
        assert q.dtype == torch.int8 and st.quant_type == "int8" and st.blocksize == bs
        assert np.array_equal(to_np(q), g[f"bw{bs}_q"]) and np.array_equal(to_np(st.absmax), g[f"bw{bs}_absmax"])
        assert np.array_equal(to_np(bnb.dequantize_blockwise(q, st)), g[f"bw{bs}_deq"])
    t = to_cuda(g["ties_in"], "float32")
    q, st = bnb.quantize_blockwise(t.flatten(), blocksize=128)
    assert np.array_equal(to_np(q), g["ties_bw_q"]) and np.array_equal(to_np(st.absmax), g["ties_bw_absmax"])
    assert np.array_equal(to_np(bnb.dequantize_blockwise(q, st)), g["ties_bw_deq"])
    # nested (absmax of absmax)
    q, st = bnb.quantize_blockwise(t.flatten(), blocksize=64, nested=True)
    assert st.state2 is not None and st.absmax.dtype == torch.int8
    eq, ea = O.quantize_blockwise(g["ties_in"].reshape(-1), 64)
    eq2, ea2 = O.quantize_blockwise(ea, 256)
    assert np.array_equal(to_np(q), eq) and np.array_equal(to_np(st.absmax), eq2)
    exp = O.dequantize_blockwise(eq, O.dequantize_blockwise(eq2, ea2, 256, "float32"), 64, "float32")
    assert np.array_equal(to_np(bnb.dequantize_blockwise(q, st)), exp)


@pytest.mark.parametrize("n", [256 * 5 + 37, 8, 256 * 1000, 255])
def test_blockwise_256_fp32_ragged_and_ties_match_oracle(n):
    """Block size 256 on fp32 input takes a warp-per-block kernel: whole blocks, a ragged last block, rounding ties
    (values that are exact multiples of absmax / 254) and an all-zero block, byte for byte against the oracle."""
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 0.05).astype(np.float32)
    x[: min(n, 16)] = 0.0
    if n > 300:
        x[256:300] = np.float32(0.5) * np.arange(44, dtype=np.float32) / np.float32(127.0)   # .5 ties after scaling by 127 / 0.5...
        x[300] = np.float32(0.5 * 43 / 127.0)
    q, st = bnb.quantize_blockwise(torch.from_numpy(x).cuda(), blocksize=256)
    eq, ea = O.quantize_blockwise(x, 256)
    assert np.array_equal(to_np(q), eq) and np.array_equal(to_np(st.absmax), ea)
    # a caller-given absmax takes the same kernel
    q2, _ = bnb.quantize_blockwise(torch.from_numpy(x).cuda(), absmax=st.absmax.clone(), blocksize=256)
    assert np.array_equal(to_np(q2), eq)


def test_rowwise_golden_and_oracle(golden):
    g = golden("int8")
    q, s = bnb.quantize_rowwise(to_cuda(g["kat_row_in"], "float32"))
    assert to_np(q).tolist() == [[127, 0, 2, 2, 0, -2]]
    for dt in ("float16", "bfloat16", "float32"):
        q, s = bnb.quantize_rowwise(to_cuda(g[f"row_{dt}_in"], dt))
        assert np.array_equal(to_np(q), g[f"row_{dt}_q"]) and np.array_equal(to_np(s), g[f"row_{dt}_s"])
        for od in ("float16", "bfloat16", "float32"):
            d = bnb.dequantize_rowwise(q, s, dtype=getattr(torch, od))
            assert np.array_equal(to_np(d), g[f"row_{dt}_deq_{od}"])
    q, s = bnb.quantize_rowwise(to_cuda(g["ties_in"], "float32"))
    assert np.array_equal(to_np(q), g["ties_q"]) and np.array_equal(to_np(s), g["ties_s"])
    # 3-D input keeps its shape; rows are the last dimension
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 5, 96)).astype(np.float32)
    q, s = bnb.quantize_rowwise(torch.from_numpy(x).cuda())
    eq, es = O.quantize_rowwise(x)
    assert tuple(q.shape) == (3, 5, 96) and np.array_equal(to_np(q), eq) and np.array_equal(to_np(s), es)


def test_double_quant_and_colrow(golden):
    g = golden("int8")
    x = to_cuda(g["dq_in"], "float16")
    oc, orow, cs, rs, outl = bnb.double_quant(x)
    assert outl is None
    assert np.array_equal(to_np(oc), g["dq_col"]) and np.array_equal(to_np(orow), g["dq_row"])
    assert np.array_equal(to_np(cs), g["dq_cs"]) and np.array_equal(to_np(rs), g["dq_rs"])
    q, r, c = bnb.quantize_colrow(x)
    assert np.array_equal(to_np(q), g["cr_q"]) and np.array_equal(to_np(r), g["cr_r"]) and np.array_equal(to_np(c), g["cr_c"])
    assert np.array_equal(to_np(bnb.dequantize_colrow(q, r, c, torch.float16)), g["cr_deq"])
    assert np.array_equal(to_np(bnb.dequantize_colrow(q, r, c, torch.bfloat16)), g["cr_deq_bf16"])
    t = to_cuda(g["ties_in"], "float32")
    oc, orow, _, _, _ = bnb.double_quant(t)
    assert np.array_equal(to_np(oc), g["ties_dq_col"]) and np.array_equal(to_np(orow), g["ties_dq_row"])
    q, r, c = bnb.quantize_colrow(t)
    assert np.array_equal(to_np(q), g["ties_cr_q"])
    # against the oracle (IEEE sqrt) the fp32 dequantised values are identical
    assert np.array_equal(to_np(bnb.dequantize_colrow(q, r, c, torch.float32)),
                          O.dequantize_colrow(g["ties_cr_q"], to_np(r), to_np(c), "float32"))
    with pytest.raises(ValueError, match="Input must be 2D"):
        bnb.double_quant(torch.zeros(4, device="cuda"))
    with pytest.raises(ValueError, match="Input must be 2D"):
        bnb.quantize_colrow(torch.zeros(4, device="cuda"))


def test_int8_family_random_vs_oracle():
    rng = np.random.default_rng(17)
    x = (rng.standard_normal((300, 1030)) * 0.5).astype(np.float32)
    x[:, 17] *= 30
    xc = torch.from_numpy(x).cuda()
    q, s = bnb.quantize_rowwise(xc)
    eq, es = O.quantize_rowwise(x)
    assert np.array_equal(to_np(q), eq) and np.array_equal(to_np(s), es)
    oc, orow, cs, rs, _ = bnb.double_quant(xc)
    eoc, eor, ecs, ers = O.double_quant(x)
    assert np.array_equal(to_np(oc), eoc) and np.array_equal(to_np(orow), eor)
    assert np.array_equal(to_np(cs), ecs) and np.array_equal(to_np(rs), ers)
    q, r, c = bnb.quantize_colrow(xc)
    eq, er, ec = O.quantize_colrow(x)
    assert np.array_equal(to_np(q), eq) and np.array_equal(to_np(r), er) and np.array_equal(to_np(c), ec)
    assert np.array_equal(to_np(bnb.dequantize_colrow(q, r, c, torch.float16)), O.dequantize_colrow(eq, er, ec, "float16"))
    # pre-computed statistics are honoured
    oc2, or2, cs2, rs2, _ = bnb.double_quant(xc, col_stats=cs * 2, row_stats=rs * 2)
    assert torch.equal(cs2, cs * 2) and (or2.abs().max() <= 64)


def test_fp8_golden_and_oracle(golden):
    g = golden("fp8")
    c, s = bnb.quantize_fp8_e4m3(to_cuda(g["kat_in"], "float32"))
    assert [f"{v:02x}" for v in to_np(c)[0]] == "77 77 77 77 77 3f 38 30 08 00 00 f7".split()
    allc = torch.arange(256, dtype=torch.uint8, device="cuda").view(1, 256)
    d = bnb.dequantize_fp8_e4m3(allc, torch.ones(1, device="cuda"), torch.float32)
    assert np.array_equal(to_np(d), g["decode_all"], equal_nan=True)
    d = bnb.dequantize_fp8_e4m3(allc, torch.tensor([0.0371], device="cuda"), torch.float16)
    assert np.array_equal(to_np(d), g["decode_all_f16"], equal_nan=True)
    c, s = bnb.quantize_fp8_e4m3(to_cuda(g["edge_in"], "float32"))
    assert float(s[0]) == 1.0 and np.array_equal(to_np(c), g["edge_codes"])
    for dt in ("float16", "bfloat16", "float32"):
        c, s = bnb.quantize_fp8_e4m3(to_cuda(g[f"rnd_{dt}_in"], dt))
        assert np.array_equal(to_np(c), g[f"rnd_{dt}_codes"]) and np.array_equal(to_np(s), g[f"rnd_{dt}_scales"])
        od = dt if dt != "float32" else "float16"
        assert np.array_equal(to_np(bnb.dequantize_fp8_e4m3(c, s, getattr(torch, od))), g[f"rnd_{dt}_deq"])
    rng = np.random.default_rng(23)
    x = (rng.standard_normal((257, 1000)) * 0.02).astype(np.float32)
    x[5] = 0
    c, s = bnb.quantize_fp8_e4m3(torch.from_numpy(x).cuda())
    ec, es = O.quantize_fp8_e4m3(x)
    assert np.array_equal(to_np(c), ec) and np.array_equal(to_np(s), es)
    # every float within a few ulps below each power of two, where fp32 log2 rounds up
    vals = [448.0]
    for e in range(-9, 9):
        x0 = np.float32(2.0 ** e)
        for _ in range(8):
            vals.append(float(x0)); x0 = np.nextafter(x0, np.float32(0))
    v = np.array([vals + [-t for t in vals]], np.float32)
    c, s = bnb.quantize_fp8_e4m3(torch.from_numpy(v).cuda())
    ec, es = O.quantize_fp8_e4m3(v)
    assert np.array_equal(to_np(c), ec)
    with pytest.raises(ValueError, match="Input must be 2D"):
        bnb.quantize_fp8_e4m3(torch.zeros(4, device="cuda"))
