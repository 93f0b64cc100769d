"""GPU parity, 4-bit: the CUDA quantise / dequantise kernels, called through the C ABI, against
(1) the stored outputs of the reference itself and (2) the oracle on fresh seeded inputs.
Bit-exact: packed bytes, absmax (fp32 or int8 + second level) and dequantised values."""
import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from oracle import oracle_c, oracle_np as O
from gpu_util import to_cuda, to_np

pytestmark = pytest.mark.gpu


def check_case(w_np, dt, bs, qt, dq):
    w = to_cuda(w_np, dt)
    packed, st = bnb.quantize_4bit(w, blocksize=bs, compress_statistics=dq, quant_type=qt)
    exp_p, exp_a, exp_a2 = O.quantize_4bit(w_np, bs, qt, dq)
    assert packed.dtype == torch.uint8 and packed.dim() == 1
    assert np.array_equal(to_np(packed), exp_p)
    assert np.array_equal(to_np(st.absmax), exp_a)
    if dq:
        assert st.absmax.dtype == torch.int8 and st.state2.blocksize == 256
        assert np.array_equal(to_np(st.state2.absmax), exp_a2)
    shape2d = w_np.shape if w_np.ndim == 2 else (1, w_np.size)
    exp_d = O.dequantize_4bit(exp_p, exp_a, shape2d, bs, qt, dt, exp_a2).reshape(w_np.shape)
    got = bnb.dequantize_4bit(packed, st)
    assert got.dtype == w.dtype and tuple(got.shape) == tuple(w_np.shape)
    assert np.array_equal(to_np(got), exp_d, equal_nan=True)
    return packed, st


def test_golden_cases_from_reference(golden):
    g = golden("4bit")
    for name, qt, dt, n, k, bs, dq in g["cases"]:
        bs, dq = int(bs), bool(int(dq))
        w = to_cuda(g[name + "_w"], dt)
        packed, st = bnb.quantize_4bit(w, blocksize=bs, compress_statistics=dq, quant_type=qt)
        assert np.array_equal(to_np(packed), g[name + "_packed"]), name
        assert np.array_equal(to_np(st.absmax), g[name + "_absmax"]), name
        if dq:
            assert np.array_equal(to_np(st.state2.absmax), g[name + "_absmax2"]), name
        assert np.array_equal(to_np(bnb.dequantize_4bit(packed, st)), g[name + "_deq"]), name


def test_known_answers_and_special_inputs(golden):
    g = golden("4bit")
    p, _ = bnb.quantize_fp4(to_cuda(g["kat_fp4_in"], "float16"))
    assert np.array_equal(to_np(p), g["kat_fp4_packed"])
    p, _ = bnb.quantize_nf4(to_cuda(g["kat_nf4_in"], "float16"))
    assert np.array_equal(to_np(p), g["kat_nf4_packed"])
    for nm in ("zeros", "one", "tiny", "max"):
        for qt in ("nf4", "fp4"):
            x = g[f"sp_{nm}_{qt}_in"]
            dt = "float32" if x.dtype == np.float32 else "float16"
            p, st = bnb.quantize_4bit(to_cuda(x, dt), quant_type=qt)
            assert np.array_equal(to_np(p), g[f"sp_{nm}_{qt}_packed"])
            assert np.array_equal(to_np(st.absmax), g[f"sp_{nm}_{qt}_absmax"])
            d = to_np(bnb.dequantize_4bit(p, st))
            assert np.array_equal(d, g[f"sp_{nm}_{qt}_deq"]) and np.isfinite(d.astype(np.float32)).all()


def test_flat_path_for_non_2d_tensors(golden):
    g = golden("4bit")
    p, st = bnb.quantize_4bit(to_cuda(g["flat_in"], "float16"), quant_type="nf4")
    assert np.array_equal(to_np(p), g["flat_packed"]) and np.array_equal(to_np(st.absmax), g["flat_absmax"])
    assert np.array_equal(to_np(bnb.dequantize_4bit(p, st)), g["flat_deq"])
    p, st = bnb.quantize_4bit(to_cuda(g["flat3_in"], "float16"), quant_type="fp4", blocksize=32)
    assert np.array_equal(to_np(p), g["flat3_packed"]) and np.array_equal(to_np(st.absmax), g["flat3_absmax"])
    d = bnb.dequantize_4bit(p, st)
    assert tuple(d.shape) == (3, 5, 24) and np.array_equal(to_np(d), g["flat3_deq"])
    # without a QuantState: absmax only, flat fp16 output of nb * blocksize values
    d2 = bnb.dequantize_4bit(p, absmax=st.absmax, blocksize=32, quant_type="fp4")
    assert d2.dtype == torch.float16 and d2.numel() == st.absmax.numel() * 32
    assert np.array_equal(to_np(d2)[:360], g["flat3_deq"].reshape(-1))


@pytest.mark.parametrize("qt", ["nf4", "fp4"])
@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("dq", [False, True])
def test_random_weights_vs_oracle(qt, dt, dq):
    rng = np.random.default_rng(hash((qt, dt, dq)) % 2**31)
    for shape, scale in (((256, 512), 0.02), ((96, 1088), 1.0), ((33, 200), 40.0)):
        w = (rng.standard_normal(shape) * scale).astype(np.float32)
        w_np = O.cast_to(w, dt)
        check_case(w_np, dt, 64, qt, dq)


@pytest.mark.parametrize("shape", [(1, 1), (1, 63), (1, 65), (7, 13), (128, 127), (1, 1024), (1024, 1), (3, 17)])
@pytest.mark.parametrize("qt", ["nf4", "fp4"])
def test_odd_shapes_round_trip(shape, qt):
    rng = np.random.default_rng(shape[0] * 131 + shape[1])
    w_np = rng.standard_normal(shape).astype(np.float16)
    check_case(w_np, "float16", 64, qt, False)


@pytest.mark.parametrize("bs", [1, 2, 8, 16, 32, 64, 128, 256, 512, 1024, 4096])
def test_block_sizes(bs):
    rng = np.random.default_rng(bs)
    w_np = rng.standard_normal((12, 1536)).astype(np.float16)
    check_case(w_np, "float16", bs, "nf4", bs >= 64)
    check_case(w_np[:, :1000], "float16", bs, "fp4", False)


@pytest.mark.parametrize("qt", ["nf4", "fp4"])
def test_every_fp16_value_against_every_kind_of_block_maximum(qt):
    """All 63488 finite fp16 values as inputs, in blocks whose maximum sweeps small, mid-range
    and large magnitudes (each block = 63 values plus one maximum): codes must equal the
    reference's 16-way search for each (the CPU proof covers ALL maxima; this runs the kernel)."""
    bits = np.arange(65536, dtype=np.uint16)
    vals = bits.view(np.float16)
    vals = vals[np.isfinite(vals)]
    rng = np.random.default_rng(7)
    maxima = np.concatenate([np.float16([6e-8, 6.1e-5, 1e-3, 0.02, 0.37, 1.0, 3.14159, 1000.0, 65504.0]),
                             np.abs(rng.standard_normal(23)).astype(np.float16) + np.float16(0.01)])
    rows = []
    for a in maxima:
        v = vals[np.abs(vals.astype(np.float32)) <= np.float32(a)]
        pad = (-len(v)) % 63
        v = np.concatenate([v, np.zeros(pad, np.float16)]).reshape(-1, 63)
        blk = np.concatenate([v, np.full((v.shape[0], 1), a, np.float16)], axis=1)
        rows.append(blk.reshape(-1))
    flat = np.concatenate(rows)
    flat = np.concatenate([flat, np.zeros((-len(flat)) % 4096, np.float16)]).reshape(-1, 4096)
    w = torch.from_numpy(flat).cuda()
    packed, st = bnb.quantize_4bit(w, quant_type=qt)
    exp_p, exp_a = oracle_c.quantize_4bit(flat.astype(np.float32), 64, qt)
    assert np.array_equal(to_np(st.absmax), exp_a)
    assert np.array_equal(to_np(packed), exp_p)
    if qt == "fp4":
        p = to_np(packed)
        assert not ((p & 15) == 8).any() and not ((p >> 4) == 8).any()    # -0.0 is never emitted


def test_input_validation_messages():
    t = torch.randn(32, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError, match="blocksize must be positive"):
        bnb.quantize_4bit(t, blocksize=-1)
    with pytest.raises(ValueError, match="blocksize must be positive"):
        bnb.quantize_4bit(t, blocksize=0)
    with pytest.raises(ValueError, match="blocksize too large"):
        bnb.quantize_4bit(t, blocksize=100000)
    with pytest.raises(ValueError, match="power of 2"):
        bnb.quantize_4bit(t, blocksize=63)
    with pytest.raises(ValueError, match="quant_type must be"):
        bnb.quantize_4bit(t, quant_type="invalid")
    with pytest.raises(ValueError, match="blocksize must be positive"):
        bnb.quantize_blockwise(torch.randn(1024, device="cuda"), blocksize=-1)
    with pytest.raises(ValueError, match="Either quant_state or absmax"):
        bnb.dequantize_4bit(torch.zeros(32, dtype=torch.uint8, device="cuda"))


def test_preallocated_out_and_given_absmax():
    rng = np.random.default_rng(5)
    w_np = rng.standard_normal((16, 256)).astype(np.float16)
    w = torch.from_numpy(w_np).cuda()
    out = torch.zeros(16, 128, dtype=torch.uint8, device="cuda")
    p, st = bnb.quantize_4bit(w, out=out)
    exp_p, exp_a, _ = O.quantize_4bit(w_np, 64, "nf4")
    assert np.array_equal(to_np(out).reshape(-1), exp_p) and np.array_equal(to_np(p), exp_p)
    # caller-supplied block maxima (twice the true ones): values normalise to half range
    am = torch.from_numpy(exp_a * 2).cuda().view(16, 4)
    p2, st2 = bnb.quantize_4bit(w, absmax=am)
    v = (w_np.astype(np.float32).reshape(16, 4, 64) / (exp_a * 2).reshape(16, 4, 1)).astype(np.float32)
    idx = np.abs(v[..., None] - O.NF4_CODE).argmin(-1).astype(np.uint8).reshape(16, 256)
    assert np.array_equal(to_np(p2), (idx[:, 0::2] | (idx[:, 1::2] << 4)).reshape(-1))
    dst = torch.empty(16, 256, dtype=torch.float16, device="cuda")
    r = bnb.dequantize_4bit(p, st, out=dst)
    assert r is dst and np.array_equal(to_np(dst), O.dequantize_4bit(exp_p, exp_a, (16, 256), 64, "nf4", "float16"))


def test_sentinels_around_outputs_stay_intact():
    """Kernels write exactly their outputs: guard bands on both sides of packed and absmax."""
    import ctypes as C
    from mps_bitsandbytes_b200 import _native as N
    rng = np.random.default_rng(9)
    for rows, cols in ((5, 200), (64, 1024), (3, 77)):
        w = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float16)).cuda()
        kp = -(-cols // 64) * 64
        guard = 256
        pbuf = torch.full((rows * kp // 2 + 2 * guard,), 0xA5, dtype=torch.uint8, device="cuda")
        abuf = torch.full((rows * kp // 64 + 2 * guard,), -777.0, dtype=torch.float32, device="cuda")
        p_view = pbuf[guard:guard + rows * kp // 2]
        a_view = abuf[guard:guard + rows * kp // 64]
        N.check(N.lib().mpsbnb_quantize_4bit(N.ptr(w), 0, N.i64(rows), N.i64(cols), C.c_int(64), C.c_int(0), None,
                                             N.ptr(p_view), N.ptr(a_view), N.stream()), "quantize_4bit")
        torch.cuda.synchronize()
        assert (pbuf[:guard] == 0xA5).all() and (pbuf[-guard:] == 0xA5).all()
        assert (abuf[:guard] == -777.0).all() and (abuf[-guard:] == -777.0).all()
        exp_p, exp_a, _ = O.quantize_4bit(to_np(w), 64, "nf4")
        assert np.array_equal(to_np(p_view), exp_p) and np.array_equal(to_np(a_view), exp_a)


def test_config1_shape_round_trip_properties():
    """BASELINE config 1 at full size (4096 x 4096 fp16 ~ N(0, 0.02)): size-independent
    properties, plus bit parity with the C oracle."""
    torch.manual_seed(0)
    w = (torch.randn(4096, 4096) * 0.02).half()
    wc = w.cuda()
    packed, st = bnb.quantize_nf4(wc)
    assert packed.numel() == 4096 * 2048 and st.absmax.numel() == 262144
    exp_p, exp_a = oracle_c.quantize_4bit(w.float().numpy(), 64, "nf4")
    assert np.array_equal(to_np(packed), exp_p) and np.array_equal(to_np(st.absmax), exp_a)
    d = bnb.dequantize_nf4(packed, st)
    exp_d = oracle_c.dequantize_4bit(exp_p, exp_a, (4096, 4096), 64, "nf4").astype(np.float16)
    assert np.array_equal(to_np(d), exp_d)
    # idempotence: quantising the dequantised tensor reproduces the same codes and maxima...
    p2, st2 = bnb.quantize_nf4(d)
    d2 = bnb.dequantize_nf4(p2, st2)
    # ...up to fp16 rounding of the block maximum; the second round trip must be a fixed point
    p3, st3 = bnb.quantize_nf4(d2)
    assert torch.equal(bnb.dequantize_nf4(p3, st3), d2)
    err = (d.float() - wc.float()).abs().mean() / wc.float().abs().mean()
    assert err < 0.25
