"""GPU parity: quantised embedding look-ups (bit-exact) and the outlier-aware INT8 linear
(matmul bound: max |y - ref| / max |ref| <= 1e-2), through the modules and the C ABI, against the
reference's stored outputs and the oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from mps_bitsandbytes_b200 import _native as N
from oracle import oracle_np as O
from gpu_util import assert_device_ok, rel_err, to_cuda, to_np

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _pad(v):
    return None if v == "None" else int(v)


def test_embedding_modules_match_reference_bit_exact(golden):
    g = golden("modules")
    for name, V, D, bs, qt, dt, pad in g["ecases"]:
        V, D, bs, pad = int(V), int(D), int(bs), _pad(pad)
        emb = torch.nn.Embedding(V, D, padding_idx=pad)
        emb.weight.data = to_cuda(g[name + "_w"], dt)
        ids = torch.from_numpy(g[name + "_ids"]).cuda()
        e4 = bnb.Embedding4bit.from_embedding(emb, quant_type=qt, blocksize=bs)
        assert np.array_equal(to_np(e4.weight_packed), g[name + "_packed"])
        assert np.array_equal(to_np(e4.weight_absmax), g[name + "_absmax"])
        out = e4(ids)
        assert tuple(out.shape) == (3, 7, D) and out.dtype == (torch.bfloat16 if dt == "bfloat16" else torch.float16)
        assert np.array_equal(to_np(out), g[name + "_out4"]), name
        assert np.array_equal(to_np(e4(ids.int())), g[name + "_out4"])          # int32 indices
        e8 = bnb.Embedding8bit.from_embedding(emb)
        assert np.array_equal(to_np(e8.weight_int8), g[name + "_q8"]) and np.array_equal(to_np(e8.weight_scales), g[name + "_s8"])
        assert np.array_equal(to_np(e8(ids)), g[name + "_out8"]), name
    assert bnb.EmbeddingFP4.from_embedding(torch.nn.Embedding(9, 64).half().cuda()).quant_type == "fp4"
    assert bnb.EmbeddingNF4(9, 64, device="cuda").quant_type == "nf4"
    with pytest.raises(ValueError, match="embedding_dim must be even"):
        bnb.Embedding4bit(4, 7)
    with pytest.raises(ValueError, match="quant_type must be 'nf4' or 'fp4'"):
        bnb.Embedding4bit(4, 8, quant_type="int4")


@pytest.mark.parametrize("V,D,bs,qt,dt,n_idx", [
    (1000, 4096, 64, "nf4", "float16", 513), (333, 80, 16, "fp4", "bfloat16", 77), (64, 6, 64, "nf4", "float16", 5),
    (50, 200, 128, "fp4", "float32", 31), (2, 64, 64, "nf4", "float16", 0)])
def test_embedding_lookup_vs_oracle(V, D, bs, qt, dt, n_idx):
    """Vector and element paths, ragged last block, fp32 output, empty index list, out-of-range index."""
    rng = np.random.default_rng(V + D)
    w = O.cast_to((rng.standard_normal((V, D)) * 0.05).astype(np.float32), "float16")
    packed, absmax, _ = O.quantize_4bit(w, bs, qt, False)
    packed = np.ascontiguousarray(packed.reshape(V, -1)[:, :D // 2]); absmax = absmax.reshape(V, -1)
    ids = rng.integers(0, V, size=n_idx)
    layer = bnb.Embedding4bit(V, D, padding_idx=1, quant_type=qt, blocksize=bs, device="cuda", dtype=getattr(torch, dt))
    layer.weight_packed.copy_(torch.from_numpy(packed)); layer.weight_absmax.copy_(torch.from_numpy(absmax))
    out = layer(torch.from_numpy(ids).cuda())
    assert np.array_equal(to_np(out), O.embedding_4bit(ids, packed, absmax, D, bs, qt, dt, 1))
    q8, s8 = O.quantize_rowwise(w)
    l8 = bnb.Embedding8bit(V, D, padding_idx=1, device="cuda", dtype=getattr(torch, dt))
    l8.weight_int8.copy_(torch.from_numpy(q8)); l8.weight_scales.copy_(torch.from_numpy(s8))
    assert np.array_equal(to_np(l8(torch.from_numpy(ids).cuda())), O.embedding_8bit(ids, q8, s8, dt, 1))
    if n_idx:
        bad = torch.tensor([0, V, -1, V - 1]).cuda()               # V and -1 are out of range: zero rows, no fault
        got = to_np(layer(bad))
        assert not got[1].any() and not got[2].any()
        assert np.array_equal(got[[0, 3]], O.embedding_4bit(np.array([0, V - 1]), packed, absmax, D, bs, qt, dt, 1))
    assert_device_ok()


def test_outlier_aware_linear_matches_reference(golden):
    g = golden("modules")
    for name, M, Nn, K, dt, bias, nout in g["ocases"]:
        lin = torch.nn.Linear(int(K), int(Nn), bias=bias == "True")
        lin.weight.data = to_cuda(g[name + "_w"], dt)
        if bias == "True":
            lin.bias.data = to_cuda(g[name + "_b"], dt)
        layer = bnb.OutlierAwareLinear.from_linear(lin.cuda(), threshold=6.0)
        assert np.array_equal(to_np(layer.outlier_indices), g[name + "_idx"])
        assert np.array_equal(to_np(layer.weight_int8), g[name + "_q"]) and np.array_equal(to_np(layer.weight_scales), g[name + "_s"])
        assert np.array_equal(to_np(layer.outlier_weights), g[name + "_ow"])
        y = layer(to_cuda(g[name + "_x"], dt))
        assert tuple(y.shape) == g[name + "_y"].shape and y.dtype == getattr(torch, dt)
        assert rel_err(to_np(y), g[name + "_y"]) <= TOL, (name, rel_err(to_np(y), g[name + "_y"]))
        assert f"outliers={nout}" in layer.extra_repr()
    # fp32 activations into an fp16 layer
    lin = torch.nn.Linear(64, 16).half()
    lin.weight.data = torch.from_numpy(g["o32_w"]); lin.bias.data = torch.from_numpy(g["o32_b"])
    layer = bnb.OutlierAwareLinear.from_linear(lin.cuda())
    assert rel_err(to_np(layer(torch.from_numpy(g["o32_x"]).cuda())), g["o32_y"]) <= TOL
    assert_device_ok()


def test_outlier_linear_config4_shape_vs_oracle():
    """LLM.int8 case of the benchmark configurations at reduced size: activations [512, K] with 0.5 % of
    the columns at magnitude ~20, the same columns large in the weight, through the C ABI."""
    rng = np.random.default_rng(4)
    M, K, Nn = 512, 1024, 768
    cols = rng.choice(K, size=5, replace=False)
    w = (rng.standard_normal((Nn, K)) * 0.02).astype(np.float32); w[:, cols] *= 15
    x = rng.standard_normal((M, K)).astype(np.float32); x[:, cols] *= 20
    w16, x16 = O.cast_to(w, "float16"), O.cast_to(x, "float16")
    q, s, idx, ow = O.outlier_from_linear(w16, 6.0, "float16")
    assert set(idx.tolist()) == set(cols.tolist())
    bias = rng.standard_normal(Nn).astype(np.float16)
    ref = O.outlier_linear(x16, q, s, idx, ow, bias, "float16")
    lib = N.lib()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    xd, qd, sd, idxd, owd, bd = t(x16), t(q), t(s), t(idx), t(ow), t(bias)
    y = torch.empty(M, Nn, dtype=torch.float16, device="cuda")
    ws = torch.empty(lib.mpsbnb_outlier_linear_workspace_bytes(N.i64(M), N.i64(Nn), N.i64(K)), dtype=torch.uint8, device="cuda")
    args = lambda wsz: (N.ptr(xd), C.c_int(N.F16), N.i64(M), N.ptr(qd), N.ptr(sd), N.ptr(idxd), N.i64(len(idx)), N.ptr(owd),
                        N.i64(Nn), N.i64(K), N.ptr(bd), C.c_int(N.F16), N.ptr(y), C.c_int(N.F16), N.ptr(ws), C.c_size_t(wsz), N.stream())
    assert lib.mpsbnb_outlier_linear(*args(ws.numel())) == 0
    assert rel_err(to_np(y), ref) <= TOL, rel_err(to_np(y), ref)
    # without the decomposition the int8 grid of x is ~20x coarser: the split must be what keeps the error small
    q0, s0 = O.quantize_rowwise(w16)
    plain = O.outlier_linear(x16, q0, s0, np.zeros(0, np.int64), np.zeros((Nn, 0), np.float16), bias, "float16")
    exact = (x16.astype(np.float32) @ w16.astype(np.float32).T) + bias.astype(np.float32)
    assert rel_err(to_np(y), exact) < 0.5 * rel_err(plain, exact)
    assert lib.mpsbnb_outlier_linear(*args(ws.numel() - 1)) == -4                  # MPSBNB_ERR_WORKSPACE
    assert_device_ok()
