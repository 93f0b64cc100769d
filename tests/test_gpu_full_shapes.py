"""GPU parity at the full shapes the benchmark quotes numbers on, against the C / numpy oracle:
the FP4 + double-quant prefill GEMM (11008 x 4096 weight, x [2048, 4096]), the INT8 / FP8 /
outlier-split matmuls (x [512, 4096] with outlier columns, weight 4096 x 16384), Llama-70B-wide
layers (28672 x 8192, 8192 x 28672, 1024 x 8192) at batch 1 / 32 / 512 and a Llama-2-7B layer at
batch 16.  Where the oracle's full matmul would take minutes, a seeded sample of the x rows is
compared over ALL output columns (every weight element takes part).  Bound: rel_err <= 1e-2
(both norms of gpu_util.rel_err)."""
import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from oracle import oracle_c, oracle_np as O
from gpu_util import assert_device_ok, rel_err, to_np

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _weights(n, k, seed, scale=0.02):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    return (torch.randn(n, k, device="cuda", generator=g) * scale).half()


def _inputs(m, k, seed):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    return torch.randn(m, k, device="cuda", generator=g).half()


def _oracle_absmax(st):
    """fp32 absmax [N * nb] of a QuantState as the oracle expands it (double quantisation undone)."""
    if st.state2 is None:
        return to_np(st.absmax).astype(np.float32)
    return oracle_c.dequantize_absmax(to_np(st.absmax), to_np(st.state2.absmax))


def _check_4bit(n, k, m, qt, seed, sample=None):
    w = _weights(n, k, seed)
    packed, st = bnb.quantize_4bit(w, compress_statistics=True, quant_type=qt)
    del w
    x = _inputs(m, k, seed + 1)
    y = bnb.matmul_4bit(x, packed, st)
    assert tuple(y.shape) == (m, n) and y.dtype == torch.float16
    rows = np.arange(m) if sample is None or sample >= m else np.sort(np.random.default_rng(seed).choice(m, sample, replace=False))
    ref = oracle_c.matmul_4bit_f16(to_np(x)[rows], to_np(packed), _oracle_absmax(st), n, k, 64, qt)
    err = rel_err(to_np(y)[rows], ref)
    assert err <= TOL, (n, k, m, qt, err)
    assert_device_ok()


def test_config2_fp4_prefill_full_size():
    """FP4 + double quant, weight 11008 x 4096, x [2048, 4096]: 64 sampled x rows, all 11008 columns."""
    _check_4bit(11008, 4096, 2048, "fp4", seed=20, sample=64)


@pytest.mark.parametrize("n,k", [(28672, 8192), (8192, 28672), (1024, 8192)])
@pytest.mark.parametrize("m", [1, 32, 512])
def test_llama70b_wide_layers(n, k, m):
    _check_4bit(n, k, m, "nf4", seed=50 + m, sample=8)


@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008)])
def test_llama7b_layer_batch16(n, k):
    _check_4bit(n, k, 16, "nf4", seed=30, sample=None)


@pytest.mark.parametrize("m", [40, 64, 100, 128, 200, 256])
def test_middle_band_batches(m):
    """33 <= M <= 256 on a 4096 x 4096 weight: the band between the decode and the prefill shapes."""
    _check_4bit(4096, 4096, m, "nf4", seed=70 + m, sample=16)


def _config4_inputs():
    M, K, Nn = 512, 4096, 16384
    w = _weights(Nn, K, 40)
    x = _inputs(M, K, 41)
    g = torch.Generator(device="cuda"); g.manual_seed(42)
    cols = torch.randperm(K, device="cuda", generator=g)[: K // 200]
    x[:, cols] *= 20.0
    return M, K, Nn, w, x, cols


def test_config4_int8_fp8_full_size():
    """x [512, 4096] with 0.5 % of the columns at magnitude ~20, weight 4096 x 16384: matmul_int8, matmul_colrow,
    matmul_fp8_e4m3 against the numpy oracle on 32 sampled rows and all 16384 columns."""
    M, K, Nn, w, x, _ = _config4_inputs()
    rows = np.sort(np.random.default_rng(4).choice(M, 32, replace=False))
    x_np = to_np(x)
    # matmul_int8: A row-wise, B = W^T with per-column scales
    aq, a_s = bnb.quantize_rowwise(x)
    bq_t, b_s = bnb.quantize_rowwise(w)
    bq = bq_t.t().contiguous()
    y = bnb.matmul_int8(aq, bq, a_s, b_s)
    ref = O.matmul_int8(to_np(aq)[rows], to_np(bq), to_np(a_s)[rows], to_np(b_s))
    assert rel_err(to_np(y)[rows], ref) <= TOL, rel_err(to_np(y)[rows], ref)
    del bq, bq_t
    # col + row scaled int8 weight, 16-bit activations
    cq, cr, cc = bnb.quantize_colrow(w)
    y = bnb.matmul_colrow(x, cq, cr, cc)
    ref = O.matmul_colrow(x_np[rows], to_np(cq), to_np(cr), to_np(cc))
    assert rel_err(to_np(y)[rows], ref) <= TOL, rel_err(to_np(y)[rows], ref)
    del cq
    # FP8 E4M3 weight
    f8, f8s = bnb.quantize_fp8_e4m3(w)
    y = bnb.matmul_fp8_e4m3(x, f8, f8s)
    ref = O.matmul_fp8_e4m3(x_np[rows], to_np(f8), to_np(f8s))
    assert rel_err(to_np(y)[rows], ref) <= TOL, rel_err(to_np(y)[rows], ref)
    assert_device_ok()


def test_config4_outlier_split_full_size():
    """OutlierAwareLinear on the same shapes: the columns that are large in x are large in the weight too, so the
    conversion keeps them in 16 bits."""
    M, K, Nn, w, x, cols = _config4_inputs()
    w[:, cols] *= 15.0
    lin = torch.nn.Linear(K, Nn, bias=False, device="cuda", dtype=torch.float16)
    lin.weight.data = w
    layer = bnb.OutlierAwareLinear.from_linear(lin)
    found = set(layer.outlier_indices.tolist())                 # the 20 scaled columns, plus columns whose largest weight
    assert set(cols.tolist()) <= found and len(found) < 200     # among 16384 rows happens to pass the 6 x mean rule
    y = layer(x)
    rows = np.sort(np.random.default_rng(5).choice(M, 32, replace=False))
    ref = O.outlier_linear(to_np(x)[rows], to_np(layer.weight_int8), to_np(layer.weight_scales),
                           to_np(layer.outlier_indices), to_np(layer.outlier_weights), None, "float16")
    assert rel_err(to_np(y)[rows], ref) <= TOL, rel_err(to_np(y)[rows], ref)
    assert_device_ok()
