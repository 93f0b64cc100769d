"""GPU parity of the two decode kernels against the oracle: the one for batch <= 8 (dot products for
batch <= 2, mma.sync above) in both activation types, and the one for batch 9 .. 32 (weights expanded into
tensor memory, tcgen05.mma).  Bound: rel_err <= 1e-2."""
import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from mps_bitsandbytes_b200 import _native, stack as S
from oracle import oracle_np as O
from gpu_util import assert_device_ok, rel_err, to_cuda, to_np
from test_gpu_stack import oracle_stack

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _case(rng, M, N, K, qt, dq, dt):
    w = O.cast_to((rng.standard_normal((N, K)) * 0.02).astype(np.float32), dt)
    x = O.cast_to(rng.standard_normal((M, K)).astype(np.float32), dt)
    bias = O.cast_to(rng.standard_normal(N).astype(np.float32), dt)
    packed, st = bnb.quantize_4bit(to_cuda(w, dt), compress_statistics=dq, quant_type=qt)
    p, a, a2 = O.quantize_4bit(w, 64, qt, dq)
    y = bnb.matmul_4bit(to_cuda(x, dt), packed, st, to_cuda(bias, dt))
    ref = O.matmul_4bit(x, p, a, (N, K), 64, qt, dt, a2, bias, "float32")
    return rel_err(to_np(y), ref)


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
@pytest.mark.parametrize("M", [1, 2, 3, 8])
def test_default_kernel_both_types(M, dt):
    rng = np.random.default_rng(100 + M)
    for (N, K, qt, dq) in [(200, 1088, "nf4", True), (96, 4104, "fp4", False), (4096, 4096, "nf4", False)]:
        assert _case(rng, M, N, K, qt, dq, dt) <= TOL, (N, K, qt, dq)
    assert_device_ok()


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
@pytest.mark.parametrize("M", [9, 12, 16, 17, 25, 32])
def test_tcgen05_kernel_matches_oracle(M, dt):
    rng = np.random.default_rng(200 + M)
    # one stage / many stages / ragged K and N / scale groups that are not 4-aligned (nb = 65) / 33 row tiles
    for (N, K, qt, dq) in [(128, 256, "nf4", False), (200, 1088, "nf4", True), (96, 4104, "fp4", False),
                           (4100, 2304, "nf4", True), (64, 64, "fp4", True)]:
        assert _case(rng, M, N, K, qt, dq, dt) <= TOL, (N, K, qt, dq)
    assert_device_ok()


@pytest.mark.parametrize("M", [9, 20, 32])
def test_tcgen05_kernel_grouped_stack(M):
    """The grouped launch cuts row tiles between CTAs (fp32 workspace + arrival counters): three layers, graph
    replayed twice, so the workspace has to come back to zero every time."""
    cfg = S.StackConfig("tiny", hidden=256, ffn=704, kv=64, layers=3)
    st = S.LayerStack(cfg, device="cuda:0", quant_type="nf4", double_quant=True, seed=5, boundary="kernel")
    x = np.random.default_rng(M).standard_normal((M, cfg.hidden)).astype(np.float16)
    st.prepare(M, use_graph=True)
    ref_h, ref_out = oracle_stack(st, x)
    for _ in range(3):
        h = st.step(torch.from_numpy(x).cuda())
        torch.cuda.synchronize()
        assert rel_err(to_np(h), ref_h) <= TOL
        for name in ("q", "k", "v", "gate", "up"):
            assert rel_err(to_np(st.out[name]), ref_out[name]) <= TOL, name
    assert_device_ok()
