"""GPU parity of the layer stack (grouped streaming GEMV for batch <= 8, per-linear kernels above)
against the oracle running the same dataflow on the weights read back from the device."""
import numpy as np
import pytest
import torch

from mps_bitsandbytes_b200 import stack as S
from oracle import oracle_np as O
from gpu_util import assert_device_ok, rel_err, to_np

pytestmark = pytest.mark.gpu


def oracle_stack(st: S.LayerStack, x: np.ndarray):
    cfg = st.cfg
    h = x.astype(np.float16)
    outs = {}
    for l in range(st.layers):
        e = np.tile(h, (1, -(-cfg.ffn // cfg.hidden)))[:, :cfg.ffn]
        y = {}
        for pr in st.proj[l]:
            a2 = None if pr.absmax2 is None else to_np(pr.absmax2)
            w = O.dequantize_4bit(to_np(pr.packed), to_np(pr.absmax), (pr.n, pr.k), 64, st.quant_type, "float16", a2)
            xin = e if pr.name == "down" else h
            y[pr.name] = xin.astype(np.float32) @ w.astype(np.float32).T
        outs = {k: v.astype(np.float16) for k, v in y.items()}
        h = (np.float32(st.alpha) * (y["o"] + y["down"])).astype(np.float16)
    return h, outs


@pytest.mark.parametrize("M,boundary", [(1, "kernel"), (1, "inline"), (1, "stream"), (3, "inline"), (3, "stream"),
                                        (8, "kernel"), (8, "stream"), (12, "kernel"), (16, "kernel"), (24, "kernel")])
@pytest.mark.parametrize("qt,dq", [("nf4", True), ("fp4", False)])
def test_small_stack_matches_oracle(M, boundary, qt, dq):
    """boundary: the layer boundary as its own kernel, as the closing step of the grouped GEMV launch (last CTA), or
    streamed tile by tile from inside the launch."""
    cfg = S.StackConfig("tiny", hidden=256, ffn=704, kv=64, layers=3)
    st = S.LayerStack(cfg, device="cuda:0", quant_type=qt, double_quant=dq, seed=5, boundary=boundary)
    rng = np.random.default_rng(M)
    x = rng.standard_normal((M, cfg.hidden)).astype(np.float16)
    for use_graph in (False, True):
        st.prepare(M, use_graph=use_graph)
        h = st.step(torch.from_numpy(x).cuda())
        torch.cuda.synchronize()
        ref_h, ref_out = oracle_stack(st, x)
        assert rel_err(to_np(h), ref_h) <= 1e-2, (use_graph, rel_err(to_np(h), ref_h))
        for name in ("q", "k", "v", "gate", "up"):
            assert rel_err(to_np(st.out[name]), ref_out[name]) <= 1e-2, name
        # a second step from the same input gives the same answer (accumulators were re-armed)
        h2 = st.step(torch.from_numpy(x).cuda()).clone()
        torch.cuda.synchronize()
        assert rel_err(to_np(h2), ref_h) <= 1e-2
    assert_device_ok()


@pytest.mark.parametrize("M", [1, 5])
def test_streamed_boundary_one_launch_per_layer(M):
    """The streamed boundary without the whole-stack launch (persistent=False): one grouped launch per layer."""
    cfg = S.StackConfig("tiny", hidden=256, ffn=704, kv=64, layers=4)
    st = S.LayerStack(cfg, device="cuda:0", seed=6, boundary="stream", persistent=False)
    x = np.random.default_rng(M).standard_normal((M, cfg.hidden)).astype(np.float16)
    st.prepare(M, use_graph=True)
    ref_h, _ = oracle_stack(st, x)
    for _ in range(2):
        h = st.step(torch.from_numpy(x).cuda())
        torch.cuda.synchronize()
        assert rel_err(to_np(h), ref_h) <= 1e-2
    assert_device_ok()


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("qt,dq", [("nf4", True), ("fp4", False)])
def test_whole_stack_in_one_launch(M, qt, dq):
    """persistent=True: all layers in ONE cooperative launch (segment = layer); layers hand h over through flags."""
    cfg = S.StackConfig("tiny", hidden=256, ffn=704, kv=64, layers=5)
    st = S.LayerStack(cfg, device="cuda:0", quant_type=qt, double_quant=dq, seed=8, boundary="stream", persistent=True)
    x = np.random.default_rng(10 + M).standard_normal((M, cfg.hidden)).astype(np.float16)
    for use_graph in (False, True):
        st.prepare(M, use_graph=use_graph)
        ref_h, ref_out = oracle_stack(st, x)
        for _ in range(3):
            h = st.step(torch.from_numpy(x).cuda())
            torch.cuda.synchronize()
            assert rel_err(to_np(h), ref_h) <= 1e-2, use_graph
            for name in ("q", "k", "v", "gate", "up"):
                assert rel_err(to_np(st.out[name]), ref_out[name]) <= 1e-2, name
    assert_device_ok()


@pytest.mark.parametrize("M,hidden,ffn", [(1, 256, 704), (3, 256, 704), (1, 2048, 5120), (1, 1024, 2816), (2, 2048, 5120)])
def test_whole_stack_in_one_launch_tagged_exchange(M, hidden, ffn):
    """tagged_exchange=True: h travels between layers as {two values, tag} entries, no flags.  Batch 1 with stages of whole
    runs of four columns goes through the loaders' staging buffers; everything else reads the entries where they lie
    (704 = a short last stage that straddles the period of `down`; 2816 = 2 x 1024 + 768; batch 2 and 3)."""
    cfg = S.StackConfig("tiny", hidden=hidden, ffn=ffn, kv=64, layers=4)
    st = S.LayerStack(cfg, device="cuda:0", seed=12, boundary="stream", persistent=True, tagged_exchange=True)
    x = np.random.default_rng(20 + M).standard_normal((M, cfg.hidden)).astype(np.float16)
    for use_graph in (False, True):
        st.prepare(M, use_graph=use_graph)
        assert st._tagged
        ref_h, ref_out = oracle_stack(st, x)
        for _ in range(3):
            h = st.step(torch.from_numpy(x).cuda())
            torch.cuda.synchronize()
            assert st.check_status() == 0
            assert rel_err(to_np(h), ref_h) <= 1e-2, use_graph
            for name in ("q", "k", "v", "gate", "up"):
                assert rel_err(to_np(st.out[name]), ref_out[name]) <= 1e-2, name
    assert_device_ok()


def test_llama7b_layer_shapes_one_layer():
    """One layer at the real Llama-2-7B widths, batch 1 (the benchmark's unit of work)."""
    st = S.LayerStack(S.LLAMA2_7B, device="cuda:0", layers=1, seed=9)
    st.prepare(1, use_graph=False)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((1, 4096)).astype(np.float16)
    h = st.step(torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    ref_h, ref_out = oracle_stack(st, x)
    assert rel_err(to_np(h), ref_h) <= 1e-2
    assert rel_err(to_np(st.out["gate"]), ref_out["gate"]) <= 1e-2
    assert_device_ok()
