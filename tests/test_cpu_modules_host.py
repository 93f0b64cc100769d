"""CPU: host logic of the module-level drop-in surface — BitsAndBytesConfig, get_memory_footprint, the
constructors and signatures of the embedding / outlier-aware modules (as the reference declares them,
mps_bitsandbytes/integration.py and nn/*.py), rejection of CPU tensors, and the argument checks of the new
C-ABI entry points (calls that return before any CUDA work)."""
import ctypes as C
import inspect

import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from mps_bitsandbytes_b200 import _native as N


def test_config_matches_reference_values(golden):
    g = golden("modules")
    cfg = bnb.BitsAndBytesConfig(load_in_4bit=True, bnb_4bit_compute_dtype=torch.bfloat16, llm_int8_skip_modules=["lm_head"])
    assert [f"{k}={v}" for k, v in cfg.to_dict().items()] == list(g["cfg_dict"])
    assert str(bnb.BitsAndBytesConfig.from_dict(cfg.to_dict()).bnb_4bit_compute_dtype) == str(g["cfg_back_dtype"])
    assert bnb.BitsAndBytesConfig.from_dict({"load_in_8bit": True, "unknown_key": 1}).load_in_8bit
    with pytest.raises(ValueError, match="Cannot load in both 4-bit and 8-bit"):
        bnb.BitsAndBytesConfig(load_in_4bit=True, load_in_8bit=True)
    with pytest.raises(ValueError, match="bnb_4bit_quant_type must be 'nf4' or 'fp4'"):
        bnb.BitsAndBytesConfig(bnb_4bit_quant_type="int4")


def test_signatures_match_reference():
    sig = lambda f: list(inspect.signature(f).parameters)
    assert sig(bnb.quantize_model) == ["model", "quantization_config", "load_in_4bit", "load_in_8bit", "device",
                                       "compute_dtype", "modules_to_not_convert"]
    assert sig(bnb.replace_linear_with_4bit)[:4] == ["model", "quantization_config", "modules_to_not_convert", "current_key_name"]
    assert sig(bnb.replace_linear_with_8bit)[:4] == ["model", "quantization_config", "modules_to_not_convert", "current_key_name"]
    assert sig(bnb.Embedding4bit.__init__)[1:] == ["num_embeddings", "embedding_dim", "padding_idx", "quant_type", "blocksize", "device", "dtype"]
    assert sig(bnb.Embedding8bit.__init__)[1:] == ["num_embeddings", "embedding_dim", "padding_idx", "device", "dtype"]
    assert sig(bnb.OutlierAwareLinear.__init__)[1:] == ["in_features", "out_features", "bias", "threshold", "compute_dtype", "device"]
    assert sig(bnb.OutlierAwareLinear.from_linear) == ["linear", "threshold", "device"]
    assert sig(bnb.Embedding4bit.from_embedding) == ["embedding", "quant_type", "blocksize", "device"]


def test_module_buffers_and_footprint():
    e4 = bnb.Embedding4bit(10, 96, padding_idx=2, quant_type="fp4", blocksize=32)
    assert tuple(e4.weight_packed.shape) == (10, 48) and tuple(e4.weight_absmax.shape) == (10, 3)
    e8 = bnb.Embedding8bit(10, 96)
    assert e8.weight_int8.dtype == torch.int8 and tuple(e8.weight_scales.shape) == (10,)
    oal = bnb.OutlierAwareLinear(96, 24, bias=True)
    assert set(dict(oal.named_buffers())) == {"weight_int8", "weight_scales", "outlier_indices", "outlier_weights", "bias"}
    assert tuple(oal.outlier_weights.shape) == (24, 0) and "outliers=0" in oal.extra_repr()
    model = torch.nn.Sequential(e8, torch.nn.Linear(96, 4))
    fp = bnb.get_memory_footprint(model)
    n = 10 * 96 + 10 + 96 * 4 + 4
    assert fp["total_params"] == n and fp["quantized_params"] == 960
    assert fp["actual_size_gb"] == (960 + 40 + (96 * 4 + 4) * 4) / 1e9 and fp["fp16_size_gb"] == n * 2 / 1e9


def test_cpu_inputs_are_rejected():
    with pytest.raises(ValueError, match="cuda"):
        bnb.Embedding4bit(10, 64)(torch.tensor([1, 2]))
    with pytest.raises(ValueError, match="cuda"):
        bnb.Embedding8bit(10, 64)(torch.tensor([1, 2]))
    with pytest.raises(ValueError, match="cuda"):
        bnb.OutlierAwareLinear(64, 8)(torch.randn(2, 64))
    with pytest.raises(ValueError, match="cuda"):
        bnb.OutlierAwareLinear.from_linear(torch.nn.Linear(64, 8).half())    # no CPU quantiser


def test_new_entry_points_check_their_arguments():
    lib = N.lib()
    one = C.c_void_p(16)                       # a non-null pointer that is never dereferenced: the checks return first
    i64 = N.i64
    # bad index width, odd dim, unknown codebook, pitch smaller than dim / 2
    assert lib.mpsbnb_embedding_4bit(one, C.c_int(2), i64(1), one, i64(32), one, i64(4), i64(64), C.c_int(64), C.c_int(0), i64(-1), one, C.c_int(0), None) == -1
    assert lib.mpsbnb_embedding_4bit(one, C.c_int(8), i64(1), one, i64(32), one, i64(4), i64(63), C.c_int(64), C.c_int(0), i64(-1), one, C.c_int(0), None) == -1
    assert lib.mpsbnb_embedding_4bit(one, C.c_int(8), i64(1), one, i64(32), one, i64(4), i64(64), C.c_int(64), C.c_int(7), i64(-1), one, C.c_int(0), None) == -1
    assert lib.mpsbnb_embedding_4bit(one, C.c_int(8), i64(1), one, i64(16), one, i64(4), i64(64), C.c_int(64), C.c_int(0), i64(-1), one, C.c_int(0), None) == -1
    # nothing to do: success without touching the device
    assert lib.mpsbnb_embedding_4bit(None, C.c_int(8), i64(0), None, i64(32), None, i64(4), i64(64), C.c_int(64), C.c_int(0), i64(-1), None, C.c_int(0), None) == 0
    assert lib.mpsbnb_embedding_8bit(None, C.c_int(4), i64(0), None, None, i64(4), i64(64), i64(-1), None, C.c_int(1), None) == 0
    assert lib.mpsbnb_embedding_8bit(one, C.c_int(4), i64(1), one, one, i64(4), i64(64), i64(-1), one, C.c_int(9), None) == -1
    # outlier linear: operand type must be 16-bit, outlier list needs its weights, workspace must be large enough
    assert lib.mpsbnb_outlier_linear_workspace_bytes(i64(4), i64(8), i64(64)) == 256 + 512 + 1024
    assert lib.mpsbnb_outlier_linear_workspace_bytes(i64(0), i64(8), i64(64)) == 0
    args = lambda op, n_out, idx, ws_bytes: (one, C.c_int(0), i64(4), one, one, idx, i64(n_out), None, i64(8), i64(64), None,
                                             C.c_int(op), one, C.c_int(0), C.c_void_p(256), C.c_size_t(ws_bytes), None)
    assert lib.mpsbnb_outlier_linear(*args(2, 0, None, 4096)) == -1
    assert lib.mpsbnb_outlier_linear(*args(0, 3, one, 4096)) == -1
    assert lib.mpsbnb_outlier_linear(*args(0, 0, None, 100)) == -4


def test_short_argument_tensors_are_refused_before_any_kernel(monkeypatch):
    """The kernels take raw pointers, so every wrapper compares the lengths of caller-supplied tensors with the shapes
    before it launches (the reference raises a shape error in the same places).  Run on CPU tensors with the device
    check switched off and a library stub that fails the test if any entry point is reached."""
    from mps_bitsandbytes_b200 import functional as F

    class NoLaunch:
        def __getattr__(self, name):
            raise AssertionError(f"{name} reached with a short argument")

    monkeypatch.setattr(F, "_check_device", lambda *a, **k: None)
    monkeypatch.setattr(N, "require_cuda", lambda *a, **k: None, raising=False)
    monkeypatch.setattr(N, "lib", lambda: NoLaunch())
    K, n = 200, 64                                                  # rows padded to 256 in the packed layout
    packed = torch.zeros(n * 128, dtype=torch.uint8)
    st = bnb.QuantState(absmax=torch.ones(n * 4), shape=torch.Size((n, K)), blocksize=64, quant_type="nf4", dtype=torch.float16)
    x = torch.zeros(3, K, dtype=torch.float16)
    with pytest.raises(ValueError, match="packed weight"):
        bnb.matmul_4bit(x, packed[:-8], st)
    with pytest.raises(ValueError, match="bias"):
        bnb.matmul_4bit(x, packed, st, torch.zeros(n - 1, dtype=torch.float16))
    short = bnb.QuantState(absmax=st.absmax[:-1], shape=st.shape, blocksize=64, quant_type="nf4", dtype=st.dtype)
    with pytest.raises(ValueError, match="absmax"):
        bnb.matmul_4bit(x, packed, short)
    q = torch.zeros(8, 32, dtype=torch.int8)
    with pytest.raises(ValueError, match="scales"):
        bnb.dequantize_rowwise(q, torch.ones(7))
    with pytest.raises(ValueError, match="scales"):
        bnb.dequantize_fp8_e4m3(q.view(torch.uint8), torch.ones(7))
    with pytest.raises(ValueError, match="col_scales"):
        bnb.dequantize_colrow(q, torch.ones(8), torch.ones(31))
    with pytest.raises(ValueError, match="B_scales"):
        bnb.matmul_int8(q, torch.zeros(32, 16, dtype=torch.int8), torch.ones(8), torch.ones(15))
    with pytest.raises(ValueError, match="weight_row_scales"):
        bnb.matmul_colrow(torch.zeros(2, 32, dtype=torch.float16), q, torch.ones(7), torch.ones(32))
    with pytest.raises(ValueError, match="weight_scales"):
        bnb.matmul_fp8_e4m3(torch.zeros(2, 32, dtype=torch.float16), q.view(torch.uint8), torch.ones(7))
    with pytest.raises(ValueError, match="row_stats"):
        bnb.double_quant(torch.zeros(8, 32), row_stats=torch.ones(7))
    with pytest.raises(ValueError, match="absmax"):
        bnb.quantize_blockwise(torch.zeros(1000), absmax=torch.ones(1), blocksize=256)
