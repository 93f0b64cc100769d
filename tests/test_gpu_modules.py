"""GPU parity, modules: Linear4bit / Linear8bit / LinearFP8 against stored reference outputs,
and the state-dict format of the reference (quantise-on-load, QuantState dict)."""
import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from gpu_util import rel_err, to_cuda, to_np

pytestmark = pytest.mark.gpu


def make_linear(g):
    lin = torch.nn.Linear(128, 48).half()
    lin.weight.data.copy_(torch.from_numpy(g["mod_w"]))
    lin.bias.data.copy_(torch.from_numpy(g["mod_b"]))
    return lin.cuda()


def test_modules_match_reference_outputs(golden):
    g = golden("matmul")
    lin = make_linear(g)
    x = to_cuda(g["mod_x"], "float16")
    l4 = bnb.Linear4bit.from_linear(lin, quant_type="nf4", compress_statistics=True)
    y = l4(x)
    assert tuple(y.shape) == (2, 3, 48) and y.dtype == torch.float16
    assert rel_err(to_np(y), g["mod_l4_nf4"]) <= 1e-2
    assert rel_err(to_np(bnb.Linear4bit.from_linear(lin, quant_type="fp4")(x)), g["mod_l4_fp4"]) <= 1e-2
    assert rel_err(to_np(bnb.Linear8bit.from_linear(lin)(x)), g["mod_l8"]) <= 1e-2
    assert rel_err(to_np(bnb.LinearFP8.from_linear(lin)(x)), g["mod_f8"]) <= 1e-2
    assert l4.weight.dtype == torch.uint8 and l4.weight.dim() == 1 and l4.quant_state is l4.weight_quant_state
    assert tuple(l4.dequantize().shape) == (48, 128)


def test_linear4bit_state_dict_round_trip_and_quantise_on_load(golden):
    g = golden("matmul")
    lin = make_linear(g)
    x = to_cuda(g["mod_x"], "float16")
    l4 = bnb.Linear4bit.from_linear(lin, quant_type="fp4", compress_statistics=True)
    sd = l4.state_dict()
    assert "weight_quant_state" in sd and set(sd["weight_quant_state"]) == {"absmax", "shape", "blocksize", "quant_type", "dtype", "state2"}
    fresh = bnb.Linear4bit(128, 48, device="cuda", quant_type="fp4", compress_statistics=True)
    fresh.load_state_dict(sd)
    assert torch.equal(fresh(x), l4(x))
    # a floating-point checkpoint is quantised while loading
    fp = bnb.Linear4bit(128, 48, device="cuda", quant_type="fp4", compress_statistics=True)
    fp.load_state_dict(lin.state_dict())
    assert torch.equal(fp.weight, l4.weight) and torch.equal(fp(x), l4(x))
    # a checkpoint with another quant_type wins, with a warning
    other = bnb.Linear4bit(128, 48, device="cuda", quant_type="nf4")
    with pytest.warns(UserWarning, match="quant_type mismatch"):
        other.load_state_dict(sd)
    assert other.quant_type == "fp4" and torch.equal(other(x), l4(x))
    with pytest.raises(RuntimeError, match="Weight not quantized"):
        bnb.Linear4bit(128, 48, device="cuda")(x)


def test_linear8bit_cache_and_fp8_dequantize(golden):
    g = golden("matmul")
    lin = make_linear(g)
    l8 = bnb.Linear8bit.from_linear(lin, use_cache=True)
    w1 = l8._get_weight()
    assert l8._get_weight() is w1
    l8.clear_cache()
    assert l8._weight_cache is None
    assert l8.weight_int8.dtype == torch.int8 and l8.weight_scales.dtype == torch.float32
    f8 = bnb.LinearFP8.from_linear(lin)
    assert tuple(f8.dequantize().shape) == (48, 128)
    # the reference's encoder maps everything in (240, 448] — the row maximum included — to 240,
    # so the check is parity with the oracle, not closeness to the original weight
    from oracle import oracle_np as O
    c8, s8 = O.quantize_fp8_e4m3(g["mod_w"])
    assert np.array_equal(to_np(f8.weight_fp8), c8) and np.array_equal(to_np(f8.weight_scales), s8)
    assert np.array_equal(to_np(f8.dequantize()), O.dequantize_fp8_e4m3(c8, s8, "float16"))
