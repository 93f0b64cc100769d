"""GPU parity: model-level helpers (BitsAndBytesConfig, quantize_model, replace_linear_with_*,
get_memory_footprint) and checkpoints written by the reference itself, against the reference's
stored outputs (tests/golden/golden_modules.npz, ref_*.pt)."""
import os

import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from gpu_util import rel_err, to_np

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


class Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj = torch.nn.Linear(64, 64)
        self.mlp = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 64))
        self.norm = torch.nn.LayerNorm(64)

    def forward(self, h):
        return self.norm(h + self.mlp(self.q_proj(h)))


class Toy(torch.nn.Module):
    """The model make_golden.py quantises with the reference."""

    def __init__(self):
        super().__init__()
        self.embed = torch.nn.Embedding(30, 64)
        self.layers = torch.nn.ModuleList([Block(), Block()])
        self.lm_head = torch.nn.Linear(64, 30, bias=False)

    def forward(self, ids):
        h = self.embed(ids)
        for layer in self.layers:
            h = layer(h)
        return self.lm_head(h)


def toy(g):
    m = Toy().half()
    m.load_state_dict({k: torch.from_numpy(g["toy_sd_" + k]) for k in g["toy_keys"]})
    return m


def test_quantize_model_matches_reference(golden):
    g = golden("modules")
    ids = torch.from_numpy(g["toy_ids"]).cuda()
    # the model starts on the CPU: layers move to the GPU one by one as they are converted
    m4 = bnb.quantize_model(toy(g), bnb.BitsAndBytesConfig(load_in_4bit=True, bnb_4bit_quant_type="fp4"),
                            modules_to_not_convert=["lm_head"])
    types = [f"{n}:{type(m).__name__}" for n, m in m4.named_modules() if "Linear" in type(m).__name__]
    assert types == list(g["toy_types4"])
    assert all(p.device.type == "cuda" for p in m4.parameters()) and all(b.device.type == "cuda" for b in m4.buffers())
    assert rel_err(to_np(m4(ids)), g["toy_y4"]) <= 1e-2
    fp = bnb.get_memory_footprint(m4)
    assert [fp["total_params"], fp["quantized_params"]] == [int(g["toy_fp4"][0]), int(g["toy_fp4"][1])]
    assert fp["fp16_size_gb"] == g["toy_fp4"][2] and fp["actual_size_gb"] == g["toy_fp4"][3]
    m8 = bnb.quantize_model(toy(g).cuda(), load_in_8bit=True)
    assert [f"{n}:{type(m).__name__}" for n, m in m8.named_modules() if "Linear" in type(m).__name__] == list(g["toy_types8"])
    assert rel_err(to_np(m8(ids)), g["toy_y8"]) <= 1e-2
    fp = bnb.get_memory_footprint(m8)
    assert [fp["total_params"], fp["quantized_params"]] == [int(g["toy_fp8"][0]), int(g["toy_fp8"][1])]
    assert fp["actual_size_gb"] == g["toy_fp8"][3] and fp["savings_pct"] > 0


def test_config_matches_reference(golden):
    g = golden("modules")
    cfg = bnb.BitsAndBytesConfig(load_in_4bit=True, bnb_4bit_compute_dtype=torch.bfloat16, llm_int8_skip_modules=["lm_head"])
    assert [f"{k}={v}" for k, v in cfg.to_dict().items()] == list(g["cfg_dict"])
    assert str(bnb.BitsAndBytesConfig.from_dict(cfg.to_dict()).bnb_4bit_compute_dtype) == str(g["cfg_back_dtype"])
    assert [cfg.quantization_method, bnb.BitsAndBytesConfig(load_in_8bit=True).quantization_method,
            bnb.BitsAndBytesConfig().quantization_method] == list(g["cfg_method"])
    assert cfg.is_quantizable and not bnb.BitsAndBytesConfig().is_quantizable
    with pytest.raises(ValueError, match="Cannot load in both 4-bit and 8-bit"):
        bnb.BitsAndBytesConfig(load_in_4bit=True, load_in_8bit=True)
    with pytest.raises(ValueError, match="bnb_4bit_quant_type must be 'nf4' or 'fp4'"):
        bnb.BitsAndBytesConfig(bnb_4bit_quant_type="int4")


def test_reference_checkpoints_load(golden):
    """state_dict() files written by the reference's own modules load into the drop-in modules and give
    the reference's outputs; what the drop-in saves has the same keys."""
    g = golden("modules")
    x = torch.from_numpy(g["ck_x"]).cuda()
    sd = torch.load(os.path.join(GOLDEN, "ref_linear4bit_nf4_dq.pt"), weights_only=False)
    l4 = bnb.Linear4bit(128, 48, device="cuda", quant_type="nf4", compress_statistics=True)
    l4.load_state_dict(sd)
    assert l4.weight_quant_state.state2 is not None and l4.weight.device.type == "cuda"
    assert np.array_equal(to_np(l4.dequantize()), g["ck_l4_deq"])                  # bit-exact dequantised weight
    assert rel_err(to_np(l4(x)), g["ck_l4"]) <= 1e-2
    sd = torch.load(os.path.join(GOLDEN, "ref_linear4bit_nf4_dq.pt"), weights_only=False)
    assert set(l4.state_dict().keys()) == set(sd.keys())
    assert torch.equal(l4.state_dict()["weight"].cpu(), sd["weight"])
    sd = torch.load(os.path.join(GOLDEN, "ref_linear4bit_fp4_bs32.pt"), weights_only=False)
    l4b = bnb.Linear4bit(128, 48, device="cuda")                                   # nf4 / 64: the checkpoint wins
    with pytest.warns(UserWarning):
        l4b.load_state_dict(sd)
    assert (l4b.quant_type, l4b.blocksize) == ("fp4", 32)
    assert rel_err(to_np(l4b(x)), g["ck_l4b"]) <= 1e-2
    l8 = bnb.Linear8bit(128, 48, device="cuda")
    l8.load_state_dict(torch.load(os.path.join(GOLDEN, "ref_linear8bit.pt"), weights_only=False))
    assert rel_err(to_np(l8(x)), g["ck_l8"]) <= 1e-2
    e4 = bnb.Embedding4bit(40, 128, device="cuda")
    e4.load_state_dict(torch.load(os.path.join(GOLDEN, "ref_embedding4bit.pt"), weights_only=False))
    assert np.array_equal(to_np(e4(torch.from_numpy(g["ck_eids"]).cuda())), g["ck_e4"])


def test_quantize_model_on_a_hugging_face_llama(golden):
    """A random-init two-layer LlamaForCausalLM (transformers) quantised by quantize_model gives the logits the
    reference's quantize_model gives for the same weights (4-bit NF4 with lm_head skipped; 8-bit everywhere)."""
    transformers = pytest.importorskip("transformers")
    g = golden("modules")
    if "hf_ids" not in g:
        pytest.skip("fixture was generated without transformers")
    cfg = transformers.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)

    def model():
        m = transformers.LlamaForCausalLM(cfg).half().eval()
        m.load_state_dict({k: torch.from_numpy(g["hf_sd_" + k]) for k in g["hf_keys"]})
        return m
    ids = torch.from_numpy(g["hf_ids"]).cuda()
    with torch.no_grad():
        m4 = bnb.quantize_model(model(), bnb.BitsAndBytesConfig(load_in_4bit=True), modules_to_not_convert=["lm_head"])
        assert sum(isinstance(m, bnb.Linear4bit) for m in m4.modules()) == int(g["hf_n4"])
        assert isinstance(m4.lm_head, torch.nn.Linear)
        assert rel_err(to_np(m4(ids).logits), g["hf_y4"]) <= 1e-2
        m8 = bnb.quantize_model(model(), load_in_8bit=True)
        assert sum(isinstance(m, bnb.Linear8bit) for m in m8.modules()) == int(g["hf_n8"])
        assert rel_err(to_np(m8(ids).logits), g["hf_y8"]) <= 1e-2
