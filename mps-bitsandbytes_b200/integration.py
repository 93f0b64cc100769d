"""Model-level helpers: a BitsAndBytesConfig-compatible configuration and the functions that
swap every ``nn.Linear`` of a model for ``Linear4bit`` / ``Linear8bit``.

Drop-in for mps_bitsandbytes/integration.py:16-287 (``BitsAndBytesConfig``,
``replace_linear_with_4bit`` / ``_8bit``, ``quantize_model``, ``get_memory_footprint``) with
``device='cuda'`` as the default target.  One difference follows from there being no CPU
quantiser here: a layer whose weight lives on the CPU is moved to the target device as it
is converted, one layer at a time, so the 16-bit model never has to fit on the GPU as a
whole (the reference quantises on whatever device the model is on and moves it afterwards,
integration.py:241-249).
"""
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch
from torch import nn

from .nn import Linear4bit, Linear8bit


@dataclass
class BitsAndBytesConfig:
    """integration.py:16-105: same fields, validation messages and dictionary form."""
    load_in_8bit: bool = False
    load_in_4bit: bool = False
    llm_int8_threshold: float = 6.0
    llm_int8_skip_modules: Optional[list] = None
    llm_int8_enable_fp32_cpu_offload: bool = False
    llm_int8_has_fp16_weight: bool = False
    bnb_4bit_compute_dtype: torch.dtype = torch.float16
    bnb_4bit_quant_type: str = "nf4"
    bnb_4bit_use_double_quant: bool = False
    bnb_4bit_quant_storage: torch.dtype = torch.uint8

    def __post_init__(self):
        if self.load_in_4bit and self.load_in_8bit:
            raise ValueError("Cannot load in both 4-bit and 8-bit")
        if self.bnb_4bit_quant_type not in ("nf4", "fp4"):
            raise ValueError(f"bnb_4bit_quant_type must be 'nf4' or 'fp4', got {self.bnb_4bit_quant_type}")
        if self.llm_int8_skip_modules is None:
            self.llm_int8_skip_modules = []

    def to_dict(self) -> Dict[str, Any]:
        return {
            "load_in_8bit": self.load_in_8bit,
            "load_in_4bit": self.load_in_4bit,
            "llm_int8_threshold": self.llm_int8_threshold,
            "llm_int8_skip_modules": self.llm_int8_skip_modules,
            "bnb_4bit_compute_dtype": str(self.bnb_4bit_compute_dtype),
            "bnb_4bit_quant_type": self.bnb_4bit_quant_type,
            "bnb_4bit_use_double_quant": self.bnb_4bit_use_double_quant,
        }

    @classmethod
    def from_dict(cls, config_dict: Dict[str, Any]) -> "BitsAndBytesConfig":
        """integration.py:77-91.  The string is matched as the reference matches it ('float16' first, which
        also matches 'torch.bfloat16'), so a round trip through to_dict() gives what the reference gives."""
        config_dict = dict(config_dict)
        dtype_str = config_dict.get("bnb_4bit_compute_dtype")
        if isinstance(dtype_str, str):
            if "float16" in dtype_str:
                config_dict["bnb_4bit_compute_dtype"] = torch.float16
            elif "bfloat16" in dtype_str:
                config_dict["bnb_4bit_compute_dtype"] = torch.bfloat16
            else:
                config_dict["bnb_4bit_compute_dtype"] = torch.float16
        return cls(**{k: v for k, v in config_dict.items() if k in cls.__dataclass_fields__})

    @property
    def is_quantizable(self) -> bool:
        return self.load_in_4bit or self.load_in_8bit

    @property
    def quantization_method(self) -> str:
        if self.load_in_4bit:
            return "bitsandbytes_4bit"
        if self.load_in_8bit:
            return "bitsandbytes_8bit"
        return "none"


def _target_device(module: nn.Linear, device):
    """Device the converted layer lives on: the request, else the layer's own when that is a CUDA device."""
    if device is not None:
        return torch.device(device)
    if module.weight.device.type == "cuda":
        return module.weight.device
    return torch.device("cuda")


def _replace(model: nn.Module, convert, modules_to_not_convert, current_key_name) -> nn.Module:
    for name, module in model.named_children():
        full_name = f"{current_key_name}.{name}" if current_key_name else name
        if isinstance(module, nn.Linear):
            if any(skip in full_name for skip in modules_to_not_convert):
                continue
            setattr(model, name, convert(module))
        else:
            _replace(module, convert, modules_to_not_convert, full_name)
    return model


def replace_linear_with_4bit(model: nn.Module, quantization_config: BitsAndBytesConfig,
                             modules_to_not_convert: Optional[list] = None,
                             current_key_name: Optional[str] = None, device=None) -> nn.Module:
    """integration.py:108-154: every nn.Linear whose dotted name contains none of the skip strings becomes a
    Linear4bit with the config's compute dtype and quant type (double quantisation is not applied, as there)."""
    skip = modules_to_not_convert if modules_to_not_convert is not None else []

    def convert(module):
        return Linear4bit.from_linear(module, device=_target_device(module, device),
                                      compute_dtype=quantization_config.bnb_4bit_compute_dtype,
                                      quant_type=quantization_config.bnb_4bit_quant_type)
    return _replace(model, convert, skip, current_key_name)


def replace_linear_with_8bit(model: nn.Module, quantization_config: BitsAndBytesConfig,
                             modules_to_not_convert: Optional[list] = None,
                             current_key_name: Optional[str] = None, device=None) -> nn.Module:
    """integration.py:157-196; the skip list defaults to the config's llm_int8_skip_modules."""
    skip = modules_to_not_convert if modules_to_not_convert is not None else (quantization_config.llm_int8_skip_modules or [])

    def convert(module):
        return Linear8bit.from_linear(module, device=_target_device(module, device))
    return _replace(model, convert, skip, current_key_name)


def quantize_model(model: nn.Module, quantization_config: Optional[BitsAndBytesConfig] = None,
                   load_in_4bit: bool = False, load_in_8bit: bool = False, device: str = "cuda",
                   compute_dtype: torch.dtype = torch.float16,
                   modules_to_not_convert: Optional[list] = None) -> nn.Module:
    """integration.py:199-251: quantise the linears, then move what is left of the model to ``device``."""
    if quantization_config is None:
        quantization_config = BitsAndBytesConfig(load_in_4bit=load_in_4bit, load_in_8bit=load_in_8bit,
                                                 bnb_4bit_compute_dtype=compute_dtype)
    if quantization_config.load_in_4bit:
        model = replace_linear_with_4bit(model, quantization_config, modules_to_not_convert, device=device)
    elif quantization_config.load_in_8bit:
        model = replace_linear_with_8bit(model, quantization_config, modules_to_not_convert, device=device)
    return model.to(device)


def get_memory_footprint(model: nn.Module) -> Dict[str, Any]:
    """integration.py:254-287: element and byte counts over parameters and buffers.  As in the reference,
    ``quantized_params`` counts buffers named ``weight_packed`` or ``weight_int8`` only (Linear4bit stores its
    packed bytes in ``weight``, so 4-bit linears do not show up there)."""
    total_bytes = 0
    total_params = 0
    quantized_params = 0
    for _, param in model.named_parameters():
        total_params += param.numel()
        total_bytes += param.numel() * param.element_size()
    for name, buf in model.named_buffers():
        total_params += buf.numel()
        total_bytes += buf.numel() * buf.element_size()
        if "weight_packed" in name or "weight_int8" in name:
            quantized_params += buf.numel()
    fp16_size = total_params * 2 / 1e9
    actual_size = total_bytes / 1e9
    return {
        "total_params": total_params,
        "quantized_params": quantized_params,
        "fp16_size_gb": fp16_size,
        "actual_size_gb": actual_size,
        "savings_gb": fp16_size - actual_size,
        "savings_pct": (1 - actual_size / fp16_size) * 100 if fp16_size > 0 else 0,
    }
