"""B200-native drop-in for the quantize / dequantize / fused dequant-matmul path of
mps-bitsandbytes (``mps_bitsandbytes/__init__.py:51-93``): the same functional names and
``Linear4bit`` / ``Linear8bit`` / ``LinearFP8`` modules, running hand-written sm_100a CUDA
kernels through a C-ABI shared library.  CUDA tensors only; no fallback path exists.

The directory name carries a hyphen; import it as ``mps_bitsandbytes_b200`` (the
repository root holds a small loader module of that name).
"""
__version__ = "0.1.0"

from .functional import (  # noqa: F401
    FP4_CODEBOOK, NF4_CODEBOOK, QuantState, create_fp4_map, create_normal_map, dequant_absmax,
    dequantize_4bit, dequantize_blockwise, dequantize_colrow, dequantize_fp4, dequantize_fp8_e4m3,
    dequantize_nf4, dequantize_rowwise, double_quant, matmul_4bit, matmul_colrow, matmul_fp4,
    matmul_fp8_e4m3, matmul_int8, matmul_nf4, quantize_4bit, quantize_blockwise, quantize_colrow,
    quantize_fp4, quantize_fp8_e4m3, quantize_nf4, quantize_rowwise)
from .nn import (  # noqa: F401
    Embedding4bit, Embedding8bit, EmbeddingFP4, EmbeddingNF4, Linear4bit, Linear8bit, LinearFP8,
    OutlierAwareLinear, Params4bit)
from .integration import (  # noqa: F401
    BitsAndBytesConfig, get_memory_footprint, quantize_model, replace_linear_with_4bit, replace_linear_with_8bit)


def is_available() -> bool:
    """True when a CUDA device is present (the reference's analogue checks for MPS, __init__.py:120-122)."""
    import torch
    return torch.cuda.is_available()


def has_native_kernels() -> bool:
    """True when the compiled CUDA library is present (the only execution path there is)."""
    import os
    from . import _native
    return os.path.exists(_native.LIB_PATH)
