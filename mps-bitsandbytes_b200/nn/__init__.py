"""Quantised linear and embedding layers (drop-in for mps_bitsandbytes.nn on CUDA)."""
from .linear4bit import Linear4bit, Params4bit
from .linear8bit import Linear8bit
from .linear_fp8 import LinearFP8
from .embedding import Embedding4bit, Embedding8bit, EmbeddingFP4, EmbeddingNF4
from .outlier_aware import OutlierAwareLinear

__all__ = ["Linear4bit", "Params4bit", "Linear8bit", "LinearFP8", "OutlierAwareLinear",
           "Embedding4bit", "Embedding8bit", "EmbeddingNF4", "EmbeddingFP4"]
