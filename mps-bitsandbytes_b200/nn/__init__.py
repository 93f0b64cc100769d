"""Quantised linear layers (drop-in for mps_bitsandbytes.nn on CUDA)."""
from .linear4bit import Linear4bit, Params4bit
from .linear8bit import Linear8bit
from .linear_fp8 import LinearFP8

__all__ = ["Linear4bit", "Params4bit", "Linear8bit", "LinearFP8"]
