"""Embedding4bit / Embedding8bit: quantised embedding tables whose look-up gathers and
dequantises in one CUDA kernel.

Drop-in for mps_bitsandbytes/nn/embedding.py:20-332: same constructors, buffer names
(``weight_packed`` [V, D/2] uint8 + ``weight_absmax`` [V, ceil(D/blocksize)] fp32;
``weight_int8`` [V, D] + ``weight_scales`` [V]), ``from_embedding`` and the NF4 / FP4
aliases.  The reference quantises the table one row at a time in Python
(embedding.py:184-195) and, off its Metal kernel, dequantises every unique row in a loop
(:111-131); here the table is quantised by one row-wise kernel call (a row of the 2-D
quantiser is exactly the flat quantisation of that row when D is a multiple of the block
size) and looked up by ``mpsbnb_embedding_4bit`` / ``mpsbnb_embedding_8bit``.
"""
import ctypes as C
from typing import Optional

import torch
from torch import Tensor, nn

from .. import _native as N
from ..functional import quantize_4bit, quantize_rowwise


def _indices(input: Tensor) -> Tensor:
    if input.dtype not in (torch.int32, torch.int64):
        input = input.long()
    return input.contiguous()


class Embedding4bit(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None,
                 quant_type: str = "nf4", blocksize: int = 64, device=None, dtype=torch.float16):
        super().__init__()
        if quant_type not in ("nf4", "fp4"):
            raise ValueError(f"quant_type must be 'nf4' or 'fp4', got {quant_type}")
        if embedding_dim % 2 != 0:
            raise ValueError(f"embedding_dim must be even, got {embedding_dim}")
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.padding_idx = padding_idx
        self.quant_type = quant_type
        self.blocksize = blocksize
        self.dtype = dtype
        num_blocks = (embedding_dim + blocksize - 1) // blocksize
        self.register_buffer("weight_packed", torch.zeros(num_embeddings, embedding_dim // 2, dtype=torch.uint8, device=device))
        self.register_buffer("weight_absmax", torch.ones(num_embeddings, num_blocks, dtype=torch.float32, device=device))

    def forward(self, input: Tensor) -> Tensor:
        """embedding.py:78-139: [*] indices -> [*, embedding_dim] in ``self.dtype``; padding rows are zero."""
        N.require_cuda(input, self.weight_packed)
        idx = _indices(input)
        out = torch.empty(*input.shape, self.embedding_dim, dtype=self.dtype, device=self.weight_packed.device)
        pad = -1 if self.padding_idx is None else int(self.padding_idx)
        packed, absmax = self.weight_packed.contiguous(), self.weight_absmax.contiguous()
        with torch.cuda.device(packed.device):
            N.check(N.lib().mpsbnb_embedding_4bit(
                N.ptr(idx), C.c_int(idx.element_size()), N.i64(idx.numel()), N.ptr(packed), N.i64(packed.shape[1]),
                N.ptr(absmax), N.i64(self.num_embeddings), N.i64(self.embedding_dim), C.c_int(self.blocksize),
                C.c_int(N.qt(self.quant_type)), N.i64(pad), N.ptr(out), N.dt(self.dtype), N.stream()), "embedding_4bit")
        return out

    @classmethod
    def from_embedding(cls, embedding: nn.Embedding, quant_type: str = "nf4", blocksize: int = 64,
                       device=None) -> "Embedding4bit":
        """embedding.py:141-197.  An odd embedding_dim is zero-padded by one column, as there."""
        if device is None:
            device = embedding.weight.device
        dtype = embedding.weight.dtype
        if dtype not in (torch.float16, torch.bfloat16):
            dtype = torch.float16
        dim = embedding.embedding_dim
        weight = embedding.weight.data
        if dim % 2 != 0:
            dim += 1
            weight = torch.nn.functional.pad(weight, (0, 1))
        layer = cls(embedding.num_embeddings, dim, padding_idx=embedding.padding_idx, quant_type=quant_type,
                    blocksize=blocksize, device=device, dtype=dtype)
        packed, state = quantize_4bit(weight.to(device), blocksize=blocksize, quant_type=quant_type)
        rows = embedding.num_embeddings
        # the row-wise quantiser pads every row to a whole number of blocks; the table keeps the D/2 bytes
        # that hold real codes (the reference's per-row copy only fits when D % blocksize == 0)
        layer.weight_packed.copy_(packed.view(rows, -1)[:, :dim // 2])
        layer.weight_absmax.copy_(state.absmax.view(rows, -1))
        return layer

    def extra_repr(self) -> str:
        return (f"{self.num_embeddings}, {self.embedding_dim}, padding_idx={self.padding_idx}, "
                f"quant_type={self.quant_type}, blocksize={self.blocksize}")


class Embedding8bit(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None,
                 device=None, dtype=torch.float16):
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.padding_idx = padding_idx
        self.dtype = dtype
        self.register_buffer("weight_int8", torch.zeros(num_embeddings, embedding_dim, dtype=torch.int8, device=device))
        self.register_buffer("weight_scales", torch.ones(num_embeddings, dtype=torch.float32, device=device))

    def forward(self, input: Tensor) -> Tensor:
        """embedding.py:244-275: q.to(dtype) * (scale / 127).to(dtype), padding rows zero."""
        N.require_cuda(input, self.weight_int8)
        idx = _indices(input)
        out = torch.empty(*input.shape, self.embedding_dim, dtype=self.dtype, device=self.weight_int8.device)
        pad = -1 if self.padding_idx is None else int(self.padding_idx)
        q, s = self.weight_int8.contiguous(), self.weight_scales.contiguous()
        with torch.cuda.device(q.device):
            N.check(N.lib().mpsbnb_embedding_8bit(
                N.ptr(idx), C.c_int(idx.element_size()), N.i64(idx.numel()), N.ptr(q), N.ptr(s),
                N.i64(self.num_embeddings), N.i64(self.embedding_dim), N.i64(pad), N.ptr(out), N.dt(self.dtype),
                N.stream()), "embedding_8bit")
        return out

    @classmethod
    def from_embedding(cls, embedding: nn.Embedding, device=None) -> "Embedding8bit":
        """embedding.py:277-304."""
        if device is None:
            device = embedding.weight.device
        dtype = embedding.weight.dtype
        if dtype not in (torch.float16, torch.bfloat16):
            dtype = torch.float16
        layer = cls(embedding.num_embeddings, embedding.embedding_dim, padding_idx=embedding.padding_idx,
                    device=device, dtype=dtype)
        q, s = quantize_rowwise(embedding.weight.data.to(device))
        layer.weight_int8.copy_(q)
        layer.weight_scales.copy_(s)
        return layer

    def extra_repr(self) -> str:
        return f"{self.num_embeddings}, {self.embedding_dim}, padding_idx={self.padding_idx}"


class EmbeddingNF4(Embedding4bit):
    """Embedding4bit with quant_type='nf4' (embedding.py:311-320)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, **kwargs):
        kwargs["quant_type"] = "nf4"
        super().__init__(num_embeddings, embedding_dim, **kwargs)

    @classmethod
    def from_embedding(cls, embedding, blocksize: int = 64, device=None) -> "EmbeddingNF4":
        return super().from_embedding(embedding, quant_type="nf4", blocksize=blocksize, device=device)


class EmbeddingFP4(Embedding4bit):
    """Embedding4bit with quant_type='fp4' (embedding.py:323-332)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, **kwargs):
        kwargs["quant_type"] = "fp4"
        super().__init__(num_embeddings, embedding_dim, **kwargs)

    @classmethod
    def from_embedding(cls, embedding, blocksize: int = 64, device=None) -> "EmbeddingFP4":
        return super().from_embedding(embedding, quant_type="fp4", blocksize=blocksize, device=device)
