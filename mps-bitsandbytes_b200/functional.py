"""Functional API: same names, argument order, return values and error messages as
``mps_bitsandbytes/functional.py`` (reference v0.7.0), executing on a CUDA device through
the C-ABI library.  Tensors must live on ``cuda``; there is no CPU or PyTorch fallback.

Every function cites the reference lines it reproduces.  Quantisers and dequantisers are
bit-exact with the reference's CPU path; matmuls agree within 1e-2 relative error
(fp16/bf16 operands, fp32 accumulation).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _native as N

# mps_bitsandbytes/functional.py:21-26
NF4_CODEBOOK = torch.tensor([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0], dtype=torch.float32)

# mps_bitsandbytes/functional.py:29-32
FP4_CODEBOOK = torch.tensor([
    0.0, 0.0625, 0.125, 0.25, 0.375, 0.5, 0.75, 1.0,
    -0.0, -0.0625, -0.125, -0.25, -0.375, -0.5, -0.75, -1.0], dtype=torch.float32)

_FLOAT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


def create_normal_map(offset=0.9677083, use_extra_value=True):
    """NF4 codebook (mps_bitsandbytes/functional.py:35-37)."""
    return NF4_CODEBOOK.clone()


def create_fp4_map(signed=True):
    """FP4 codebook (mps_bitsandbytes/functional.py:40-42)."""
    return FP4_CODEBOOK.clone()


def _check_device(tensor: Tensor, operation: str = "operation"):
    """The reference accepts 'mps'/'cpu' (functional.py:76-83); this build accepts 'cuda' only."""
    if tensor.device.type != "cuda":
        raise ValueError(
            f"mps-bitsandbytes_b200 {operation} requires tensor on a 'cuda' device, "
            f"got '{tensor.device.type}'. Move tensor with .to('cuda')")


def _need(name: str, t: Optional[Tensor], count: int, what: str):
    """Raises the shape error the reference raises (there by broadcasting / indexing) when a caller-supplied
    tensor holds fewer elements than the kernel is going to read: the kernels take raw pointers."""
    if t is not None and t.numel() < count:
        raise ValueError(f"{name} has {t.numel()} elements, {what} needs {count}")


def _as_float(t: Tensor) -> Tensor:
    """Kernels take fp16 / bf16 / fp32; anything else is widened to fp32 as the reference's .float()."""
    return t if t.dtype in _FLOAT_DTYPES else t.float()


@dataclass
class QuantState:
    """Quantisation state, field-compatible with mps_bitsandbytes/functional.py:90-156."""
    absmax: Tensor
    shape: torch.Size
    code: Optional[Tensor] = None
    blocksize: int = 64
    quant_type: str = "nf4"
    dtype: torch.dtype = torch.float16
    offset: Optional[Tensor] = None
    state2: Optional["QuantState"] = None

    def __post_init__(self):
        if self.code is None:
            self.code = NF4_CODEBOOK if self.quant_type == "nf4" else FP4_CODEBOOK

    def to(self, device):
        self.absmax = self.absmax.to(device)
        if self.code is not None:
            self.code = self.code.to(device)
        if self.offset is not None:
            self.offset = self.offset.to(device)
        if self.state2 is not None:
            self.state2 = self.state2.to(device)
        return self

    def as_dict(self, packed=False):
        return {
            "absmax": self.absmax,
            "shape": self.shape,
            "blocksize": self.blocksize,
            "quant_type": self.quant_type,
            "dtype": self.dtype,
            "state2": self.state2.as_dict() if self.state2 else None,
        }

    @classmethod
    def from_dict(cls, state_dict, device="cpu"):
        state2 = None
        if state_dict.get("state2") is not None:
            state2 = cls.from_dict(state_dict["state2"], device)
        return cls(
            absmax=state_dict["absmax"].to(device),
            shape=state_dict["shape"],
            blocksize=state_dict.get("blocksize", 64),
            quant_type=state_dict.get("quant_type", "nf4"),
            dtype=state_dict.get("dtype", torch.float16),
            state2=state2,
        )


def _padded(k: int, blocksize: int) -> int:
    kp = ((k + blocksize - 1) // blocksize) * blocksize
    if kp % 2 != 0:
        kp += blocksize
    return kp


# =============================================================================
# 4-bit
# =============================================================================

def quantize_4bit(
    A: Tensor,
    absmax: Optional[Tensor] = None,
    out: Optional[Tensor] = None,
    blocksize: int = 64,
    compress_statistics: bool = False,
    quant_type: str = "nf4",
    quant_storage: torch.dtype = torch.uint8,
) -> Tuple[Tensor, QuantState]:
    """Blockwise NF4/FP4 quantisation (mps_bitsandbytes/functional.py:163-303).

    2-D tensors are quantised row-wise (:216-255), anything else flat (:257-286).  Returns
    the flattened packed tensor and a QuantState; with ``compress_statistics`` absmax is
    itself int8-quantised in blocks of 256 (:288-292).
    """
    if quant_type not in ("nf4", "fp4"):
        raise ValueError(f"quant_type must be 'nf4' or 'fp4', got {quant_type}")
    _check_device(A, "quantize_4bit")
    if blocksize <= 0:
        raise ValueError(f"blocksize must be positive, got {blocksize}")
    if blocksize > 65536:
        raise ValueError(f"blocksize too large ({blocksize}), max is 65536")
    if (blocksize & (blocksize - 1)) != 0:
        raise ValueError(f"blocksize must be a power of 2, got {blocksize}")
    max_safe_numel = 2**31 - 1
    if A.numel() > max_safe_numel:
        raise ValueError(f"Tensor too large ({A.numel()} elements), max is {max_safe_numel}")

    orig_shape, orig_dtype = A.shape, A.dtype
    src = _as_float(A).contiguous()
    rows, cols = (src.shape if src.dim() == 2 else (1, src.numel()))
    kp = _padded(cols, blocksize)
    nb = kp // blocksize
    packed = torch.empty(rows * (kp // 2), dtype=torch.uint8, device=A.device)
    am_in = None
    if absmax is not None:
        am_in = absmax.to(device=A.device, dtype=torch.float32).contiguous()
        if am_in.numel() != rows * nb:
            raise ValueError(f"absmax has {am_in.numel()} elements, expected {rows * nb}")
        am = am_in.flatten()
    else:
        am = torch.empty(rows * nb, dtype=torch.float32, device=A.device)
    with torch.cuda.device(A.device):
        N.check(N.lib().mpsbnb_quantize_4bit(
            N.ptr(src), N.dt(src.dtype), N.i64(rows), N.i64(cols), C.c_int(blocksize), C.c_int(N.qt(quant_type)),
            N.ptr(am_in), N.ptr(packed), N.ptr(None if am_in is not None else am), N.stream()), "quantize_4bit")
    if quant_storage != torch.uint8:
        packed = packed.to(quant_storage)
    if out is not None:
        out[:] = packed.view(out.shape)
        packed = out.flatten()

    state2 = None
    if compress_statistics:
        am, state2 = quantize_blockwise(am, blocksize=256)
    return packed, QuantState(absmax=am, shape=orig_shape, blocksize=blocksize, quant_type=quant_type,
                              dtype=orig_dtype, state2=state2)


def _expand_absmax(absmax: Tensor, state2: Optional[QuantState]):
    """Returns (absmax tensor, absmax2 or None) in the form the kernels take: fp32 absmax,
    or int8 absmax plus fp32 second-level maxima over blocks of 256 (functional.py:335-337)."""
    if state2 is None:
        return absmax.to(torch.float32).contiguous(), None
    if state2.blocksize == 256 and state2.state2 is None and absmax.dtype == torch.int8:
        return absmax.contiguous(), state2.absmax.to(torch.float32).contiguous()
    return dequantize_blockwise(absmax, state2).to(torch.float32).contiguous(), None


def dequantize_4bit(
    A: Tensor,
    quant_state: Optional[QuantState] = None,
    absmax: Optional[Tensor] = None,
    out: Optional[Tensor] = None,
    blocksize: int = 64,
    quant_type: str = "nf4",
) -> Tensor:
    """Inverse of quantize_4bit (mps_bitsandbytes/functional.py:306-416)."""
    _check_device(A, "dequantize_4bit")
    state2 = None
    if quant_state is not None:
        absmax = quant_state.absmax
        blocksize = quant_state.blocksize
        quant_type = quant_state.quant_type
        shape = quant_state.shape
        dtype = quant_state.dtype
        state2 = quant_state.state2
    else:
        if absmax is None:
            raise ValueError("Either quant_state or absmax must be provided")
        shape = None
        dtype = torch.float16
    if quant_type not in ("nf4", "fp4"):
        raise ValueError(f"quant_type must be 'nf4' or 'fp4', got {quant_type}")
    out_dtype = dtype if dtype in _FLOAT_DTYPES else torch.float32

    if shape is not None and len(shape) == 2:
        rows, cols = int(shape[0]), int(shape[1])
        result_shape = (rows, cols)
    elif shape is not None:
        rows, cols = 1, int(torch.Size(shape).numel())
        result_shape = tuple(shape)
    else:
        rows, cols = 1, absmax.numel() * blocksize                      # :399-412
        result_shape = (cols,)
    kp = _padded(cols, blocksize)
    am, am2 = _expand_absmax(absmax.to(A.device), state2)
    if am.numel() < rows * (kp // blocksize) or A.numel() < rows * (kp // 2):
        raise ValueError("packed tensor / absmax too small for the given shape")
    res = torch.empty(result_shape, dtype=out_dtype, device=A.device)
    packed = A.contiguous()
    if packed.dtype != torch.uint8:
        packed = packed.to(torch.uint8)
    with torch.cuda.device(A.device):
        N.check(N.lib().mpsbnb_dequantize_4bit(
            N.ptr(packed), N.ptr(am), N.ptr(am2), N.i64(rows), N.i64(cols), C.c_int(blocksize),
            C.c_int(N.qt(quant_type)), N.ptr(res), N.dt(out_dtype), N.stream()), "dequantize_4bit")
    if out_dtype != dtype:
        res = res.to(dtype)
    if out is not None:
        out[:] = res.flatten()[:out.numel()].view(out.shape)
        return out
    return res


def quantize_nf4(A, absmax=None, out=None, blocksize=64, compress_statistics=False,
                 quant_storage=torch.uint8):
    """mps_bitsandbytes/functional.py:419-428."""
    return quantize_4bit(A, absmax, out, blocksize, compress_statistics, "nf4", quant_storage)


def dequantize_nf4(A, quant_state=None, absmax=None, out=None, blocksize=64):
    """mps_bitsandbytes/functional.py:431-439."""
    return dequantize_4bit(A, quant_state, absmax, out, blocksize, "nf4")


def quantize_fp4(A, absmax=None, out=None, blocksize=64, compress_statistics=False,
                 quant_storage=torch.uint8):
    """mps_bitsandbytes/functional.py:442-451."""
    return quantize_4bit(A, absmax, out, blocksize, compress_statistics, "fp4", quant_storage)


def dequantize_fp4(A, quant_state=None, absmax=None, out=None, blocksize=64):
    """mps_bitsandbytes/functional.py:454-462."""
    return dequantize_4bit(A, quant_state, absmax, out, blocksize, "fp4")


# =============================================================================
# Blockwise int8
# =============================================================================

def quantize_blockwise(
    A: Tensor,
    code: Optional[Tensor] = None,
    absmax: Optional[Tensor] = None,
    out: Optional[Tensor] = None,
    blocksize: int = 4096,
    nested: bool = False,
) -> Tuple[Tensor, QuantState]:
    """Flat blockwise int8 quantisation (mps_bitsandbytes/functional.py:469-539)."""
    _check_device(A, "quantize_blockwise")
    if blocksize <= 0:
        raise ValueError(f"blocksize must be positive, got {blocksize}")
    if blocksize > 65536:
        raise ValueError(f"blocksize too large ({blocksize}), max is 65536")
    orig_shape, orig_dtype = A.shape, A.dtype
    src = _as_float(A).contiguous().flatten()
    n = src.numel()
    nblk = (n + blocksize - 1) // blocksize
    q = torch.empty(n, dtype=torch.int8, device=A.device)
    am_in = None
    if absmax is not None:
        am_in = absmax.to(device=A.device, dtype=torch.float32).contiguous().flatten()
        _need("absmax", am_in, nblk, "quantize_blockwise")
        am = am_in
    else:
        am = torch.empty(nblk, dtype=torch.float32, device=A.device)
    with torch.cuda.device(A.device):
        N.check(N.lib().mpsbnb_quantize_blockwise(
            N.ptr(src), N.dt(src.dtype), N.i64(n), C.c_int(blocksize), N.ptr(am_in), N.ptr(q),
            N.ptr(None if am_in is not None else am), N.stream()), "quantize_blockwise")
    if out is not None:
        out.view(-1)[:n] = q
    q = q.view(orig_shape)
    state2 = None
    if nested:
        am, state2 = quantize_blockwise(am, blocksize=256)
    return q, QuantState(absmax=am, shape=orig_shape, blocksize=blocksize, quant_type="int8",
                         dtype=orig_dtype, state2=state2)


def dequantize_blockwise(
    A: Tensor,
    quant_state: Optional[QuantState] = None,
    absmax: Optional[Tensor] = None,
    code: Optional[Tensor] = None,
    out: Optional[Tensor] = None,
    blocksize: int = 4096,
    nested: bool = False,
) -> Tensor:
    """mps_bitsandbytes/functional.py:542-600."""
    _check_device(A, "dequantize_blockwise")
    if quant_state is not None:
        absmax = quant_state.absmax
        blocksize = quant_state.blocksize
        shape = quant_state.shape
        dtype = quant_state.dtype
        if quant_state.state2 is not None:
            absmax = dequantize_blockwise(absmax, quant_state.state2)
    else:
        if absmax is None:
            raise ValueError("Either quant_state or absmax must be provided")
        shape = A.shape
        dtype = torch.float16
    out_dtype = dtype if dtype in _FLOAT_DTYPES else torch.float32
    q = A.contiguous().flatten()
    if q.dtype != torch.int8:
        q = q.to(torch.int8)
    n = q.numel()
    am = absmax.to(device=A.device, dtype=torch.float32).contiguous().flatten()
    if am.numel() * blocksize < n:
        raise ValueError("absmax too small for the tensor")
    res = torch.empty(n, dtype=out_dtype, device=A.device)
    with torch.cuda.device(A.device):
        N.check(N.lib().mpsbnb_dequantize_blockwise(
            N.ptr(q), N.ptr(am), N.i64(n), C.c_int(blocksize), N.ptr(res), N.dt(out_dtype), N.stream()),
            "dequantize_blockwise")
    res = res.view(shape)
    if out_dtype != dtype:
        res = res.to(dtype)
    if out is not None:
        out[:] = res
        return out
    return res


# =============================================================================
# Row-wise int8
# =============================================================================

def quantize_rowwise(tensor: Tensor) -> Tuple[Tensor, Tensor]:
    """Per-row absmax int8 (mps_bitsandbytes/functional.py:607-625); scales are the row maxima."""
    _check_device(tensor, "quantize_rowwise")
    src = _as_float(tensor).contiguous()
    cols = src.shape[-1]
    rows = src.numel() // cols if cols else 0
    q = torch.empty(src.shape, dtype=torch.int8, device=tensor.device)
    scales = torch.empty(rows, dtype=torch.float32, device=tensor.device)
    with torch.cuda.device(tensor.device):
        N.check(N.lib().mpsbnb_quantize_rowwise(N.ptr(src), N.dt(src.dtype), N.i64(rows), N.i64(cols), N.ptr(q),
                                                N.ptr(scales), N.stream()), "quantize_rowwise")
    return q, scales


def dequantize_rowwise(quantized: Tensor, scales: Tensor, dtype: torch.dtype = torch.float16) -> Tensor:
    """mps_bitsandbytes/functional.py:628-636."""
    _check_device(quantized, "dequantize_rowwise")
    q = quantized.contiguous()
    cols = q.shape[-1]
    rows = q.numel() // cols if cols else 0
    s = scales.to(device=q.device, dtype=torch.float32).contiguous().view(-1)
    _need("scales", s, rows, "dequantize_rowwise")
    out = torch.empty(q.shape, dtype=dtype, device=q.device)
    with torch.cuda.device(q.device):
        N.check(N.lib().mpsbnb_dequantize_rowwise(N.ptr(q), N.ptr(s), N.i64(rows), N.i64(cols), N.ptr(out),
                                                  N.dt(dtype), N.stream()), "dequantize_rowwise")
    return out


# =============================================================================
# FP8 E4M3
# =============================================================================

def quantize_fp8_e4m3(tensor: Tensor) -> Tuple[Tensor, Tensor]:
    """Row-scaled FP8 E4M3 with the reference's Python encoder semantics
    (mps_bitsandbytes/functional.py:643-663, 1086-1163)."""
    if tensor.dim() != 2:
        raise ValueError("Input must be 2D")
    _check_device(tensor, "quantize_fp8_e4m3")
    src = _as_float(tensor).contiguous()
    rows, cols = src.shape
    codes = torch.empty(rows, cols, dtype=torch.uint8, device=tensor.device)
    scales = torch.empty(rows, dtype=torch.float32, device=tensor.device)
    with torch.cuda.device(tensor.device):
        N.check(N.lib().mpsbnb_quantize_fp8_e4m3(N.ptr(src), N.dt(src.dtype), N.i64(rows), N.i64(cols),
                                                 N.ptr(codes), N.ptr(scales), N.stream()), "quantize_fp8_e4m3")
    return codes, scales


def dequantize_fp8_e4m3(quantized: Tensor, scales: Tensor, dtype: torch.dtype = torch.float16) -> Tensor:
    """mps_bitsandbytes/functional.py:666-673, 1166-1216."""
    _check_device(quantized, "dequantize_fp8_e4m3")
    q = quantized.contiguous()
    rows, cols = q.shape
    s = scales.to(device=q.device, dtype=torch.float32).contiguous()
    _need("scales", s, rows, "dequantize_fp8_e4m3")
    out = torch.empty(rows, cols, dtype=dtype, device=q.device)
    with torch.cuda.device(q.device):
        N.check(N.lib().mpsbnb_dequantize_fp8_e4m3(N.ptr(q), N.ptr(s), N.i64(rows), N.i64(cols), N.ptr(out),
                                                   N.dt(dtype), N.stream()), "dequantize_fp8_e4m3")
    return out


# =============================================================================
# Matrix multiplication with quantised weights
# =============================================================================

def _mma_dtype(*dtypes) -> torch.dtype:
    """Operand type of the tensor-core paths: bf16 if any participant is bf16, else fp16."""
    return torch.bfloat16 if torch.bfloat16 in dtypes else torch.float16


def _workspace(nbytes: int, device) -> Tensor:
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)


def matmul_4bit(
    A: Tensor,
    B: Tensor,
    quant_state: QuantState,
    bias: Optional[Tensor] = None,
    compute_dtype: Optional[torch.dtype] = None,
) -> Tensor:
    """y = A @ dequantize(B)^T (+ bias), fused (mps_bitsandbytes/functional.py:680-773).

    Up to 32 rows of A take the weight-streaming GEMV; more rows dequantise into a
    workspace and run the tcgen05 GEMM.  Output dtype is ``compute_dtype`` (default A.dtype).
    """
    if compute_dtype is None:
        compute_dtype = A.dtype
    _check_device(A, "matmul_4bit")
    _check_device(B, "matmul_4bit")
    if len(quant_state.shape) != 2:
        raise ValueError("matmul_4bit needs a 2-D weight (quant_state.shape = [out_features, in_features])")
    n, k = int(quant_state.shape[0]), int(quant_state.shape[1])
    if A.shape[-1] != k:
        raise RuntimeError(f"input has {A.shape[-1]} features, weight expects {k}")
    orig_shape = A.shape
    op = _mma_dtype(quant_state.dtype, A.dtype)
    x = A.reshape(-1, k).to(op).contiguous()
    m = x.shape[0]
    b = None if bias is None else bias.to(device=A.device, dtype=op).contiguous()
    y_dtype = compute_dtype if compute_dtype in _FLOAT_DTYPES else torch.float32
    y = torch.empty(m, n, dtype=y_dtype, device=A.device)
    am, am2 = _expand_absmax(quant_state.absmax.to(A.device), quant_state.state2)
    packed = B.contiguous()
    if packed.dtype != torch.uint8:
        packed = packed.to(torch.uint8)       # quant_storage other than uint8 holds the byte VALUES (functional.py:299-300)
    bs, qt = quant_state.blocksize, N.qt(quant_state.quant_type)
    kp = _padded(k, bs)
    _need("packed weight", packed, n * (kp // 2), "matmul_4bit")
    _need("absmax", am, n * (kp // bs), "matmul_4bit")
    if am2 is not None:
        _need("second-level absmax", am2, (n * (kp // bs) + 255) // 256, "matmul_4bit")
    _need("bias", b, n, "matmul_4bit")
    lib = N.lib()
    with torch.cuda.device(A.device):
        if bs == 64 and m <= lib.mpsbnb_gemv_4bit_max_m():
            N.check(lib.mpsbnb_gemv_4bit(N.ptr(x), N.dt(op), N.i64(m), N.ptr(packed), N.ptr(am), N.ptr(am2),
                                         N.i64(n), N.i64(k), C.c_int(bs), C.c_int(qt), N.ptr(b), N.ptr(y),
                                         N.dt(y_dtype), N.stream()), "gemv_4bit")
        else:
            nbytes = lib.mpsbnb_gemm_4bit_workspace_bytes(N.i64(m), N.i64(n), N.i64(k), C.c_int(bs))
            ws = _workspace(nbytes, A.device)
            N.check(lib.mpsbnb_gemm_4bit(N.ptr(x), N.dt(op), N.i64(m), N.ptr(packed), N.ptr(am), N.ptr(am2),
                                         N.i64(n), N.i64(k), C.c_int(bs), C.c_int(qt), N.ptr(b), N.ptr(y),
                                         N.dt(y_dtype), N.ptr(ws), C.c_size_t(ws.numel()), N.stream()), "gemm_4bit")
    if y_dtype != compute_dtype:
        y = y.to(compute_dtype)
    if len(orig_shape) != 2:
        y = y.reshape(*orig_shape[:-1], n)
    return y


def matmul_nf4(input: Tensor, weight_packed: Tensor, weight_state: QuantState,
               bias: Optional[Tensor] = None) -> Tensor:
    """mps_bitsandbytes/functional.py:776-779."""
    return matmul_4bit(input, weight_packed, weight_state, bias)


def matmul_fp4(input: Tensor, weight_packed: Tensor, weight_state: QuantState,
               bias: Optional[Tensor] = None) -> Tensor:
    """mps_bitsandbytes/functional.py:782-785."""
    return matmul_4bit(input, weight_packed, weight_state, bias)


def matmul_int8(A: Tensor, B: Tensor, A_scales: Tensor, B_scales: Tensor,
                dtype: torch.dtype = torch.float16) -> Tensor:
    """INT8 x INT8 matmul with row scales on A [M,K] and column scales on B [K,N]
    (mps_bitsandbytes/functional.py:788-793)."""
    _check_device(A, "matmul_int8")
    _check_device(B, "matmul_int8")
    a = A.contiguous()
    b = B.contiguous()
    m, k = a.shape
    k2, n = b.shape
    if k != k2:
        raise RuntimeError(f"shape mismatch: A is {tuple(a.shape)}, B is {tuple(b.shape)}")
    sa = A_scales.to(device=a.device, dtype=torch.float32).contiguous().view(-1)
    sb = B_scales.to(device=a.device, dtype=torch.float32).contiguous().view(-1)
    _need("A_scales", sa, m, "matmul_int8")
    _need("B_scales", sb, n, "matmul_int8")
    y = torch.empty(m, n, dtype=dtype, device=a.device)
    lib = N.lib()
    with torch.cuda.device(a.device):
        ws = _workspace(lib.mpsbnb_matmul_int8_workspace_bytes(N.i64(m), N.i64(n), N.i64(k)), a.device)
        N.check(lib.mpsbnb_matmul_int8(N.ptr(a), N.ptr(b), N.ptr(sa), N.ptr(sb), N.i64(m), N.i64(n), N.i64(k),
                                       N.ptr(y), N.dt(dtype), N.ptr(ws), C.c_size_t(ws.numel()), N.stream()),
                "matmul_int8")
    return y


def _linear_int8(x: Tensor, w: Tensor, row_scales: Tensor, col_scales: Optional[Tensor],
                 bias: Optional[Tensor], dtype: torch.dtype) -> Tensor:
    """y = x @ dequant(W int8 [N,K])^T + bias, W8A16 (shared by matmul_colrow and Linear8bit)."""
    n, k = w.shape
    orig_shape = x.shape
    op = dtype if dtype in (torch.float16, torch.bfloat16) else _mma_dtype(x.dtype)
    x2 = x.reshape(-1, k).to(op).contiguous()
    m = x2.shape[0]
    r = row_scales.to(device=x.device, dtype=torch.float32).contiguous().view(-1)
    c = None if col_scales is None else col_scales.to(device=x.device, dtype=torch.float32).contiguous().view(-1)
    b = None if bias is None else bias.to(device=x.device, dtype=op).contiguous()
    if x.shape[-1] != k:
        raise RuntimeError(f"input has {x.shape[-1]} features, weight expects {k}")
    _need("weight_row_scales", r, n, "the int8 linear")
    _need("weight_col_scales", c, k, "the int8 linear")
    _need("bias", b, n, "the int8 linear")
    y = torch.empty(m, n, dtype=dtype, device=x.device)
    lib = N.lib()
    with torch.cuda.device(x.device):
        ws = _workspace(lib.mpsbnb_linear_int8_workspace_bytes(N.i64(m), N.i64(n), N.i64(k)), x.device)
        N.check(lib.mpsbnb_linear_int8(N.ptr(x2), N.dt(op), N.i64(m), N.ptr(w.contiguous()), N.ptr(r), N.ptr(c),
                                       N.i64(n), N.i64(k), N.ptr(b), N.ptr(y), N.dt(dtype), N.ptr(ws),
                                       C.c_size_t(ws.numel()), N.stream()), "linear_int8")
    return y.reshape(*orig_shape[:-1], n) if len(orig_shape) != 2 else y


def matmul_fp8_e4m3(input: Tensor, weight: Tensor, weight_scales: Tensor,
                    bias: Optional[Tensor] = None, dtype: torch.dtype = torch.float16) -> Tensor:
    """mps_bitsandbytes/functional.py:796-807."""
    _check_device(input, "matmul_fp8_e4m3")
    _check_device(weight, "matmul_fp8_e4m3")
    is_1d = input.dim() == 1
    x = input.unsqueeze(0) if is_1d else input
    n, k = weight.shape
    orig_shape = x.shape
    op = dtype if dtype in (torch.float16, torch.bfloat16) else _mma_dtype(x.dtype)
    x2 = x.reshape(-1, k).to(op).contiguous()
    m = x2.shape[0]
    s = weight_scales.to(device=x.device, dtype=torch.float32).contiguous().view(-1)
    b = None if bias is None else bias.to(device=x.device, dtype=op).contiguous()
    if x.shape[-1] != k:
        raise RuntimeError(f"input has {x.shape[-1]} features, weight expects {k}")
    _need("weight_scales", s, n, "matmul_fp8_e4m3")
    _need("bias", b, n, "matmul_fp8_e4m3")
    y = torch.empty(m, n, dtype=dtype, device=x.device)
    lib = N.lib()
    with torch.cuda.device(x.device):
        ws = _workspace(lib.mpsbnb_linear_fp8_workspace_bytes(N.i64(m), N.i64(n), N.i64(k)), x.device)
        N.check(lib.mpsbnb_linear_fp8_e4m3(N.ptr(x2), N.dt(op), N.i64(m), N.ptr(weight.contiguous()), N.ptr(s),
                                           N.i64(n), N.i64(k), N.ptr(b), N.ptr(y), N.dt(dtype), N.ptr(ws),
                                           C.c_size_t(ws.numel()), N.stream()), "linear_fp8_e4m3")
    if len(orig_shape) != 2:
        y = y.reshape(*orig_shape[:-1], n)
    return y.squeeze(0) if is_1d else y


# =============================================================================
# LLM.int8-style statistics
# =============================================================================

def double_quant(
    A: Tensor,
    col_stats: Optional[Tensor] = None,
    row_stats: Optional[Tensor] = None,
    out_col: Optional[Tensor] = None,
    out_row: Optional[Tensor] = None,
    threshold: float = 0.0,
):
    """Row- and column-quantised int8 copies plus their statistics
    (mps_bitsandbytes/functional.py:814-863; ``threshold`` is ignored there too)."""
    if A.dim() != 2:
        raise ValueError("Input must be 2D")
    _check_device(A, "double_quant")
    src = _as_float(A).contiguous()
    rows, cols = src.shape
    dev = A.device
    rs_in = None if row_stats is None else row_stats.to(device=dev, dtype=torch.float32).contiguous()
    cs_in = None if col_stats is None else col_stats.to(device=dev, dtype=torch.float32).contiguous()
    _need("row_stats", rs_in, rows, "double_quant")
    _need("col_stats", cs_in, cols, "double_quant")
    rs = rs_in if rs_in is not None else torch.empty(rows, dtype=torch.float32, device=dev)
    cs = cs_in if cs_in is not None else torch.empty(cols, dtype=torch.float32, device=dev)
    new_row = torch.empty(rows, cols, dtype=torch.int8, device=dev) if out_row is None else None
    new_col = torch.empty(rows, cols, dtype=torch.int8, device=dev) if out_col is None else None
    with torch.cuda.device(dev):
        N.check(N.lib().mpsbnb_double_quant(
            N.ptr(src), N.dt(src.dtype), N.i64(rows), N.i64(cols), N.ptr(rs_in), N.ptr(cs_in), N.ptr(new_row),
            N.ptr(new_col), N.ptr(None if rs_in is not None else rs), N.ptr(None if cs_in is not None else cs),
            N.stream()), "double_quant")
    return (out_col if out_col is not None else new_col, out_row if out_row is not None else new_row,
            col_stats if col_stats is not None else cs, row_stats if row_stats is not None else rs, None)


def dequant_absmax(absmax_quant: Tensor, absmax_scales, blocksize: int = 256) -> Tensor:
    """mps_bitsandbytes/functional.py:866-889: absmax_quant * per-group scale (no /127);
    with a QuantState it is dequantize_blockwise."""
    if isinstance(absmax_scales, QuantState):
        return dequantize_blockwise(absmax_quant, absmax_scales)
    _check_device(absmax_quant, "dequant_absmax")
    one_d = absmax_quant.dim() == 1
    q = (absmax_quant.unsqueeze(0) if one_d else absmax_quant).contiguous()
    if q.dtype != torch.int8:
        q = q.to(torch.int8)
    rows, nblk = q.shape[0], q.numel() // max(q.shape[0], 1)
    s = absmax_scales.to(device=q.device, dtype=torch.float32).contiguous().view(rows, -1)
    ndq = s.shape[1]
    if ndq * blocksize < nblk:
        raise ValueError(f"absmax_scales has {ndq} groups per row, {nblk} blocks need {(nblk + blocksize - 1) // blocksize}")
    out = torch.empty(rows, nblk, dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        N.check(N.lib().mpsbnb_dequant_absmax(N.ptr(q), N.ptr(s), N.i64(rows), N.i64(nblk), N.i64(ndq), C.c_int(blocksize),
                                              N.ptr(out), N.stream()), "dequant_absmax")
    return out.squeeze(0) if one_d else out


def quantize_colrow(tensor: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    """int8 with scale sqrt(row_absmax * col_absmax) (mps_bitsandbytes/functional.py:896-924)."""
    if tensor.dim() != 2:
        raise ValueError("Input must be 2D")
    _check_device(tensor, "quantize_colrow")
    src = _as_float(tensor).contiguous()
    rows, cols = src.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=tensor.device)
    r = torch.empty(rows, dtype=torch.float32, device=tensor.device)
    c = torch.empty(cols, dtype=torch.float32, device=tensor.device)
    with torch.cuda.device(tensor.device):
        N.check(N.lib().mpsbnb_quantize_colrow(N.ptr(src), N.dt(src.dtype), N.i64(rows), N.i64(cols), N.ptr(q),
                                               N.ptr(r), N.ptr(c), N.stream()), "quantize_colrow")
    return q, r, c


def dequantize_colrow(quantized: Tensor, row_scales: Tensor, col_scales: Tensor,
                      dtype: torch.dtype = torch.float16) -> Tensor:
    """mps_bitsandbytes/functional.py:927-932."""
    _check_device(quantized, "dequantize_colrow")
    q = quantized.contiguous()
    rows, cols = q.shape
    r = row_scales.to(device=q.device, dtype=torch.float32).contiguous()
    c = col_scales.to(device=q.device, dtype=torch.float32).contiguous()
    _need("row_scales", r, rows, "dequantize_colrow")
    _need("col_scales", c, cols, "dequantize_colrow")
    out = torch.empty(rows, cols, dtype=dtype, device=q.device)
    with torch.cuda.device(q.device):
        N.check(N.lib().mpsbnb_dequantize_colrow(N.ptr(q), N.ptr(r), N.ptr(c), N.i64(rows), N.i64(cols),
                                                 N.ptr(out), N.dt(dtype), N.stream()), "dequantize_colrow")
    return out


def matmul_colrow(input: Tensor, weight_int8: Tensor, weight_row_scales: Tensor, weight_col_scales: Tensor,
                  bias: Optional[Tensor] = None, dtype: torch.dtype = torch.float16) -> Tensor:
    """mps_bitsandbytes/functional.py:935-945 (no threshold, no outlier split)."""
    _check_device(input, "matmul_colrow")
    _check_device(weight_int8, "matmul_colrow")
    return _linear_int8(input, weight_int8, weight_row_scales, weight_col_scales, bias, dtype)
