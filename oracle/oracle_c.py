"""ctypes front end of the C oracle (oracle.c).  TEST INFRASTRUCTURE ONLY."""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None
QT = {"nf4": 0, "fp4": 1}


def lib():
    global _lib
    if _lib is None:
        path = _build.OUT if os.path.exists(_build.OUT) else _build.build()
        _lib = C.CDLL(path)
        _lib.o_padded_k.restype = C.c_int64
        _lib.o_padded_k.argtypes = [C.c_int64, C.c_int64]
        _lib.o_prove_quantizer.restype = C.c_int64
        _lib.o_prove_quantizer.argtypes = [C.c_int, C.c_int, C.c_int64, C.c_float, C.c_float]
        _lib.o_prove_thresholds.restype = C.c_int64
        _lib.o_prove_thresholds.argtypes = [C.c_int, C.c_int, C.c_int64]
        _lib.o_threshold.restype = C.c_float
        _lib.o_threshold.argtypes = [C.c_float, C.c_float, C.c_int]
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def quantize_4bit(A, blocksize=64, quant_type="nf4"):
    """Returns (packed uint8 [rows*Kp/2], absmax fp32 [rows*nb]); A is [rows, cols]."""
    A = np.ascontiguousarray(A, dtype=np.float32)
    rows, cols = A.shape
    kp = lib().o_padded_k(cols, blocksize)
    packed = np.empty(rows * kp // 2, np.uint8)
    absmax = np.empty(rows * kp // blocksize, np.float32)
    lib().o_quantize_4bit(_p(A), C.c_int64(rows), C.c_int64(cols), C.c_int64(blocksize),
                          C.c_int(QT[quant_type]), _p(packed), _p(absmax))
    return packed, absmax


def dequantize_4bit(packed, absmax, shape, blocksize=64, quant_type="nf4"):
    """fp32 values code[idx] * absmax, shape [rows, cols] (round to the target dtype yourself)."""
    rows, cols = shape
    packed = np.ascontiguousarray(packed, np.uint8)
    absmax = np.ascontiguousarray(absmax, np.float32)
    out = np.empty((rows, cols), np.float32)
    lib().o_dequantize_4bit(_p(packed), _p(absmax), C.c_int64(rows), C.c_int64(cols),
                            C.c_int64(blocksize), C.c_int(QT[quant_type]), _p(out))
    return out


def dequantize_absmax(q, absmax2):
    q = np.ascontiguousarray(q, np.int8)
    absmax2 = np.ascontiguousarray(absmax2, np.float32)
    out = np.empty(q.size, np.float32)
    lib().o_dequantize_absmax(_p(q), _p(absmax2), C.c_int64(q.size), _p(out))
    return out


def matmul_4bit_f16(x, packed, absmax, N, K, blocksize=64, quant_type="nf4", bias=None, scratch=None):
    """y[M,N] fp16 = x[M,K] fp16 @ dequant(W)^T, whole weight re-materialised in fp16 first."""
    x = np.ascontiguousarray(x, np.float16)
    M = x.shape[0]
    packed = np.ascontiguousarray(packed, np.uint8)
    absmax = np.ascontiguousarray(absmax, np.float32)
    y = np.empty((M, N), np.float16)
    if scratch is None:
        scratch = np.empty((N, K), np.float16)
    b = None if bias is None else np.ascontiguousarray(bias, np.float16)
    lib().o_matmul_4bit_f16(_p(x), _p(packed), _p(absmax), C.c_int64(M), C.c_int64(N), C.c_int64(K),
                            C.c_int64(blocksize), C.c_int(QT[quant_type]),
                            _p(b) if b is not None else None, _p(y), _p(scratch))
    return y


def thresholds(quant_type):
    n = 15 if quant_type == "nf4" else 7
    t = np.empty(15, np.float32)
    (lib().o_nf4_thresholds if quant_type == "nf4" else lib().o_fp4_thresholds)(_p(t))
    return t[:n].copy()
