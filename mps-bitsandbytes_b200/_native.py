"""ctypes binding of the C-ABI CUDA library (``lib/libmpsbnb_b200.so``).

There is no fallback of any kind: if the library is missing, or no CUDA device is
present, every operation raises.  The binding only unwraps ``data_ptr()`` and the current
CUDA stream; all arithmetic happens in the library's sm_100a kernels.
"""
import ctypes as C
import os
import re

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# MPSBNB_B200_LIB points at a library built elsewhere (default: the in-tree build)
LIB_PATH = os.environ.get("MPSBNB_B200_LIB") or os.path.join(_HERE, "lib", "libmpsbnb_b200.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "mpsbnb_b200.h")

F16, BF16, F32 = 0, 1, 2
GROUP_PDL = 1
NF4, FP4 = 0, 1
_DT = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}
_QT = {"nf4": NF4, "fp4": FP4}

_lib = None


class Linear4Desc(C.Structure):
    """mpsbnb_linear4_desc of include/mpsbnb_b200.h."""
    _fields_ = [("x", C.c_void_p), ("x_ld", C.c_int64), ("x_period", C.c_int64), ("packed", C.c_void_p),
                ("absmax", C.c_void_p), ("absmax2", C.c_void_p), ("bias", C.c_void_p), ("y", C.c_void_p),
                ("acc", C.c_void_p), ("N", C.c_int64), ("K", C.c_int64), ("segment", C.c_int64)]


class GroupEpilogue(C.Structure):
    """mpsbnb_group_epilogue of include/mpsbnb_b200.h."""
    _fields_ = [("acc", C.c_void_p), ("peer_h", C.c_void_p), ("peer_flags", C.c_void_p), ("step", C.c_void_p),
                ("counter", C.c_void_p), ("tile_cnt", C.c_void_p), ("alpha", C.c_float), ("M", C.c_int), ("hs", C.c_int),
                ("H", C.c_int), ("rank", C.c_int), ("nranks", C.c_int), ("mul", C.c_int), ("add", C.c_int),
                ("tile_expect", C.c_int), ("nbuf", C.c_int), ("count_tiles", C.c_int)]


class GroupPlan(C.Structure):
    """mpsbnb_group_plan of include/mpsbnb_b200.h."""
    _fields_ = [("dev", C.c_void_p), ("units_offset", C.c_int64), ("n_linears", C.c_int), ("n_units", C.c_int),
                ("M", C.c_int), ("x_dtype", C.c_int), ("quant_type", C.c_int), ("flags", C.c_int),
                ("aux_offset", C.c_int64), ("grid", C.c_int), ("impl", C.c_int),
                ("wait_flags", C.c_void_p), ("wait_step", C.c_void_p), ("wait_n", C.c_int), ("wait_mul", C.c_int),
                ("wait_add", C.c_int), ("acc_parts", C.c_int), ("n_segments", C.c_int), ("wait_seg_mul", C.c_int), ("ep", GroupEpilogue)]


class NativeLibraryError(RuntimeError):
    pass


def lib():
    """Load the shared library once.  Raises NativeLibraryError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeLibraryError(
                f"{LIB_PATH} not found: build it with `python mps-bitsandbytes_b200/build.py` "
                "(there is no CPU or PyTorch fallback)")
        l = C.CDLL(LIB_PATH)
        l.mpsbnb_status_string.restype = C.c_char_p
        l.mpsbnb_last_cuda_error_string.restype = C.c_char_p
        for name in ("mpsbnb_gemv_4bit_group_plan_bytes", "mpsbnb_gemm_4bit_workspace_bytes", "mpsbnb_matmul_int8_workspace_bytes",
                     "mpsbnb_linear_int8_workspace_bytes", "mpsbnb_linear_fp8_workspace_bytes",
                     "mpsbnb_outlier_linear_workspace_bytes", "mpsbnb_gemm_4bit_static_max_bytes", "mpsbnb_gemm_4bit_static_bytes"):
            if hasattr(l, name):
                getattr(l, name).restype = C.c_size_t
        _lib = l
    return _lib


def declared_symbols():
    """Names of every function declared in include/mpsbnb_b200.h."""
    with open(HEADER_PATH) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(mpsbnb_[a-z0-9_]+)\s*\(", text)))


def dt(dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}; expected float16, bfloat16 or float32") from None


def qt(quant_type: str) -> int:
    return _QT[quant_type]


def ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def i64(v):
    return C.c_int64(int(v))


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and t.device.type != "cuda":
            raise ValueError(
                f"mps-bitsandbytes_b200 requires tensors on a 'cuda' device, got '{t.device.type}'. "
                "Move the tensor with .to('cuda'); there is no CPU path")


def check(status: int, what: str):
    if status == 0:
        return
    l = lib()
    msg = l.mpsbnb_status_string(status).decode()
    if status == -3:
        msg += ": " + l.mpsbnb_last_cuda_error_string().decode()
    raise RuntimeError(f"{what} failed ({status}): {msg}")
