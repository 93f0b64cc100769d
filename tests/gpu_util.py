"""Helpers shared by the GPU parity tests (tensor <-> numpy, error norms)."""
import numpy as np
import torch

TD = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def to_cuda(a: np.ndarray, dtype: str):
    """numpy (bf16 held as exact float32) -> CUDA tensor of the named dtype."""
    return torch.from_numpy(np.ascontiguousarray(a)).to(TD[dtype]).cuda()


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    return t.float().numpy() if t.dtype == torch.bfloat16 else t.numpy()


def rel_err(y, ref) -> float:
    """max |y - ref| / max |ref|: the matmul parity norm (bound 1e-2)."""
    y = np.asarray(y, np.float32); ref = np.asarray(ref, np.float32)
    return float(np.abs(y - ref).max() / max(float(np.abs(ref).max()), 1e-30))


def assert_device_ok():
    """No kernel of the library recorded a timed-out wait."""
    import ctypes as C
    from mps_bitsandbytes_b200 import _native
    st = C.c_int(0)
    assert _native.lib().mpsbnb_device_status(C.byref(st), C.c_int(1)) == 0
    assert st.value == 0, f"device status word = {st.value}"
