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
    """The matmul parity figure (bound 1e-2): the larger of two norms,
      max |y - ref| / max |ref|                     (error against the largest output), and
      max_i |y_i - ref_i| / (|ref_i| + rms(ref))    (<= 1e-2 is allclose(rtol=1e-2, atol=1e-2 rms(ref)):
                                                     a small output may not be wholly wrong)."""
    y = np.asarray(y, np.float32); ref = np.asarray(ref, np.float32)
    if ref.size == 0:
        return 0.0
    d = np.abs(y - ref)
    n1 = float(d.max() / max(float(np.abs(ref).max()), 1e-30))
    rms = float(np.sqrt(np.mean(np.square(ref.astype(np.float64)))))
    n2 = float((d / (np.abs(ref) + max(rms, 1e-30))).max())
    return max(n1, n2)


def assert_device_ok():
    """No kernel of the library recorded a timed-out wait."""
    import ctypes as C
    from mps_bitsandbytes_b200 import _native
    st = C.c_int(0)
    assert _native.lib().mpsbnb_device_status(C.byref(st), C.c_int(1)) == 0
    assert st.value == 0, f"device status word = {st.value}"
