"""Failure detection of the layer-boundary exchange without a GPU fault: a wait whose flag nobody raises runs
out after about a second, the kernel returns, the host reads status 502, and the context is still usable."""
import ctypes as C
import time

import pytest
import torch

from mps_bitsandbytes_b200 import _native

pytestmark = pytest.mark.gpu


def test_flag_wait_times_out_and_reports():
    lib = _native.lib()
    code = C.c_int(0)
    assert lib.mpsbnb_device_status(C.byref(code), C.c_int(1)) == 0            # start clean
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    flags[0] = 7                                                               # one peer arrived, the other never does
    step = torch.ones(1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    rc = lib.mpsbnb_flags_wait(_native.ptr(flags), C.c_int(2), _native.ptr(step), C.c_int(1), C.c_int(5), C.c_int(0),
                               _native.stream())
    assert rc == 0
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert 0.3 < dt < 10.0, dt                                                 # bounded: about a second
    assert lib.mpsbnb_device_status(C.byref(code), C.c_int(1)) == 0 and code.value == 502
    # the context is alive and the status word is clear again
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
    assert lib.mpsbnb_device_status(C.byref(code), C.c_int(0)) == 0 and code.value == 0
    # a satisfied wait returns at once
    flags.fill_(6)
    assert lib.mpsbnb_flags_wait(_native.ptr(flags), C.c_int(2), _native.ptr(step), C.c_int(1), C.c_int(5), C.c_int(0),
                                 _native.stream()) == 0
    torch.cuda.synchronize()
    assert lib.mpsbnb_device_status(C.byref(code), C.c_int(1)) == 0 and code.value == 0
