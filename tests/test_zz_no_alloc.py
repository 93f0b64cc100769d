"""The workspace-free 4-bit GEMM entry point (scratch inside the library's device image).

Collected last on purpose (file name): it must pass both alone and after every other GPU test
has used the library.  Calls go through the C ABI; the reference results are the workspace-taking
entry point (the fused kernel: agreement within the matmul tolerance), the entry point itself on a
second call (exact) and the CPU oracle.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from mps_bitsandbytes_b200 import _native as N
    lib = N.lib()
    lib.mpsbnb_gemm_4bit_static_max_bytes.restype = C.c_size_t
    lib.mpsbnb_gemm_4bit_static_bytes.restype = C.c_size_t
    lib.mpsbnb_gemm_4bit_workspace_bytes.restype = C.c_size_t
    return N, lib


def _problem(M, N_, K, seed, dtype=torch.float16, double_quant=True, quant_type="nf4"):
    import mps_bitsandbytes_b200 as bnb
    from mps_bitsandbytes_b200.functional import _expand_absmax
    g = torch.Generator(device="cpu"); g.manual_seed(seed)
    w = (torch.randn(N_, K, generator=g) * 0.02).to(dtype).cuda()
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    bias = torch.randn(N_, generator=g).to(dtype).cuda()
    packed, st = bnb.quantize_4bit(w, blocksize=64, compress_statistics=double_quant, quant_type=quant_type)
    absmax, absmax2 = _expand_absmax(st.absmax, st.state2)
    return x, packed, absmax, absmax2, bias


def _with_workspace(N, lib, x, packed, absmax, absmax2, bias, M, N_, K, qt):
    y = torch.empty(M, N_, dtype=x.dtype, device="cuda")
    nbytes = lib.mpsbnb_gemm_4bit_workspace_bytes(N.i64(M), N.i64(N_), N.i64(K), C.c_int(64))
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    N.check(lib.mpsbnb_gemm_4bit(N.ptr(x), N.dt(x.dtype), N.i64(M), N.ptr(packed), N.ptr(absmax), N.ptr(absmax2),
                                 N.i64(N_), N.i64(K), C.c_int(64), C.c_int(N.qt(qt)), N.ptr(bias), N.ptr(y),
                                 N.dt(x.dtype), N.ptr(ws), C.c_size_t(nbytes), N.stream()), "gemm_4bit")
    return y


def _static(N, lib, x, packed, absmax, absmax2, bias, M, N_, K, qt, y=None):
    y = torch.empty(M, N_, dtype=x.dtype, device="cuda") if y is None else y
    rc = lib.mpsbnb_gemm_4bit_static(N.ptr(x), N.dt(x.dtype), N.i64(M), N.ptr(packed), N.ptr(absmax), N.ptr(absmax2),
                                     N.i64(N_), N.i64(K), C.c_int(64), C.c_int(N.qt(qt)), N.ptr(bias), N.ptr(y),
                                     N.dt(x.dtype), N.stream())
    return rc, y


@pytest.mark.parametrize("M,N_,K,qt,dq", [(160, 512, 1024, "nf4", True), (33, 200, 1004, "fp4", False)])
def test_static_matches_workspace_entry_point_twice(M, N_, K, qt, dq):
    N, lib = _lib()
    x, packed, absmax, absmax2, bias = _problem(M, N_, K, seed=11, double_quant=dq, quant_type=qt)
    want = _with_workspace(N, lib, x, packed, absmax, absmax2, bias, M, N_, K, qt)
    rc1, got1 = _static(N, lib, x, packed, absmax, absmax2, bias, M, N_, K, qt)
    # a second problem in between leaves other bytes in the shared scratch
    x2, p2, a2, a22, b2 = _problem(64, 256, 512, seed=12, double_quant=dq, quant_type=qt)
    want2 = _with_workspace(N, lib, x2, p2, a2, a22, b2, 64, 256, 512, qt)
    rcm, gotm = _static(N, lib, x2, p2, a2, a22, b2, 64, 256, 512, qt)
    rc2, got2 = _static(N, lib, x, packed, absmax, absmax2, bias, M, N_, K, qt)
    torch.cuda.synchronize()
    assert (rc1, rcm, rc2) == (0, 0, 0)
    def close(a, b):
        a, b = a.float(), b.float()
        return float((a - b).abs().max() / b.abs().max()) <= 1e-2
    assert close(got1, want)
    assert close(gotm, want2)
    assert torch.equal(got2, got1)                              # the call repeats exactly, whatever the scratch held
    # ... and against the CPU oracle of the reference's path (dequantise the whole weight, then matmul)
    if x.dtype == torch.float16:
        import numpy as np
        from oracle import oracle_c
        am = absmax.cpu().numpy() if absmax2 is None else oracle_c.dequantize_absmax(absmax.cpu().numpy(), absmax2.cpu().numpy())
        ref = oracle_c.matmul_4bit_f16(x.cpu().numpy(), packed.cpu().numpy(), am.astype(np.float32), N_, K, 64, qt,
                                       bias=bias.cpu().numpy())
        err = np.abs(got2.cpu().numpy().astype(np.float32) - ref.astype(np.float32)).max() / np.abs(ref.astype(np.float32)).max()
        assert err <= 1e-2, err
    code = C.c_int(0)
    assert lib.mpsbnb_device_status(C.byref(code), C.c_int(0)) == 0 and code.value == 0


def test_static_refuses_what_does_not_fit():
    N, lib = _lib()
    limit = lib.mpsbnb_gemm_4bit_static_max_bytes()
    assert limit == 32 << 20
    # 4096 x 4096 fp16 is exactly the limit; one more row is beyond it.  Nothing is enqueued, so the
    # (small) tensors passed here are never read at these sizes.
    x, packed, absmax, absmax2, bias = _problem(16, 64, 128, seed=13)
    assert lib.mpsbnb_gemm_4bit_static_bytes(N.ptr(x), N.i64(16), N.i64(4096), N.i64(4096)) == limit
    assert lib.mpsbnb_gemm_4bit_static_bytes(N.ptr(x), N.i64(16), N.i64(4097), N.i64(4096)) > limit
    y = torch.full((16, 64), 7.0, dtype=torch.float16, device="cuda")
    rc, _ = _static(N, lib, x, packed, absmax, absmax2, bias, 16, 4097, 4096, "nf4", y=y)
    torch.cuda.synchronize()
    assert rc == -5                                            # MPSBNB_ERR_TOO_LARGE
    assert bool((y == 7.0).all())
    rc, _ = _static(N, lib, x, packed, absmax, absmax2, bias, 16, 1 << 30, 1 << 30, "nf4", y=y)
    assert rc == -5
    # sizes beyond 32-bit are refused before any size arithmetic
    rc, _ = _static(N, lib, x, packed, absmax, absmax2, bias, 16, 64, (1 << 63) - 1, "nf4", y=y)
    assert rc == -5
    lib.mpsbnb_gemm_4bit_static_forget()                        # drops the cached address; the next call resolves it again
    rc, y2 = _static(N, lib, x, packed, absmax, absmax2, bias, 16, 64, 128, "nf4")
    torch.cuda.synchronize()
    assert rc == 0 and bool(torch.isfinite(y2.float()).all())
