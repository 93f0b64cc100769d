"""GPU parity, matmuls: the fused dequantise-GEMV (decode), the tcgen05 GEMM (prefill) and the
INT8 / FP8 linears, through the C ABI, against the oracle and the stored reference outputs.
Bound: max |y - y_ref| / max |y_ref| <= 1e-2 (fp16/bf16 operands, fp32 accumulation)."""
import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from oracle import oracle_c, oracle_np as O
from gpu_util import assert_device_ok, rel_err, to_cuda, to_np

pytestmark = pytest.mark.gpu
TOL = 1e-2


def quantized(rng, n, k, qt, dq, dt="float16", scale=0.02):
    w_np = O.cast_to((rng.standard_normal((n, k)) * scale).astype(np.float32), dt)
    packed, st = bnb.quantize_4bit(to_cuda(w_np, dt), compress_statistics=dq, quant_type=qt)
    p, a, a2 = O.quantize_4bit(w_np, 64, qt, dq)
    return packed, st, (p, a, a2)


def test_golden_matmul_4bit(golden):
    g = golden("matmul")
    for i in range(int(g["mm4_n"])):
        M, N, K, qt, dq, bias, dt = g[f"mm4_{i}_meta"]
        packed, st = bnb.quantize_4bit(to_cuda(g[f"mm4_{i}_w"], dt), compress_statistics=bool(int(dq)), quant_type=qt)
        b = to_cuda(g[f"mm4_{i}_b"], dt) if int(bias) else None
        y = bnb.matmul_4bit(to_cuda(g[f"mm4_{i}_x"], dt), packed, st, b)
        assert y.dtype == getattr(torch, dt) and tuple(y.shape) == (int(M), int(N))
        assert rel_err(to_np(y), g[f"mm4_{i}_y"]) <= TOL, (i, rel_err(to_np(y), g[f"mm4_{i}_y"]))
    assert_device_ok()


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16, 17, 24, 25, 32])
@pytest.mark.parametrize("qt,dq", [("nf4", False), ("nf4", True), ("fp4", True)])
def test_gemv_decode_shapes(M, qt, dq):
    rng = np.random.default_rng(M * 7 + len(qt) + dq)
    N, K = 200, 1088
    packed, st, (p, a, a2) = quantized(rng, N, K, qt, dq)
    x = rng.standard_normal((M, K)).astype(np.float16)
    bias = rng.standard_normal(N).astype(np.float16)
    y = bnb.matmul_4bit(torch.from_numpy(x).cuda(), packed, st, torch.from_numpy(bias).cuda())
    ref = O.matmul_4bit(x, p, a, (N, K), 64, qt, "float16", a2, bias, "float16")
    assert rel_err(to_np(y), ref) <= TOL


@pytest.mark.parametrize("M,K,N", [(1, 64, 128), (7, 64, 128), (32, 63, 127), (32, 64, 65), (3, 1, 5), (5, 130, 33),
                                   (1, 4096, 4096), (16, 11008, 512), (4, 4104, 96)])
def test_gemv_odd_shapes(M, K, N):
    rng = np.random.default_rng(M + K + N)
    packed, st, (p, a, a2) = quantized(rng, N, K, "nf4", False)
    x = rng.standard_normal((M, K)).astype(np.float16)
    y = bnb.matmul_nf4(torch.from_numpy(x).cuda(), packed, st)
    ref = O.matmul_4bit(x, p, a, (N, K), 64, "nf4", "float16")
    assert tuple(y.shape) == (M, N) and np.isfinite(to_np(y).astype(np.float32)).all()
    assert rel_err(to_np(y), ref) <= TOL


def test_gemv_bf16_and_output_dtypes():
    rng = np.random.default_rng(77)
    N, K = 96, 512
    packed, st, (p, a, a2) = quantized(rng, N, K, "nf4", True, "bfloat16")
    x = O.cast_to(rng.standard_normal((3, K)).astype(np.float32), "bfloat16")
    ref = O.matmul_4bit(x, p, a, (N, K), 64, "nf4", "bfloat16", a2, None, "float32")
    for cd in (torch.bfloat16, torch.float16, torch.float32):
        y = bnb.matmul_4bit(to_cuda(x, "bfloat16"), packed, st, None, compute_dtype=cd)
        assert y.dtype == cd and rel_err(to_np(y), ref) <= TOL
    # batched (3-D) input keeps its leading dimensions
    xb = to_cuda(np.stack([x, x]), "bfloat16")
    yb = bnb.matmul_4bit(xb, packed, st)
    assert tuple(yb.shape) == (2, 3, N) and torch.equal(yb[0], yb[1])


def test_gemm_f16_dense_vs_fp32_reference():
    """The tcgen05 GEMM on plain fp16/bf16 operands vs an fp32 matmul of the same operands."""
    import ctypes as C
    from mps_bitsandbytes_b200 import _native as Nn
    rng = np.random.default_rng(3)
    for (M, N, K, dt) in [(128, 256, 64, torch.float16), (128, 256, 512, torch.float16), (300, 520, 200, torch.float16),
                          (1024, 768, 1024, torch.bfloat16), (40, 136, 72, torch.bfloat16), (257, 129, 4096, torch.float16)]:
        a = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(dt).cuda()
        b = torch.from_numpy((rng.standard_normal((N, K)) * 0.05).astype(np.float32)).to(dt).cuda()
        bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).to(dt).cuda()
        y = torch.empty(M, N, dtype=dt, device="cuda")
        Nn.check(Nn.lib().mpsbnb_gemm_f16(Nn.ptr(a), Nn.i64(K), Nn.ptr(b), Nn.i64(K), Nn.dt(dt), Nn.i64(M), Nn.i64(N),
                                          Nn.i64(K), None, None, Nn.ptr(bias), Nn.ptr(y), Nn.dt(dt), Nn.stream()), "gemm_f16")
        ref = a.float() @ b.float().T + bias.float()
        torch.cuda.synchronize()
        assert rel_err(to_np(y), to_np(ref)) <= 4e-3, (M, N, K, rel_err(to_np(y), to_np(ref)))
    assert_device_ok()


@pytest.mark.parametrize("M,N,K", [(33, 64, 128), (128, 256, 512), (130, 96, 192), (512, 320, 1024), (100, 77, 136),
                                   (64, 130, 127)])
@pytest.mark.parametrize("qt,dq", [("nf4", True), ("fp4", False)])
def test_gemm_prefill_shapes(M, N, K, qt, dq):
    rng = np.random.default_rng(M + N + K)
    packed, st, (p, a, a2) = quantized(rng, N, K, qt, dq)
    x = rng.standard_normal((M, K)).astype(np.float16)
    bias = rng.standard_normal(N).astype(np.float16)
    y = bnb.matmul_4bit(torch.from_numpy(x).cuda(), packed, st, torch.from_numpy(bias).cuda())
    ref = O.matmul_4bit(x, p, a, (N, K), 64, qt, "float16", a2, bias, "float16")
    assert rel_err(to_np(y), ref) <= TOL
    assert_device_ok()


def test_gemv_and_gemm_paths_agree_and_are_linear():
    """Same weight through both kernels; and y(x1 + x2) = y(x1) + y(x2) within rounding."""
    rng = np.random.default_rng(11)
    N, K = 1024, 2048
    packed, st, _ = quantized(rng, N, K, "nf4", True)
    x = torch.from_numpy(rng.standard_normal((64, K)).astype(np.float16)).cuda()
    y_gemm = bnb.matmul_4bit(x, packed, st)                    # M = 64: tensor-core GEMM
    y_gemv = torch.cat([bnb.matmul_4bit(x[i:i + 16], packed, st) for i in range(0, 64, 16)])
    assert rel_err(to_np(y_gemv), to_np(y_gemm)) <= 4e-3
    y12 = bnb.matmul_4bit((x[:8].float() * 0.5 + x[8:16].float() * 0.5).half(), packed, st).float()
    assert rel_err(to_np(y12), to_np(y_gemv[:8].float() * 0.5 + y_gemv[8:16].float() * 0.5)) <= 4e-3
    assert_device_ok()


def test_fifty_repeated_matmuls_are_identical():
    rng = np.random.default_rng(5)
    packed, st, _ = quantized(rng, 256, 512, "nf4", False)
    x = torch.from_numpy(rng.standard_normal((4, 512)).astype(np.float16)).cuda()
    y0 = bnb.matmul_4bit(x, packed, st)
    for _ in range(50):
        assert torch.equal(bnb.matmul_4bit(x, packed, st), y0)


def test_config1_full_size_matmul_vs_c_oracle():
    """BASELINE config 1: 4096 x 4096 NF4 weight, x [1, 4096]."""
    torch.manual_seed(0)
    w = (torch.randn(4096, 4096) * 0.02).half()
    torch.manual_seed(1)
    x = torch.randn(1, 4096).half()
    packed, st = bnb.quantize_nf4(w.cuda())
    y = bnb.matmul_nf4(x.cuda(), packed, st)
    ref = oracle_c.matmul_4bit_f16(x.numpy(), to_np(packed), to_np(st.absmax), 4096, 4096, 64, "nf4")
    assert rel_err(to_np(y), ref) <= TOL


def test_int8_and_fp8_matmuls(golden):
    g = golden("matmul")
    y = bnb.matmul_int8(to_cuda(g["i8_Aq"], "float32").to(torch.int8), to_cuda(g["i8_Bq"], "float32").to(torch.int8),
                        to_cuda(g["i8_As"], "float32"), to_cuda(g["i8_Bs"], "float32"))
    assert rel_err(to_np(y), g["i8_y"]) <= TOL
    A = to_cuda(g["i8_A"], "float16"); W = to_cuda(g["cr_W"], "float16"); b = to_cuda(g["cr_b"], "float16")
    q, r, c = bnb.quantize_colrow(W)
    assert rel_err(to_np(bnb.matmul_colrow(A, q, r, c, b)), g["cr_y"]) <= TOL
    c8, s8 = bnb.quantize_fp8_e4m3(W)
    assert rel_err(to_np(bnb.matmul_fp8_e4m3(A, c8, s8, b)), g["f8_y"]) <= TOL
    y1 = bnb.matmul_fp8_e4m3(A[0], c8, s8, b)                  # 1-D input
    assert y1.dim() == 1 and y1.numel() == W.shape[0]
    # larger, against the oracle
    rng = np.random.default_rng(41)
    M, K, N = 192, 520, 328
    x = rng.standard_normal((M, K)).astype(np.float16)
    x[:, ::97] *= 20                                            # a few large-magnitude input columns
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    xq, xs = O.quantize_rowwise(x)
    wq_t, ws = O.quantize_rowwise(w)
    Bq = np.ascontiguousarray(wq_t.T)                           # [K, N], per-column scales
    y = bnb.matmul_int8(torch.from_numpy(xq).cuda(), torch.from_numpy(Bq).cuda(), torch.from_numpy(xs).cuda(),
                        torch.from_numpy(ws).cuda())
    assert rel_err(to_np(y), O.matmul_int8(xq, Bq, xs, ws)) <= TOL
    q, r, c = O.quantize_colrow(w)
    y = bnb.matmul_colrow(torch.from_numpy(x).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(r).cuda(),
                          torch.from_numpy(c).cuda())
    assert rel_err(to_np(y), O.matmul_colrow(x, q, r, c)) <= TOL
    c8, s8 = O.quantize_fp8_e4m3(w)
    y = bnb.matmul_fp8_e4m3(torch.from_numpy(x).cuda(), torch.from_numpy(c8).cuda(), torch.from_numpy(s8).cuda())
    assert rel_err(to_np(y), O.matmul_fp8_e4m3(x, c8, s8)) <= TOL
    assert_device_ok()


def test_short_argument_tensors_raise_instead_of_reading_out_of_bounds():
    """The kernels take raw pointers: tensors shorter than the shapes imply are refused on the host."""
    rng = np.random.default_rng(9)
    packed, st, _ = quantized(rng, 64, 200, "nf4", True)           # K = 200: rows are padded to 256 in the layout
    x = torch.randn(3, 200, device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError, match="packed weight"):
        bnb.matmul_4bit(x, packed[:-8], st)
    with pytest.raises(ValueError, match="bias"):
        bnb.matmul_4bit(x, packed, st, torch.zeros(63, device="cuda", dtype=torch.float16))
    short = bnb.QuantState(absmax=st.absmax[:-1], shape=st.shape, blocksize=64, quant_type="nf4", dtype=st.dtype, state2=st.state2)
    with pytest.raises(ValueError, match="absmax"):
        bnb.matmul_4bit(x, packed, short)
    # a packed tensor stored in another integer type holds the byte VALUES and is converted back
    y = bnb.matmul_4bit(x, packed, st)
    assert torch.equal(bnb.matmul_4bit(x, packed.to(torch.int32), st), y)
    q = torch.zeros(8, 32, dtype=torch.int8, device="cuda")
    with pytest.raises(ValueError, match="scales"):
        bnb.dequantize_rowwise(q, torch.ones(7, device="cuda"))
    with pytest.raises(ValueError, match="scales"):
        bnb.dequantize_fp8_e4m3(q.view(torch.uint8), torch.ones(7, device="cuda"))
    with pytest.raises(ValueError, match="col_scales"):
        bnb.dequantize_colrow(q, torch.ones(8, device="cuda"), torch.ones(31, device="cuda"))
    with pytest.raises(ValueError, match="B_scales"):
        bnb.matmul_int8(q, torch.zeros(32, 16, dtype=torch.int8, device="cuda"), torch.ones(8, device="cuda"), torch.ones(15, device="cuda"))
    with pytest.raises(ValueError, match="weight_row_scales"):
        bnb.matmul_colrow(torch.zeros(2, 32, device="cuda", dtype=torch.float16), q, torch.ones(7, device="cuda"), torch.ones(32, device="cuda"))
    with pytest.raises(ValueError, match="weight_scales"):
        bnb.matmul_fp8_e4m3(torch.zeros(2, 32, device="cuda", dtype=torch.float16), q.view(torch.uint8), torch.ones(7, device="cuda"))
    with pytest.raises(ValueError, match="row_stats"):
        bnb.double_quant(torch.zeros(8, 32, device="cuda"), row_stats=torch.ones(7, device="cuda"))
    with pytest.raises(ValueError, match="absmax"):
        bnb.quantize_blockwise(torch.zeros(1000, device="cuda"), absmax=torch.ones(1, device="cuda"), blocksize=256)
    # dequant_absmax (tensor form) runs on a kernel
    aq = torch.randint(-127, 128, (3, 600), dtype=torch.int8, device="cuda")
    sc = torch.rand(3, 3, device="cuda") + 0.5
    ref = aq.float() * sc[:, torch.arange(600, device="cuda") // 256]
    assert torch.equal(bnb.dequant_absmax(aq, sc, 256), ref)
    assert torch.equal(bnb.dequant_absmax(aq[0], sc[0], 256), ref[0])
    assert_device_ok()
