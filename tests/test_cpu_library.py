"""CPU-side checks: the C-ABI library loads and exports every declared symbol, the decision
thresholds compiled into the CUDA quantiser are the ones the oracle derives, the shortcuts of
the quantiser are proven against the reference arithmetic, and the Python surface mirrors
the reference's names and argument order.  No kernel runs here."""
import ctypes as C
import inspect
import os
import re

import numpy as np
import pytest
import torch

import mps_bitsandbytes_b200 as bnb
from mps_bitsandbytes_b200 import _native
from oracle import oracle_c


def test_library_loads_and_exports_every_declared_symbol():
    lib = _native.lib()
    names = _native.declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mpsbnb_b200.h but not exported"
    assert lib.mpsbnb_abi_version() >= 1
    assert lib.mpsbnb_status_string(0).decode() == "ok"
    assert "workspace" in lib.mpsbnb_status_string(-4).decode()
    assert lib.mpsbnb_gemv_4bit_max_m() == 32


def test_workspace_size_queries_need_no_gpu():
    lib = _native.lib()
    import ctypes as C
    # block size 64 runs fused: room for a re-pitched copy of x only; other block sizes expand the weight first
    n = lib.mpsbnb_gemm_4bit_workspace_bytes(C.c_int64(2048), C.c_int64(11008), C.c_int64(4096), C.c_int(64))
    assert 2048 * 4096 * 2 <= n < 11008 * 4096 * 2
    n = lib.mpsbnb_gemm_4bit_workspace_bytes(C.c_int64(2048), C.c_int64(11008), C.c_int64(4096), C.c_int(128))
    assert n >= 11008 * 4096 * 2
    assert lib.mpsbnb_gemm_4bit_workspace_bytes(C.c_int64(0), C.c_int64(8), C.c_int64(8), C.c_int(64)) == 0


def test_compiled_thresholds_match_oracle():
    src = open(os.path.join(os.path.dirname(_native.LIB_PATH), "..", "csrc", "quant4.cu")).read()
    for qt, n in (("NF4", 15), ("FP4", 7)):
        t = oracle_c.thresholds(qt.lower())
        for i in range(n):
            m = re.search(rf"#define {qt}_T{i} (\S+)f\b", src)
            assert m, f"{qt}_T{i} missing"
            assert np.float32(float.fromhex(m.group(1))) == t[i], (qt, i)


@pytest.mark.parametrize("qt", [0, 1])
def test_threshold_search_equals_16_way_search(qt):
    assert oracle_c.lib().o_prove_thresholds(qt, 2048, 2_000_000) == 0


def test_nf4_bucket_search_equals_threshold_search():
    """The fast quantiser's NF4 search (bucket by trunc(fma(v, 8, 8)), two compares) against the threshold search
    on every third float bit pattern, values outside [-1, 1] included (stride 1, every float, also returns 0)."""
    fn = oracle_c.lib().o_prove_nf4_buckets
    fn.restype = C.c_int64
    assert fn(C.c_int64(3)) == 0


def test_nf4_bucket_search_by_truncating_fma_equals_threshold_search():
    """The streaming quantiser's form (32 buckets of one threshold at most, bucket = low bits of
    fma_rz(v, 16, 2^23 + 16), no conversion, no clamp) on every third float of [-1, 1], the range of x / absmax inside
    a block (stride 1 also returns 0)."""
    fn = oracle_c.lib().o_prove_nf4_buckets32_rz
    fn.restype = C.c_int64
    assert fn(C.c_int64(3)) == 0


def test_fp4_bucket_search_by_truncating_fma_equals_threshold_search():
    """FP4 form of the streaming quantiser (16 buckets over |v|, bucket = low bits of fma_rz(|v|, 16, 2^23)) on every
    third float of [-1, 1] (stride 1 also returns 0)."""
    fn = oracle_c.lib().o_prove_fp4_buckets16_rz
    fn.restype = C.c_int64
    assert fn(C.c_int64(3)) == 0


@pytest.mark.parametrize("qt,bf16", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_reciprocal_division_shortcut_is_exact_for_16bit_inputs(qt, bf16):
    """Every (x, absmax) pair of the format with absmax in the range where the kernel uses the
    shortcut, [1e-30, 1e30]; a stride of 3 over absmax keeps the CPU suite short (the full
    sweep, stride 1, also returns 0)."""
    assert oracle_c.lib().o_prove_quantizer(qt, bf16, 3, 1e-30, 1e30) == 0


def test_c_oracle_matches_numpy_oracle():
    from oracle import oracle_np as O
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((64, 320)) * 0.02).astype(np.float16)
    for qt in ("nf4", "fp4"):
        p, a, _ = O.quantize_4bit(w, 64, qt)
        pc, ac = oracle_c.quantize_4bit(w.astype(np.float32), 64, qt)
        assert np.array_equal(p, pc) and np.array_equal(a, ac)
        d = O.dequantize_4bit(p, a, w.shape, 64, qt, "float16")
        dc = oracle_c.dequantize_4bit(pc, ac, w.shape, 64, qt).astype(np.float16)
        assert np.array_equal(d, dc)
        x = rng.standard_normal((3, 320)).astype(np.float16)
        y = O.matmul_4bit(x, p, a, w.shape, 64, qt)
        yc = oracle_c.matmul_4bit_f16(x, pc, ac, 64, 320, 64, qt)
        assert np.abs(y.astype(np.float32) - yc.astype(np.float32)).max() <= 1e-2 * np.abs(y.astype(np.float32)).max()


def test_public_names_and_argument_order_match_reference():
    ref_signatures = {
        "quantize_4bit": ["A", "absmax", "out", "blocksize", "compress_statistics", "quant_type", "quant_storage"],
        "dequantize_4bit": ["A", "quant_state", "absmax", "out", "blocksize", "quant_type"],
        "quantize_nf4": ["A", "absmax", "out", "blocksize", "compress_statistics", "quant_storage"],
        "dequantize_fp4": ["A", "quant_state", "absmax", "out", "blocksize"],
        "matmul_4bit": ["A", "B", "quant_state", "bias", "compute_dtype"],
        "matmul_nf4": ["input", "weight_packed", "weight_state", "bias"],
        "matmul_int8": ["A", "B", "A_scales", "B_scales", "dtype"],
        "matmul_fp8_e4m3": ["input", "weight", "weight_scales", "bias", "dtype"],
        "matmul_colrow": ["input", "weight_int8", "weight_row_scales", "weight_col_scales", "bias", "dtype"],
        "double_quant": ["A", "col_stats", "row_stats", "out_col", "out_row", "threshold"],
        "quantize_blockwise": ["A", "code", "absmax", "out", "blocksize", "nested"],
        "dequantize_blockwise": ["A", "quant_state", "absmax", "code", "out", "blocksize", "nested"],
        "dequant_absmax": ["absmax_quant", "absmax_scales", "blocksize"],
        "quantize_rowwise": ["tensor"], "dequantize_rowwise": ["quantized", "scales", "dtype"],
        "quantize_colrow": ["tensor"], "dequantize_colrow": ["quantized", "row_scales", "col_scales", "dtype"],
        "quantize_fp8_e4m3": ["tensor"], "dequantize_fp8_e4m3": ["quantized", "scales", "dtype"],
    }
    for name, params in ref_signatures.items():
        assert list(inspect.signature(getattr(bnb, name)).parameters) == params, name
    for name in ("Linear4bit", "Linear8bit", "LinearFP8", "QuantState", "NF4_CODEBOOK", "FP4_CODEBOOK"):
        assert hasattr(bnb, name)
    assert bnb.NF4_CODEBOOK[7] == 0 and bnb.FP4_CODEBOOK[3] == 0.25


def test_cpu_tensors_are_rejected_not_silently_computed():
    w = torch.randn(8, 64)
    with pytest.raises(ValueError, match="cuda"):
        bnb.quantize_4bit(w)
    with pytest.raises(ValueError, match="quant_type must be"):
        bnb.quantize_4bit(w, quant_type="int3")
    with pytest.raises(ValueError, match="cuda"):
        bnb.quantize_rowwise(w)
    with pytest.raises(ValueError, match="Input must be 2D"):
        bnb.quantize_fp8_e4m3(torch.randn(4))


def test_quant_state_dict_round_trip():
    qs = bnb.QuantState(absmax=torch.ones(4, dtype=torch.int8), shape=torch.Size([2, 128]), quant_type="fp4",
                        dtype=torch.bfloat16, state2=bnb.QuantState(absmax=torch.ones(1), shape=torch.Size([4]),
                                                                    blocksize=256, quant_type="int8", dtype=torch.float32))
    d = qs.as_dict()
    assert set(d) == {"absmax", "shape", "blocksize", "quant_type", "dtype", "state2"}
    back = bnb.QuantState.from_dict(d)
    assert back.quant_type == "fp4" and back.state2.blocksize == 256 and back.dtype == torch.bfloat16
    assert torch.equal(back.code, bnb.FP4_CODEBOOK)
