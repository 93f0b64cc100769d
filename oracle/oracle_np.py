"""CPU oracle for the blockwise quantize -> dequantize -> matmul path (numpy).

TEST INFRASTRUCTURE ONLY.  This file restates, in plain numpy, the arithmetic of the
reference's pure-PyTorch CPU path (``mps_bitsandbytes/functional.py``) so that the CUDA
kernels can be checked bit-for-bit (codes, absmax, dequantised values) and within
tolerance (matmuls).  Nothing in the shipped package imports it; only the tests, the
smoke check and the benchmark's CPU-baseline leg do, and only as the checker.

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the reference itself on
seeded inputs and stores its outputs; ``tests/test_oracle_golden.py`` checks every
function below against those stored outputs.

All arithmetic is IEEE fp32 done in the same order as the reference (torch CPU ops and
numpy ops are both correctly rounded for + - * / sqrt and round-half-even), so results
are reproducible across machines.  The one transcendental, ``log2`` in the FP8 encoder,
is replaced by an exact integer rule (see ``_fp8_exponent``).

bf16 has no numpy dtype: bf16 tensors travel as float32 arrays holding bf16-exact
values, and ``cast_to`` rounds float32 -> bf16 (round-to-nearest-even) on the bits.
"""
from __future__ import annotations

import numpy as np

# mps_bitsandbytes/functional.py:21-26
NF4_CODE = np.array([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0], dtype=np.float32)

# mps_bitsandbytes/functional.py:29-32 (index 8 is -0.0)
FP4_CODE = np.array([
    0.0, 0.0625, 0.125, 0.25, 0.375, 0.5, 0.75, 1.0,
    -0.0, -0.0625, -0.125, -0.25, -0.375, -0.5, -0.75, -1.0], dtype=np.float32)


def codebook(quant_type: str) -> np.ndarray:
    if quant_type == "nf4":
        return NF4_CODE
    if quant_type == "fp4":
        return FP4_CODE
    raise ValueError(f"quant_type must be 'nf4' or 'fp4', got {quant_type}")


# --------------------------------------------------------------------------- dtype helpers
def f32_to_bf16_rne(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bf16 (ties to even), returned as float32 holding the bf16 value."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    nan = np.isnan(x)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    out = (r.astype(np.uint32) << np.uint32(16)).view(np.float32).copy()
    out[nan] = np.nan
    return out.reshape(x.shape)


def cast_to(x32: np.ndarray, dtype: str) -> np.ndarray:
    """Round an fp32 array to 'float16' / 'bfloat16' / 'float32' (torch ``.to(dtype)``)."""
    if dtype == "float16":
        with np.errstate(over="ignore"):
            return x32.astype(np.float16)
    if dtype == "bfloat16":
        return f32_to_bf16_rne(x32)
    if dtype == "float32":
        return x32.astype(np.float32)
    raise ValueError(dtype)


def padded_k(K: int, blocksize: int) -> int:
    """mps_bitsandbytes/functional.py:219-221."""
    kp = ((K + blocksize - 1) // blocksize) * blocksize
    if kp % 2 != 0:
        kp += blocksize
    return kp


def rdiv(c: float, t: np.ndarray) -> np.ndarray:
    """``c / t`` for a Python scalar ``c`` and a tensor ``t`` as torch evaluates it:
    ``Tensor.__rtruediv__`` is ``t.reciprocal() * c`` — two fp32 roundings, not one.
    Every ``127.0 / scale`` of the reference (mps_bitsandbytes/functional.py:518, 621,
    852, 859, 920) goes through it, and it decides round-half-even ties."""
    t = np.asarray(t, dtype=np.float32)
    return ((np.float32(1.0) / t).astype(np.float32) * np.float32(c)).astype(np.float32)


# --------------------------------------------------------------------------- 4-bit
def quantize_4bit(A: np.ndarray, blocksize: int = 64, quant_type: str = "nf4",
                  compress_statistics: bool = False, row_chunk: int = 256):
    """Blockwise 4-bit quantisation (mps_bitsandbytes/functional.py:163-303).

    ``A`` is [N, K] (any float dtype; a non-2-D tensor is passed as [1, numel], which
    is the reference's flat path :257-286).  Per row: zero-pad K to ``padded_k``;
    absmax = max|x| in fp32, clamped to >= 1e-8 (:232); v = x / absmax (:239);
    idx = first index minimising |v - code[i]| in fp32 (:242-243);
    byte = idx[2j] | idx[2j+1] << 4 (:251).

    Returns (packed uint8 [N*Kp/2], absmax, state2): absmax is fp32 [N*nb], or int8
    plus ``state2 = absmax2 fp32 [ceil(N*nb/256)]`` when ``compress_statistics``
    (:288-292).  Rows are processed in chunks: the [rows, nb, bs, 16] difference tensor
    costs 64 B per element.
    """
    code = codebook(quant_type)
    A = np.asarray(A)
    assert A.ndim == 2
    N, K = A.shape
    Kp = padded_k(K, blocksize)
    nb = Kp // blocksize
    packed = np.empty((N, Kp // 2), dtype=np.uint8)
    absmax = np.empty((N, nb), dtype=np.float32)
    for r0 in range(0, N, row_chunk):
        r1 = min(N, r0 + row_chunk)
        blk = np.zeros((r1 - r0, Kp), dtype=np.float32)
        blk[:, :K] = A[r0:r1].astype(np.float32)
        blk = blk.reshape(r1 - r0, nb, blocksize)
        am = np.maximum(np.abs(blk).max(axis=2), np.float32(1e-8)).astype(np.float32)
        v = (blk / am[:, :, None]).astype(np.float32)
        d = np.abs(v[..., None] - code.reshape(1, 1, 1, 16))
        idx = d.argmin(axis=-1).astype(np.uint8).reshape(r1 - r0, Kp)
        packed[r0:r1] = idx[:, 0::2] | (idx[:, 1::2] << 4)
        absmax[r0:r1] = am
    packed = packed.reshape(-1)
    absmax = absmax.reshape(-1)
    if compress_statistics:
        q, absmax2 = quantize_blockwise(absmax, 256)
        return packed, q, absmax2
    return packed, absmax, None


def dequantize_4bit(packed: np.ndarray, absmax: np.ndarray, shape, blocksize: int = 64,
                    quant_type: str = "nf4", dtype: str = "float16",
                    absmax2: np.ndarray | None = None) -> np.ndarray:
    """mps_bitsandbytes/functional.py:306-416.

    Low nibble -> even k, high nibble -> odd k (:360-366); w = code[idx] * absmax in
    fp32 (:375-376); slice to K; round to ``dtype`` (:382).  With ``absmax2`` the int8
    absmax is first expanded by ``dequantize_blockwise`` (:335-337).
    """
    code = codebook(quant_type)
    N, K = shape
    Kp = padded_k(K, blocksize)
    nb = Kp // blocksize
    if absmax2 is not None:
        absmax = dequantize_blockwise(absmax, absmax2, 256)
    absmax = np.asarray(absmax, dtype=np.float32).reshape(N, nb)
    p = np.asarray(packed, dtype=np.uint8).reshape(N, Kp // 2)
    idx = np.empty((N, Kp), dtype=np.uint8)
    idx[:, 0::2] = p & 0x0F
    idx[:, 1::2] = p >> 4
    vals = code[idx].reshape(N, nb, blocksize) * absmax[:, :, None]
    vals = vals.astype(np.float32).reshape(N, Kp)[:, :K]
    return cast_to(np.ascontiguousarray(vals), dtype)


# --------------------------------------------------------------------------- blockwise int8
def quantize_blockwise(A: np.ndarray, blocksize: int = 4096):
    """mps_bitsandbytes/functional.py:469-539: flat, zero-padded to a multiple of
    ``blocksize``; absmax clamp 1e-8 (:515); scale = 127.0 / absmax evaluated as reciprocal * 127 (:518, see ``rdiv``);
    q = clamp(round_half_even(a * scale), -127, 127) as int8 (:520)."""
    a = np.asarray(A).astype(np.float32).reshape(-1)
    n = a.size
    nbk = (n + blocksize - 1) // blocksize
    pad = np.zeros(nbk * blocksize, dtype=np.float32)
    pad[:n] = a
    pad = pad.reshape(nbk, blocksize)
    am = np.maximum(np.abs(pad).max(axis=1), np.float32(1e-8)).astype(np.float32)
    scale = rdiv(127.0, am)
    q = np.clip(np.round((pad * scale[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    return q.reshape(-1)[:n].reshape(np.asarray(A).shape), am


def dequantize_blockwise(q: np.ndarray, absmax: np.ndarray, blocksize: int = 4096,
                         dtype: str = "float32") -> np.ndarray:
    """mps_bitsandbytes/functional.py:542-600: a = float(q) * (absmax / 127.0)
    (divide first, :592-593), rounded to ``dtype``."""
    qf = np.asarray(q).astype(np.float32).reshape(-1)
    n = qf.size
    nbk = (n + blocksize - 1) // blocksize
    pad = np.zeros(nbk * blocksize, dtype=np.float32)
    pad[:n] = qf
    scale = (np.asarray(absmax, dtype=np.float32).reshape(-1) / np.float32(127.0)).astype(np.float32)
    out = (pad.reshape(nbk, blocksize) * scale[:, None]).astype(np.float32)
    return cast_to(out.reshape(-1)[:n].reshape(np.asarray(q).shape), dtype)


# --------------------------------------------------------------------------- row-wise int8
def quantize_rowwise(x: np.ndarray):
    """mps_bitsandbytes/functional.py:607-625: per last-dim row s = max|x| clamp 1e-8;
    q = clamp(round(x * rdiv(127.0, s)), +-127); returns (q int8, s fp32)."""
    x = np.asarray(x)
    x2 = x.reshape(-1, x.shape[-1]).astype(np.float32)
    s = np.maximum(np.abs(x2).max(axis=-1), np.float32(1e-8)).astype(np.float32)
    f = rdiv(127.0, s)
    q = np.clip(np.round((x2 * f[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    return q.reshape(x.shape), s


def dequantize_rowwise(q: np.ndarray, s: np.ndarray, dtype: str = "float16") -> np.ndarray:
    """mps_bitsandbytes/functional.py:628-636: float(q) * (s / 127.0) -> dtype."""
    q = np.asarray(q)
    q2 = q.reshape(-1, q.shape[-1]).astype(np.float32)
    f = (np.asarray(s, dtype=np.float32).reshape(-1) / np.float32(127.0)).astype(np.float32)
    return cast_to((q2 * f[:, None]).astype(np.float32).reshape(q.shape), dtype)


def double_quant(A: np.ndarray):
    """mps_bitsandbytes/functional.py:814-863: row- and column-quantised int8 copies and
    their absmax statistics (threshold ignored, no outlier extraction)."""
    a = np.asarray(A).astype(np.float32)
    row = np.maximum(np.abs(a).max(axis=1), np.float32(1e-8)).astype(np.float32)
    col = np.maximum(np.abs(a).max(axis=0), np.float32(1e-8)).astype(np.float32)
    out_row = np.clip(np.round((a * rdiv(127.0, row)[:, None]).astype(np.float32)),
                      -127, 127).astype(np.int8)
    out_col = np.clip(np.round((a * rdiv(127.0, col)[None, :]).astype(np.float32)),
                      -127, 127).astype(np.int8)
    return out_col, out_row, col, row


def quantize_colrow(W: np.ndarray):
    """mps_bitsandbytes/functional.py:896-924: S[n,k] = sqrt(r[n] * c[k]);
    q = clamp(round(W * rdiv(127.0, S)), +-127)."""
    w = np.asarray(W).astype(np.float32)
    r = np.maximum(np.abs(w).max(axis=1), np.float32(1e-8)).astype(np.float32)
    c = np.maximum(np.abs(w).max(axis=0), np.float32(1e-8)).astype(np.float32)
    S = np.sqrt((r[:, None] * c[None, :]).astype(np.float32)).astype(np.float32)
    q = np.clip(np.round((w * rdiv(127.0, S)).astype(np.float32)),
                -127, 127).astype(np.int8)
    return q, r, c


def dequantize_colrow(q: np.ndarray, r: np.ndarray, c: np.ndarray, dtype: str = "float16"):
    """mps_bitsandbytes/functional.py:927-932: float(q) * (S / 127.0) -> dtype."""
    r = np.asarray(r, dtype=np.float32)
    c = np.asarray(c, dtype=np.float32)
    S = np.sqrt((r[:, None] * c[None, :]).astype(np.float32)).astype(np.float32)
    return cast_to((np.asarray(q).astype(np.float32) * (S / np.float32(127.0)).astype(np.float32))
                   .astype(np.float32), dtype)


# --------------------------------------------------------------------------- FP8 E4M3
def _fp8_exponent(a: np.ndarray) -> np.ndarray:
    """floor(log2(a)) as the reference evaluates it in fp32
    (mps_bitsandbytes/functional.py:1128-1129), for finite a > 0.

    A correctly rounded fp32 log2 returns the integer E itself for the few floats just
    below 2^E: with a = 2^E * (1 - k * 2^-24) (k ulps below), log2(a) = E - d_k,
    d_k ~= k * 1.4427 * 2^-24, and the result rounds to E when d_k is under half the
    spacing of fp32 numbers next to E on that side, 2^(j-24) with
    j = ceil(log2 E) - 1 for E > 0 and j = floor(log2 |E|) for E < 0 (never for E = 0).
    So floor() gives E instead of E - 1 for k <= max_k(j) = 0, 1, 2, 5, 11, 22, ...
    ``tests/golden/make_golden.py`` checks this rule against torch's CPU log2.
    """
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32)
    ebits = ((bits >> 23) & 0xFF).astype(np.int32)
    e = ebits - 127
    man = (bits & np.uint32(0x7FFFFF)).astype(np.int64)
    sub = ebits == 0
    # subnormal fp32 inputs lie far below 2^-7: any very negative exponent encodes as zero
    e = np.where(sub, np.int32(-127), e)
    E = (e + 1).astype(np.int64)
    k = np.int64(0x800000) - man                      # ulps below 2^E
    absE = np.maximum(np.abs(E), 1)
    fl = np.floor(np.log2(absE.astype(np.float64))).astype(np.int64)
    ce = np.ceil(np.log2(absE.astype(np.float64))).astype(np.int64)
    j = np.where(E > 0, ce - 1, fl)
    # largest k with -log2(1 - k 2^-24) < 2^(j-24)
    kmax = np.floor((1.0 - np.exp2(-np.exp2(j.astype(np.float64) - 24.0))) * 2.0 ** 24).astype(np.int64)
    kmax = np.where(E == 0, 0, kmax)
    bump = (k <= kmax) & ~sub
    return np.where(bump, e + 1, e).astype(np.int32)


def float_to_fp8_e4m3(n: np.ndarray) -> np.ndarray:
    """mps_bitsandbytes/functional.py:1106-1163, applied to already-normalised values."""
    n = np.ascontiguousarray(n, dtype=np.float32)
    nan = np.isnan(n)
    sign = (n < 0).astype(np.uint8) << 7
    a = np.minimum(np.abs(n), np.float32(448.0)).astype(np.float32)
    zero = a == 0
    a_safe = np.where(zero | nan, np.float32(1.0), a).astype(np.float32)
    e = np.where(zero, 0, _fp8_exponent(a_safe)).astype(np.int32)
    biased = e + 7
    pow2 = np.ldexp(np.float32(1.0), e).astype(np.float32)
    pow2 = np.where(zero, np.float32(1.0), pow2)
    with np.errstate(over="ignore", invalid="ignore"):
        mf = ((a / pow2).astype(np.float32) - np.float32(1.0)).astype(np.float32)
        mb = ((mf * np.float32(8.0)).astype(np.float32) + np.float32(0.5)).astype(np.float32)
    mb = np.clip(np.nan_to_num(mb, nan=0.0), 0, 7).astype(np.uint8)  # trunc toward zero
    normal = sign | (np.clip(biased, 0, 15).astype(np.uint8) << 3) | mb
    res = np.where(zero, sign, normal)
    res = np.where((biased <= 0) & ~zero, sign, res)
    res = np.where(biased >= 15, sign | np.uint8(0x77), res)
    res = np.where(nan, np.uint8(0x7F), res)
    return res.astype(np.uint8)


def quantize_fp8_e4m3(x: np.ndarray):
    """mps_bitsandbytes/functional.py:1086-1103: scale = clamp(rowmax / 448, 1e-12);
    n = clamp(x / scale, +-448); codes = float_to_fp8_e4m3(n)."""
    x = np.asarray(x).astype(np.float32)
    assert x.ndim == 2
    am = np.abs(x).max(axis=1).astype(np.float32)
    scales = np.maximum((am / np.float32(448.0)).astype(np.float32), np.float32(1e-12))
    n = np.clip((x / scales[:, None]).astype(np.float32), np.float32(-448.0), np.float32(448.0))
    return float_to_fp8_e4m3(n), scales.astype(np.float32)


def fp8_e4m3_to_float(codes: np.ndarray) -> np.ndarray:
    """mps_bitsandbytes/functional.py:1178-1216."""
    c = np.asarray(codes, dtype=np.uint8).astype(np.int32)
    sign = (c >> 7) & 1
    exp = (c >> 3) & 0xF
    man = c & 7
    normal = (np.float32(1.0) + man.astype(np.float32) / np.float32(8.0)) * \
        np.ldexp(np.float32(1.0), exp - 7).astype(np.float32)
    subn = (man.astype(np.float32) / np.float32(8.0)) * np.float32(2.0 ** -6)
    res = np.where(exp == 0, subn, normal).astype(np.float32)
    res = np.where((exp == 15) & (man == 7), np.float32(np.nan), res)
    return np.where(sign == 1, -res, res).astype(np.float32)


def dequantize_fp8_e4m3(codes: np.ndarray, scales: np.ndarray, dtype: str = "float16"):
    """mps_bitsandbytes/functional.py:1166-1175: decode * scale[row] -> dtype."""
    f = fp8_e4m3_to_float(codes)
    return cast_to((f * np.asarray(scales, dtype=np.float32)[:, None]).astype(np.float32), dtype)


# --------------------------------------------------------------------------- matmuls
def linear(x: np.ndarray, w: np.ndarray, bias: np.ndarray | None, out_dtype: str) -> np.ndarray:
    """y = x @ w.T (+ bias) with fp32 accumulation, rounded once to ``out_dtype``.

    Stands for ``torch.nn.functional.linear`` on fp16/bf16 operands
    (mps_bitsandbytes/functional.py:767): operands are already rounded to the storage
    dtype, products are accumulated in fp32.  Accumulation order differs from any BLAS,
    hence matmul parity is a tolerance (1e-2), not bit equality.
    """
    y = np.asarray(x, dtype=np.float32) @ np.asarray(w, dtype=np.float32).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32)[None, :]
    return cast_to(y.astype(np.float32), out_dtype)


def matmul_4bit(x, packed, absmax, shape, blocksize=64, quant_type="nf4", w_dtype="float16",
                absmax2=None, bias=None, out_dtype="float16"):
    """mps_bitsandbytes/functional.py:752-773: dequantise the whole weight to its
    original dtype, cast x (and bias) to that dtype, linear, cast to the output dtype."""
    w = dequantize_4bit(packed, absmax, shape, blocksize, quant_type, w_dtype, absmax2)
    xw = cast_to(np.asarray(x, dtype=np.float32), w_dtype)
    b = None if bias is None else cast_to(np.asarray(bias, dtype=np.float32), w_dtype)
    y = linear(xw, w, b, w_dtype)
    return cast_to(np.asarray(y, dtype=np.float32), out_dtype)


def matmul_int8(A_q, B_q, A_s, B_s, dtype="float16"):
    """mps_bitsandbytes/functional.py:788-793: A [M,K] with row scales, B [K,N] with
    per-column scales; both dequantised to ``dtype`` and multiplied."""
    a = dequantize_rowwise(A_q, A_s, dtype)
    b_t = dequantize_rowwise(np.ascontiguousarray(np.asarray(B_q).T), B_s, dtype)  # [N,K]
    return linear(a, b_t, None, dtype)


def matmul_colrow(x, W_q, r, c, bias=None, dtype="float16"):
    """mps_bitsandbytes/functional.py:935-945."""
    w = dequantize_colrow(W_q, r, c, dtype)
    b = None if bias is None else cast_to(np.asarray(bias, dtype=np.float32), dtype)
    return linear(cast_to(np.asarray(x, dtype=np.float32), dtype), w, b, dtype)


def matmul_fp8_e4m3(x, codes, scales, bias=None, dtype="float16"):
    """mps_bitsandbytes/functional.py:796-807."""
    w = dequantize_fp8_e4m3(codes, scales, dtype)
    return linear(cast_to(np.asarray(x, dtype=np.float32), dtype), w, bias, dtype)


# --------------------------------------------------------------------------- embeddings
def mul_in(a: np.ndarray, b: np.ndarray, dtype: str) -> np.ndarray:
    """Elementwise ``a * b`` for operands already rounded to ``dtype``, result rounded to
    ``dtype`` (a torch multiply in float16 / bfloat16: the exact product rounded once)."""
    return cast_to((np.asarray(a, dtype=np.float32) * np.asarray(b, dtype=np.float32)).astype(np.float32), dtype)


def embedding_4bit(indices, packed, absmax, dim: int, blocksize: int = 64, quant_type: str = "nf4",
                   dtype: str = "float16", padding_idx=None) -> np.ndarray:
    """mps_bitsandbytes/nn/embedding.py:111-139 (the Python path): every looked-up row is
    ``dequantize_4bit`` of that row alone (flat path, functional.py:388-416), rows equal to
    ``padding_idx`` are zero.  ``packed`` [V, dim/2], ``absmax`` [V, ceil(dim/blocksize)]."""
    idx = np.asarray(indices)
    p = np.asarray(packed, dtype=np.uint8)
    V = p.shape[0]
    nb = (dim + blocksize - 1) // blocksize
    Kp = padded_k(dim, blocksize)
    full = np.zeros((V, Kp // 2), dtype=np.uint8)
    full[:, :dim // 2] = p[:, :dim // 2]
    table = dequantize_4bit(full, np.asarray(absmax, dtype=np.float32).reshape(V, nb), (V, dim), blocksize, quant_type, dtype)
    out = table[idx.reshape(-1)].reshape(*idx.shape, dim).copy()
    if padding_idx is not None:
        out[idx == padding_idx] = 0
    return out


def embedding_8bit(indices, q, scales, dtype: str = "float16", padding_idx=None) -> np.ndarray:
    """mps_bitsandbytes/nn/embedding.py:266-275: ``q.to(dtype) * (scales / 127.0).to(dtype)``
    (the scale is rounded to ``dtype`` before the multiply), padding rows zero."""
    idx = np.asarray(indices)
    qi = np.asarray(q)[idx]
    s = cast_to((np.asarray(scales, dtype=np.float32)[idx] / np.float32(127.0)).astype(np.float32), dtype)
    out = mul_in(qi.astype(np.float32), np.asarray(s, dtype=np.float32)[..., None], dtype)
    if padding_idx is not None:
        out[idx == padding_idx] = 0
    return out


# --------------------------------------------------------------------------- outlier-aware int8 linear
def outlier_from_linear(weight: np.ndarray, threshold: float = 6.0, dtype: str = "float16"):
    """mps_bitsandbytes/nn/outlier_aware.py:184-207 for a weight already in ``dtype``:
    outlier columns = col_max|w| > threshold * mean|w| (statistics rounded to ``dtype`` as torch
    computes them on a 16-bit tensor: the mean is accumulated in fp32 and rounded once);
    those columns are kept as they are and zeroed before the row-wise int8 quantisation.
    Returns (weight_int8, weight_scales, outlier_indices, outlier_weights)."""
    w = np.asarray(weight, dtype=np.float32)
    col_max = np.abs(w).max(axis=0)
    mean_abs = cast_to(np.array([np.abs(w).astype(np.float64).mean()], dtype=np.float32), dtype)[0]
    limit = cast_to(np.array([np.float32(threshold) * np.float32(mean_abs)], dtype=np.float32), dtype)[0]
    idx = np.where(col_max > np.float32(limit))[0].astype(np.int64)
    w8 = w.copy()
    w8[:, idx] = 0
    q, s = quantize_rowwise(w8)
    return q, s, idx, cast_to(w[:, idx], dtype)


def outlier_linear(x, weight_int8, weight_scales, outlier_idx, outlier_w, bias=None, dtype: str = "float16"):
    """mps_bitsandbytes/nn/outlier_aware.py:84-146.  Main columns: x is quantised row-wise, both
    operands are dequantised as ``q.to(dtype) * (s / 127).to(dtype)`` and multiplied; outlier
    columns: x (cast to ``dtype``) times the 16-bit outlier weights; the two results (each rounded
    to ``dtype``) are added, then the bias is added, each addition rounded to ``dtype``."""
    x = np.asarray(x)
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    idx = np.asarray(outlier_idx, dtype=np.int64)
    mask = np.ones(K, dtype=bool)
    mask[idx] = False
    xq, xs = quantize_rowwise(x2[:, mask])
    xs_t = cast_to((xs / np.float32(127.0)).astype(np.float32), dtype)
    x_fp = mul_in(xq.astype(np.float32), np.asarray(xs_t, dtype=np.float32)[:, None], dtype)
    ws_t = cast_to((np.asarray(weight_scales, dtype=np.float32) / np.float32(127.0)).astype(np.float32), dtype)
    w_fp = mul_in(np.asarray(weight_int8)[:, mask].astype(np.float32), np.asarray(ws_t, dtype=np.float32)[:, None], dtype)
    y = linear(x_fp, w_fp, None, dtype)
    if idx.size:
        y_out = linear(cast_to(x2[:, idx].astype(np.float32), dtype), np.asarray(outlier_w, dtype=np.float32), None, dtype)
        y = cast_to((np.asarray(y, dtype=np.float32) + np.asarray(y_out, dtype=np.float32)).astype(np.float32), dtype)
    if bias is not None:
        y = cast_to((np.asarray(y, dtype=np.float32) + np.asarray(bias, dtype=np.float32)[None, :]).astype(np.float32), dtype)
    return y.reshape(*x.shape[:-1], -1)
