"""CPU: the oracle's restatement of the embedding and outlier-aware modules against outputs of
the reference itself (tests/golden/golden_modules.npz, written by make_golden.py).
Embedding look-ups and the stored quantised tables must be bit-exact; the outlier-aware forward
is a matmul and is held to the matmul bound (max |y - ref| / max |ref| <= 1e-2)."""
import numpy as np

from oracle import oracle_np as O


def rel_err(y, ref):
    y = np.asarray(y, np.float32); ref = np.asarray(ref, np.float32)
    return float(np.abs(y - ref).max() / max(float(np.abs(ref).max()), 1e-30))


def _pad(v):
    return None if v == "None" else int(v)


def test_embedding_tables_and_lookups_bit_exact(golden):
    g = golden("modules")
    for name, V, D, bs, qt, dt, pad in g["ecases"]:
        V, D, bs, pad = int(V), int(D), int(bs), _pad(pad)
        out_dt = dt if dt in ("float16", "bfloat16") else "float16"      # embedding.py:163-165
        w = g[name + "_w"]
        packed, absmax, _ = O.quantize_4bit(w, bs, qt, False)
        assert np.array_equal(packed.reshape(V, -1)[:, :D // 2], g[name + "_packed"])
        assert np.array_equal(absmax.reshape(V, -1), g[name + "_absmax"])
        out4 = O.embedding_4bit(g[name + "_ids"], g[name + "_packed"], g[name + "_absmax"], D, bs, qt, out_dt, pad)
        assert out4.shape == g[name + "_out4"].shape and np.array_equal(out4, g[name + "_out4"]), name
        q8, s8 = O.quantize_rowwise(w)
        assert np.array_equal(q8, g[name + "_q8"]) and np.array_equal(s8, g[name + "_s8"])
        out8 = O.embedding_8bit(g[name + "_ids"], q8, s8, out_dt, pad)
        assert np.array_equal(out8, g[name + "_out8"]), name
        if pad is not None:
            assert not out4[g[name + "_ids"] == pad].any() and not out8[g[name + "_ids"] == pad].any()


def test_outlier_aware_conversion_exact_and_forward_within_bound(golden):
    g = golden("modules")
    for name, M, N, K, dt, bias, nout in g["ocases"]:
        q, s, idx, ow = O.outlier_from_linear(g[name + "_w"], 6.0, dt)
        assert np.array_equal(idx, g[name + "_idx"]) and len(idx) == int(nout)
        assert np.array_equal(q, g[name + "_q"]) and np.array_equal(s, g[name + "_s"])
        assert np.array_equal(ow, g[name + "_ow"])
        b = g[name + "_b"] if bias == "True" else None
        y = O.outlier_linear(g[name + "_x"], q, s, idx, ow, b, dt)
        assert y.shape == g[name + "_y"].shape
        assert rel_err(y, g[name + "_y"]) <= 1e-2, (name, rel_err(y, g[name + "_y"]))
    q, s, idx, ow = O.outlier_from_linear(g["o32_w"], 6.0, "float16")
    assert np.array_equal(idx, g["o32_idx"])
    assert rel_err(O.outlier_linear(g["o32_x"], q, s, idx, ow, g["o32_b"], "float16"), g["o32_y"]) <= 1e-2
