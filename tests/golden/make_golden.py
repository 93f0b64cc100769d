"""Generate the golden fixtures in this folder by RUNNING THE REFERENCE ITSELF.

Usage (only where the reference checkout is available; it is pure Python + torch CPU):

    python tests/golden/make_golden.py /path/to/mps-bitsandbytes [--only-modules]

(``--only-modules`` rewrites just ``golden_modules.npz`` and the ``ref_*.pt`` checkpoints.)

It imports ``mps_bitsandbytes.functional`` from that path (the native extension is
absent off macOS, so every call takes the reference's pure-PyTorch CPU code), feeds it
seeded inputs and stores inputs and outputs in ``golden_*.npz``; the module section also has
the reference write real checkpoints (``ref_*.pt``: ``state_dict()`` of its Linear4bit /
Linear8bit / Embedding4bit through ``torch.save``), which the drop-in modules must load.  The fixtures pin the
numpy/C oracles (``tests/test_oracle_golden.py``) and, through them and directly, the
CUDA kernels (``tests/test_gpu_*.py``).  bf16 tensors are stored as float32 (exact).

It also checks, against torch's CPU ``log2``, the integer rule the oracle uses for the
FP8 exponent, and prints the result.
"""
import sys
import warnings

import numpy as np
import torch

OUT = __file__.rsplit("/", 1)[0]
DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def npy(t):
    if t.dtype == torch.bfloat16:
        return t.float().numpy()
    return t.numpy()


def main(ref_path):
    sys.path.insert(0, ref_path)
    warnings.simplefilter("ignore")
    import mps_bitsandbytes.functional as F
    from mps_bitsandbytes.nn import Linear4bit, Linear8bit, LinearFP8

    # ------------------------------------------------------------------ 4-bit
    g = {}
    cases = []
    shapes = [(32, 256), (7, 13), (128, 127), (1, 1), (3, 17), (1, 1024), (5, 65), (16, 192)]
    seed = 0
    for qt in ("nf4", "fp4"):
        for dt in ("float16", "bfloat16", "float32"):
            for shp in shapes:
                for bs, dq in ((64, False), (64, True), (32, False), (128, True), (256, False)):
                    if dt != "float16" and (bs != 64 or shp not in ((32, 256), (7, 13))):
                        continue
                    seed += 1
                    torch.manual_seed(seed)
                    scale = [0.02, 1.0, 37.0][seed % 3]
                    w = (torch.randn(*shp) * scale).to(DT[dt])
                    packed, st = F.quantize_4bit(w, blocksize=bs, compress_statistics=dq, quant_type=qt)
                    deq = F.dequantize_4bit(packed, st)
                    name = f"q4_{len(cases)}"
                    cases.append((name, qt, dt, shp[0], shp[1], bs, int(dq)))
                    g[name + "_w"] = npy(w)
                    g[name + "_packed"] = packed.numpy()
                    g[name + "_absmax"] = st.absmax.numpy()
                    if dq:
                        g[name + "_absmax2"] = st.state2.absmax.numpy()
                    g[name + "_deq"] = npy(deq)
    g["cases"] = np.array(cases, dtype=str)

    # known-answer blocks (ties and extremes)
    kat = torch.zeros(1, 64)
    kat[0, :6] = torch.tensor([1, .03125, -.03125, .875, -.875, -.09375])
    p, st = F.quantize_4bit(kat.half(), quant_type="fp4")
    g["kat_fp4_in"] = kat.half().numpy(); g["kat_fp4_packed"] = p.numpy()
    kat2 = torch.zeros(1, 64); kat2[0, :2] = torch.tensor([1.0, -1.0])
    p, st = F.quantize_4bit(kat2.half(), quant_type="nf4")
    g["kat_nf4_in"] = kat2.half().numpy(); g["kat_nf4_packed"] = p.numpy()
    # special inputs: zeros, one non-zero, tiny, fp16 max
    for nm, t in (("zeros", torch.zeros(4, 128)), ("one", torch.zeros(4, 128).index_put((torch.tensor([2]), torch.tensor([77])), torch.tensor(3.5))),
                  ("tiny", torch.full((2, 64), 1e-38)), ("max", torch.full((2, 64), 65504.0))):
        src = t.half() if nm != "tiny" else t.float()
        for qt in ("nf4", "fp4"):
            p, st = F.quantize_4bit(src, quant_type=qt)
            g[f"sp_{nm}_{qt}_in"] = src.numpy(); g[f"sp_{nm}_{qt}_packed"] = p.numpy()
            g[f"sp_{nm}_{qt}_absmax"] = st.absmax.numpy(); g[f"sp_{nm}_{qt}_deq"] = F.dequantize_4bit(p, st).numpy()
    # flat (non 2-D) path
    torch.manual_seed(999)
    v = torch.randn(1000).half()
    p, st = F.quantize_4bit(v, quant_type="nf4")
    g["flat_in"] = v.numpy(); g["flat_packed"] = p.numpy(); g["flat_absmax"] = st.absmax.numpy()
    g["flat_deq"] = F.dequantize_4bit(p, st).numpy()
    v3 = torch.randn(3, 5, 24).half()
    p, st = F.quantize_4bit(v3, quant_type="fp4", blocksize=32)
    g["flat3_in"] = v3.numpy(); g["flat3_packed"] = p.numpy(); g["flat3_absmax"] = st.absmax.numpy()
    g["flat3_deq"] = F.dequantize_4bit(p, st).numpy()
    np.savez_compressed(f"{OUT}/golden_4bit.npz", **g)

    # ------------------------------------------------------------------ int8 family
    g = {}
    torch.manual_seed(11)
    a = torch.randn(5000) * 3
    for bs in (256, 4096, 64):
        q, st = F.quantize_blockwise(a, blocksize=bs)
        g[f"bw{bs}_in"] = a.numpy(); g[f"bw{bs}_q"] = q.numpy(); g[f"bw{bs}_absmax"] = st.absmax.numpy()
        g[f"bw{bs}_deq"] = F.dequantize_blockwise(q, st).numpy()
    x = torch.tensor([[127, .5, 1.5, 2.5, -.5, -1.5]])
    q, s = F.quantize_rowwise(x)
    g["kat_row_in"] = x.numpy(); g["kat_row_q"] = q.numpy(); g["kat_row_s"] = s.numpy()
    torch.manual_seed(12)
    for dt in ("float16", "bfloat16", "float32"):
        x = (torch.randn(48, 96) * 2).to(DT[dt])
        x[5] = 0
        q, s = F.quantize_rowwise(x)
        g[f"row_{dt}_in"] = npy(x); g[f"row_{dt}_q"] = q.numpy(); g[f"row_{dt}_s"] = s.numpy()
        for od in ("float16", "bfloat16", "float32"):
            g[f"row_{dt}_deq_{od}"] = npy(F.dequantize_rowwise(q, s, DT[od]))
    x = (torch.randn(40, 72) * 0.3).half()
    oc, orow, cs, rs, _ = F.double_quant(x)
    g["dq_in"] = x.numpy(); g["dq_col"] = oc.numpy(); g["dq_row"] = orow.numpy(); g["dq_cs"] = cs.numpy(); g["dq_rs"] = rs.numpy()
    q, r, c = F.quantize_colrow(x)
    g["cr_q"] = q.numpy(); g["cr_r"] = r.numpy(); g["cr_c"] = c.numpy()
    g["cr_deq"] = F.dequantize_colrow(q, r, c, torch.float16).numpy()
    g["cr_deq_bf16"] = npy(F.dequantize_colrow(q, r, c, torch.bfloat16))
    # exact half-way cases: x = s * (j + 0.5) / 127 decides between 127.0/s computed as one
    # division or as reciprocal * 127 (torch does the latter for scalar / tensor)
    rng = np.random.default_rng(13)
    svals = rng.uniform(0.01, 50.0, 64).astype(np.float32)
    ties = np.stack([np.concatenate([[sv], (sv * (np.arange(127) + 0.5) / 127.0)]) for sv in svals]).astype(np.float32)
    tt = torch.from_numpy(ties)
    q, s_ = F.quantize_rowwise(tt)
    g["ties_in"] = ties; g["ties_q"] = q.numpy(); g["ties_s"] = s_.numpy()
    qb, stb = F.quantize_blockwise(tt.flatten(), blocksize=128)
    g["ties_bw_q"] = qb.numpy(); g["ties_bw_absmax"] = stb.absmax.numpy()
    g["ties_bw_deq"] = F.dequantize_blockwise(qb, stb).numpy()
    qc, rr, cc = F.quantize_colrow(tt)
    g["ties_cr_q"] = qc.numpy(); g["ties_cr_deq"] = F.dequantize_colrow(qc, rr, cc, torch.float32).numpy()
    oc, orow, cs, rs, _ = F.double_quant(tt)
    g["ties_dq_col"] = oc.numpy(); g["ties_dq_row"] = orow.numpy()
    np.savez_compressed(f"{OUT}/golden_int8.npz", **g)

    # ------------------------------------------------------------------ FP8 E4M3
    g = {}
    kat = torch.tensor([[448, 300, 256, 255, 240, 1.97, 1, .5, 2.0 ** -6, 2.0 ** -7, 0, -448]])
    c8, s8 = F.quantize_fp8_e4m3(kat)
    g["kat_in"] = kat.numpy(); g["kat_codes"] = c8.numpy(); g["kat_scales"] = s8.numpy()
    # all 256 codes decoded
    allc = torch.arange(256, dtype=torch.uint8).view(1, 256)
    g["decode_all"] = F.dequantize_fp8_e4m3(allc, torch.ones(1), torch.float32).numpy()
    g["decode_all_f16"] = F.dequantize_fp8_e4m3(allc, torch.tensor([0.0371]), torch.float16).numpy()
    # encoder on normalised values near every power of two (scale == 1 because rowmax is 448)
    vals = [448.0]
    for e in range(-9, 9):
        p2 = np.float32(2.0 ** e)
        for k in range(-4, 5):
            vals.append(float(np.float32(p2) + k * np.spacing(np.float32(p2)) * (1 if k >= 0 else 0.5)))
    for m in range(8):
        for e in (-3, 0, 4):
            base = (1 + m / 8) * 2.0 ** e
            step = 2.0 ** e / 16
            for k in (-2, -1, 0, 1, 2):
                vals.append(float(np.float32(base + step + k * np.spacing(np.float32(base + step)))))
    t = torch.tensor([vals + [-v for v in vals]], dtype=torch.float32)
    c8, s8 = F.quantize_fp8_e4m3(t)
    assert float(s8[0]) == 1.0
    g["edge_in"] = t.numpy(); g["edge_codes"] = c8.numpy()
    torch.manual_seed(21)
    for dt in ("float16", "bfloat16", "float32"):
        x = (torch.randn(24, 160) * 0.02).to(DT[dt])
        x[3] = 0
        c8, s8 = F.quantize_fp8_e4m3(x)
        g[f"rnd_{dt}_in"] = npy(x); g[f"rnd_{dt}_codes"] = c8.numpy(); g[f"rnd_{dt}_scales"] = s8.numpy()
        g[f"rnd_{dt}_deq"] = npy(F.dequantize_fp8_e4m3(c8, s8, DT[dt] if dt != "float32" else torch.float16))
    np.savez_compressed(f"{OUT}/golden_fp8.npz", **g)

    # exponent rule: floor(log2(a)) in fp32 == integer rule of oracle_np._fp8_exponent
    sys.path.insert(0, OUT + "/../..")
    from oracle import oracle_np as O
    probe = []
    for e in range(-20, 12):
        p2 = np.float32(2.0 ** e)
        for k in range(1, 6):
            x = p2
            for _ in range(k):
                x = np.nextafter(x, np.float32(0))
            probe.append(x)
        probe += [p2, np.nextafter(p2, np.float32(1e9))]
    rng = np.random.default_rng(5)
    probe = np.concatenate([np.array(probe, np.float32),
                            np.exp2(rng.uniform(-12, 9, 2_000_000)).astype(np.float32)])
    ref_e = torch.floor(torch.log2(torch.from_numpy(probe))).to(torch.int32).numpy()
    mine = O._fp8_exponent(probe)
    print("fp8 exponent rule mismatches vs torch.log2:", int((ref_e != mine).sum()), "of", probe.size)

    # ------------------------------------------------------------------ larger unsaved cross-check
    torch.manual_seed(77)
    big = torch.randn(512, 2048) * 0.02
    bad = 0
    for qt in ("nf4", "fp4"):
        p_, st_ = F.quantize_4bit(big.half(), compress_statistics=True, quant_type=qt)
        op, oa, oa2 = O.quantize_4bit(big.half().numpy(), 64, qt, True)
        bad += int((op != p_.numpy()).sum()) + int((oa != st_.absmax.numpy()).sum()) + int((oa2 != st_.state2.absmax.numpy()).sum())
        bad += int((O.dequantize_4bit(op, oa, (512, 2048), 64, qt, "float16", oa2) != F.dequantize_4bit(p_, st_).numpy()).sum())
    q_, s_ = F.quantize_rowwise(big); oq, os_ = O.quantize_rowwise(big.numpy())
    bad += int((oq != q_.numpy()).sum()) + int((os_ != s_.numpy()).sum())
    bad += int((O.dequantize_rowwise(oq, os_, "float16") != F.dequantize_rowwise(q_, s_).numpy()).sum())
    q_, r_, c_ = F.quantize_colrow(big); oq, or_, oc_ = O.quantize_colrow(big.numpy())
    bad += int((oq != q_.numpy()).sum())
    bad += int((O.dequantize_colrow(oq, or_, oc_, "float16") != F.dequantize_colrow(q_, r_, c_).numpy()).sum())
    c_, s_ = F.quantize_fp8_e4m3(big); oc8, os8 = O.quantize_fp8_e4m3(big.numpy())
    bad += int((oc8 != c_.numpy()).sum()) + int((os8 != s_.numpy()).sum())
    bad += int((O.dequantize_fp8_e4m3(oc8, os8, "float16") != F.dequantize_fp8_e4m3(c_, s_).numpy()).sum())
    print("oracle vs reference on 512x2048 (4-bit, rowwise, colrow, fp8): mismatching elements =", bad)
    # torch's CPU sqrt is not correctly rounded when torch is built with MKL's vector maths
    # (about 0.6 % of inputs are one ulp low on x86); the oracle uses the IEEE sqrt.  The only
    # op it touches is the col+row scale sqrt(r*c): rare one-ulp differences in the fp32
    # dequantised value, which the col+row parity tests allow for.
    probe = torch.rand(1_000_000) * 100
    print("torch.sqrt != IEEE sqrt on", int((torch.sqrt(probe).numpy() != np.sqrt(probe.numpy())).sum()), "of 1000000 inputs")

    # ------------------------------------------------------------------ matmuls (tolerance checks)
    g = {}
    torch.manual_seed(31)
    for i, (M, N, K, qt, dq, bias, dt) in enumerate([
            (1, 64, 256, "nf4", False, False, "float16"), (5, 48, 320, "fp4", True, True, "float16"),
            (16, 33, 127, "nf4", True, True, "bfloat16"), (40, 64, 128, "nf4", False, True, "float16"),
            (130, 96, 192, "fp4", False, False, "float16")]):
        w = (torch.randn(N, K) * 0.02).to(DT[dt]); x = torch.randn(M, K).to(DT[dt])
        b = torch.randn(N).to(DT[dt]) if bias else None
        p, st = F.quantize_4bit(w, compress_statistics=dq, quant_type=qt)
        y = F.matmul_4bit(x, p, st, b)
        g[f"mm4_{i}_w"] = npy(w); g[f"mm4_{i}_x"] = npy(x); g[f"mm4_{i}_y"] = npy(y)
        if bias: g[f"mm4_{i}_b"] = npy(b)
        g[f"mm4_{i}_meta"] = np.array([M, N, K, qt, int(dq), int(bias), dt], dtype=str)
    g["mm4_n"] = np.array(5)
    A = torch.randn(24, 96).half(); B = (torch.randn(96, 40) * 0.02).half()
    Aq, As = F.quantize_rowwise(A); Bq_t, Bs = F.quantize_rowwise(B.T.contiguous())
    Bq = Bq_t.T.contiguous()
    g["i8_A"] = A.numpy(); g["i8_B"] = B.numpy(); g["i8_Aq"] = Aq.numpy(); g["i8_As"] = As.numpy()
    g["i8_Bq"] = Bq.numpy(); g["i8_Bs"] = Bs.numpy(); g["i8_y"] = F.matmul_int8(Aq, Bq, As, Bs).numpy()
    W = (torch.randn(40, 96) * 0.02).half(); bb = torch.randn(40).half()
    q, r, c = F.quantize_colrow(W)
    g["cr_W"] = W.numpy(); g["cr_b"] = bb.numpy(); g["cr_y"] = F.matmul_colrow(A, q, r, c, bb).numpy()
    c8, s8 = F.quantize_fp8_e4m3(W)
    g["f8_y"] = F.matmul_fp8_e4m3(A, c8, s8, bb).numpy()
    # modules
    torch.manual_seed(41)
    lin = torch.nn.Linear(128, 48).half()
    xin = torch.randn(2, 3, 128).half()
    g["mod_w"] = lin.weight.data.numpy(); g["mod_b"] = lin.bias.data.numpy(); g["mod_x"] = xin.numpy()
    g["mod_l4_nf4"] = Linear4bit.from_linear(lin, quant_type="nf4", compress_statistics=True)(xin).detach().numpy()
    g["mod_l4_fp4"] = Linear4bit.from_linear(lin, quant_type="fp4")(xin).detach().numpy()
    g["mod_l8"] = Linear8bit.from_linear(lin)(xin).detach().numpy()
    g["mod_f8"] = LinearFP8.from_linear(lin)(xin).detach().numpy()
    np.savez_compressed(f"{OUT}/golden_matmul.npz", **g)
    modules(ref_path)
    print("golden fixtures written to", OUT)


def modules(ref_path):
    """Embeddings, the outlier-aware linear, the model-level helpers and on-disk checkpoints."""
    if ref_path not in sys.path:
        sys.path.insert(0, ref_path)
    warnings.simplefilter("ignore")
    import mps_bitsandbytes as ref
    from mps_bitsandbytes.nn import (Embedding4bit, Embedding8bit, EmbeddingFP4, Linear4bit, Linear8bit,
                                     OutlierAwareLinear)
    g = {}
    # ---- embeddings: (name, V, D, blocksize, quant_type, dtype, padding_idx)
    torch.manual_seed(51)
    ecases = [("e0", 50, 128, 64, "nf4", "float16", 3), ("e1", 37, 96, 32, "fp4", "float16", None),
              ("e2", 20, 256, 64, "nf4", "bfloat16", 0), ("e3", 11, 64, 64, "fp4", "float32", None)]
    for name, V, D, bs, qt, dt, pad in ecases:
        emb = torch.nn.Embedding(V, D, padding_idx=pad).to(DT[dt])
        emb.weight.data.mul_(0.3)
        ids = torch.randint(0, V, (3, 7))
        if pad is not None:
            ids[0, 2] = pad; ids[2, 5] = pad
        e4 = Embedding4bit.from_embedding(emb, quant_type=qt, blocksize=bs)
        e8 = Embedding8bit.from_embedding(emb)
        g[name + "_w"] = npy(emb.weight.data); g[name + "_ids"] = ids.numpy()
        g[name + "_packed"] = e4.weight_packed.numpy(); g[name + "_absmax"] = e4.weight_absmax.numpy()
        g[name + "_out4"] = npy(e4(ids)); g[name + "_q8"] = e8.weight_int8.numpy(); g[name + "_s8"] = e8.weight_scales.numpy()
        g[name + "_out8"] = npy(e8(ids))
    g["ecases"] = np.array([[str(v) for v in c] for c in ecases], dtype=str)
    e4 = EmbeddingFP4.from_embedding(torch.nn.Embedding(9, 64).half())
    assert e4.quant_type == "fp4"
    # ---- outlier-aware linear: (name, M, N, K, dtype, bias, outlier columns planted in W, in x)
    torch.manual_seed(52)
    ocases = [("o0", 6, 40, 96, "float16", True, 3), ("o1", 5, 24, 64, "float16", False, 0),
              ("o2", 9, 32, 128, "bfloat16", True, 5), ("o3", 130, 72, 200, "float16", True, 4)]
    for name, M, N, K, dt, bias, nout in ocases:
        lin = torch.nn.Linear(K, N, bias=bias)
        lin.weight.data.mul_(0.2)
        cols = torch.randperm(K)[:nout]
        lin.weight.data[:, cols] *= 12.0
        lin = lin.to(DT[dt])
        layer = OutlierAwareLinear.from_linear(lin, threshold=6.0)
        assert len(layer.outlier_indices) == nout, (name, len(layer.outlier_indices))
        x = torch.randn(2, M, K)
        x[..., cols] *= 20.0
        x = x.to(DT[dt])
        g[name + "_w"] = npy(lin.weight.data); g[name + "_x"] = npy(x)
        if bias: g[name + "_b"] = npy(lin.bias.data)
        g[name + "_q"] = layer.weight_int8.numpy(); g[name + "_s"] = layer.weight_scales.numpy()
        g[name + "_idx"] = layer.outlier_indices.numpy(); g[name + "_ow"] = npy(layer.outlier_weights)
        g[name + "_y"] = npy(layer(x))
    g["ocases"] = np.array([[str(v) for v in c] for c in ocases], dtype=str)
    # fp32 activations into an fp16 layer (the row-wise quantiser then sees fp32 values)
    lin = torch.nn.Linear(64, 16).half()
    lin.weight.data[:, 7] *= 30
    layer = OutlierAwareLinear.from_linear(lin)
    x32 = torch.randn(4, 64)
    g["o32_w"] = lin.weight.data.numpy(); g["o32_b"] = lin.bias.data.numpy(); g["o32_x"] = x32.numpy()
    g["o32_idx"] = layer.outlier_indices.numpy(); g["o32_y"] = layer(x32).numpy()
    # ---- model-level helpers on a small two-block model
    torch.manual_seed(53)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = torch.nn.Linear(64, 64)
            self.mlp = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 64))
            self.norm = torch.nn.LayerNorm(64)

        def forward(self, h):
            return self.norm(h + self.mlp(self.q_proj(h)))

    class Toy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = torch.nn.Embedding(30, 64)
            self.layers = torch.nn.ModuleList([Block(), Block()])
            self.lm_head = torch.nn.Linear(64, 30, bias=False)

        def forward(self, ids):
            h = self.embed(ids)
            for layer in self.layers:
                h = layer(h)
            return self.lm_head(h)

    torch.manual_seed(55)
    base = Toy().half()
    ids = torch.randint(0, 30, (2, 5))
    g["toy_ids"] = ids.numpy()
    for k_, v_ in base.state_dict().items():
        g["toy_sd_" + k_] = v_.numpy()
    g["toy_keys"] = np.array(list(base.state_dict().keys()), dtype=str)
    import copy
    m4 = ref.quantize_model(copy.deepcopy(base), ref.BitsAndBytesConfig(load_in_4bit=True, bnb_4bit_quant_type="fp4"),
                            device="cpu", modules_to_not_convert=["lm_head"])
    g["toy_y4"] = m4(ids).detach().numpy()
    g["toy_types4"] = np.array([f"{n}:{type(m).__name__}" for n, m in m4.named_modules() if "Linear" in type(m).__name__], dtype=str)
    fp = ref.get_memory_footprint(m4)
    g["toy_fp4"] = np.array([fp["total_params"], fp["quantized_params"], fp["fp16_size_gb"], fp["actual_size_gb"]], dtype=np.float64)
    m8 = ref.quantize_model(copy.deepcopy(base), load_in_8bit=True, device="cpu")
    g["toy_y8"] = m8(ids).detach().numpy()
    g["toy_types8"] = np.array([f"{n}:{type(m).__name__}" for n, m in m8.named_modules() if "Linear" in type(m).__name__], dtype=str)
    fp = ref.get_memory_footprint(m8)
    g["toy_fp8"] = np.array([fp["total_params"], fp["quantized_params"], fp["fp16_size_gb"], fp["actual_size_gb"]], dtype=np.float64)
    cfg = ref.BitsAndBytesConfig(load_in_4bit=True, bnb_4bit_compute_dtype=torch.bfloat16, llm_int8_skip_modules=["lm_head"])
    g["cfg_dict"] = np.array([f"{k}={v}" for k, v in cfg.to_dict().items()], dtype=str)
    back = ref.BitsAndBytesConfig.from_dict(cfg.to_dict())
    g["cfg_back_dtype"] = np.array(str(back.bnb_4bit_compute_dtype))
    g["cfg_method"] = np.array([cfg.quantization_method, ref.BitsAndBytesConfig(load_in_8bit=True).quantization_method,
                                ref.BitsAndBytesConfig().quantization_method], dtype=str)
    # ---- a Hugging Face model (random-init tiny Llama; no checkpoint is involved) through quantize_model
    try:
        from transformers import LlamaConfig, LlamaForCausalLM
        hcfg = LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
        torch.manual_seed(57)
        hf = LlamaForCausalLM(hcfg).half().eval()
        hids = torch.randint(0, 96, (2, 9))
        g["hf_ids"] = hids.numpy()
        g["hf_keys"] = np.array(list(hf.state_dict().keys()), dtype=str)
        for k_, v_ in hf.state_dict().items():
            g["hf_sd_" + k_] = v_.numpy()
        with torch.no_grad():
            h4 = ref.quantize_model(copy.deepcopy(hf), ref.BitsAndBytesConfig(load_in_4bit=True), device="cpu",
                                    modules_to_not_convert=["lm_head"])
            g["hf_y4"] = h4(hids).logits.numpy()
            g["hf_n4"] = np.array(sum(type(m).__name__ == "Linear4bit" for m in h4.modules()))
            h8 = ref.quantize_model(copy.deepcopy(hf), load_in_8bit=True, device="cpu")
            g["hf_y8"] = h8(hids).logits.numpy()
            g["hf_n8"] = np.array(sum(type(m).__name__ == "Linear8bit" for m in h8.modules()))
    except ImportError:
        print("transformers not importable: Hugging Face fixture skipped")
    # ---- checkpoints written by the reference
    torch.manual_seed(56)
    lin = torch.nn.Linear(128, 48).half()
    xin = torch.randn(4, 128).half()
    l4 = Linear4bit.from_linear(lin, quant_type="nf4", compress_statistics=True)
    torch.save(l4.state_dict(), f"{OUT}/ref_linear4bit_nf4_dq.pt")
    l4b = Linear4bit.from_linear(lin, quant_type="fp4", blocksize=32)
    torch.save(l4b.state_dict(), f"{OUT}/ref_linear4bit_fp4_bs32.pt")
    l8 = Linear8bit.from_linear(lin)
    torch.save(l8.state_dict(), f"{OUT}/ref_linear8bit.pt")
    emb = torch.nn.Embedding(40, 128).half()
    e4 = Embedding4bit.from_embedding(emb)
    torch.save(e4.state_dict(), f"{OUT}/ref_embedding4bit.pt")
    eids = torch.randint(0, 40, (6,))
    g["ck_x"] = xin.numpy(); g["ck_l4"] = l4(xin).detach().numpy(); g["ck_l4b"] = l4b(xin).detach().numpy()
    g["ck_l8"] = l8(xin).detach().numpy(); g["ck_eids"] = eids.numpy(); g["ck_e4"] = e4(eids).numpy()
    g["ck_l4_deq"] = l4.dequantize().numpy()
    np.savez_compressed(f"{OUT}/golden_modules.npz", **g)
    print("module fixtures written")


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    if not args:
        sys.exit("usage: make_golden.py <path to a checkout of mps-bitsandbytes v0.7.0> [--only-modules]")
    path = args[0]
    if "--only-modules" in sys.argv:
        modules(path)
    else:
        main(path)
