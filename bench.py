"""Benchmark of the fused dequantise-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch M] [--model NAME]
                    [--layers L] [--skip-extras] [--prefill-only] [--int8-only] [--quant-only]

Workload (every N): the Llama-70B-shaped NF4 decode stack of BASELINE config 5 - 80 layers x
{q,o 8192x8192, k,v 1024x8192, gate/up 28672x8192, down 8192x28672}, double-quantised absmax,
fp16, batch 1 - one "step" = one pass over all 560 linears (35.3 GB of packed weights and
absmax, far larger than the 126 MB L2, so every step streams from HBM), by default ONE
cooperative kernel launch.  For N > 1 (launched by torchrun, one rank per GPU) the stack is
N-sharded over the ranks; at each layer boundary every rank stores its shard of the next input
into all ranks' buffers over NVLink and raises flags (--exchange nccl: an NCCL all-gather
instead); the per-GPU work shrinks with N (strong scaling of a fixed model).

Prints ONE JSON line: metric nf4_decode_gbs = algorithmic bytes per step / step time (median of
blocks of --steps steps, repeated until at least a second has been timed), with the HBM
roofline, an end-to-end figure through the public LayerStack API with host buffers, a parity
figure (a reduced-depth instance of the same stack checked against the C oracle before the
timed region), the device status word, a CPU baseline, and further objects: the same stack at
batch 32 (HBM roofline) and batch 512 (tensor roofline), and at N = 1 the Llama-2-7B stack of
BASELINE config 3 at batch 1 and 16, the prefill GEMM of BASELINE config 2 and the INT8 / FP8 /
outlier-split matmuls of BASELINE config 4, each with its own parity figure.

--layers L runs a stack of only L layers (a reduced workload for profiler captures; the JSON
line names it) and --skip-extras leaves out the further objects and the CPU baseline.  The timed
region of the main object is bracketed by cudaProfilerStart/Stop so that a profiler started with
--profile-from-start off sees exactly the timed launches.

--prefill-only / --int8-only / --quant-only run just that object (used for profiler captures).

--impl reference times the reference's CPU algorithm (the C oracle: dequantise the whole
weight, then matmul, as mps_bitsandbytes/functional.py:752-773 does on CPU) on one layer of
the same stack per step, on all host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of one decode launch at batch 1, from a profiler
# capture of a two-layer launch (213.5 MB moved for 209.1 MB of weights, scales and activations); DRAM traffic grows
# in proportion to the units a launch processes, so a full-depth launch moves this ratio times its algorithmic bytes
NCU_TRAFFIC_RATIO_DECODE_B1 = 213.5 / 209.11


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu_index, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# CPU arm: the C oracle on one layer of the stack
# --------------------------------------------------------------------------------------------
def cpu_layer_setup(cfg, M, seed=0):
    import numpy as np
    rng = np.random.default_rng(seed)
    layer = []
    for name, n, k in cfg.projections():
        packed = rng.integers(0, 256, size=n * k // 2, dtype=np.uint8)        # uniformly random codes
        absmax = rng.uniform(0.03, 0.09, size=n * k // 64).astype(np.float32)  # block maxima of N(0, 0.02) data
        x = rng.standard_normal((M, k)).astype(np.float16)
        layer.append((name, n, k, packed, absmax, x, np.empty((n, k), np.float16)))
    return layer


def cpu_threads():
    """All host cores for the CPU arms, whatever OMP_NUM_THREADS the launcher exported (torch.distributed.run sets 1);
    returns the number of threads the C oracle's OpenMP loops will use."""
    from oracle import oracle_c
    return int(oracle_c.lib().o_threads(os.cpu_count() or 1))


def cpu_layer_pass(layer):
    from oracle import oracle_c
    for name, n, k, packed, absmax, x, scratch in layer:
        oracle_c.matmul_4bit_f16(x, packed, absmax, n, k, 64, "nf4", scratch=scratch)


def cpu_baseline(cfg, M, budget_s=12.0):
    """GB/s of the reference CPU algorithm (C port, OpenMP on all cores) on one layer, scaled per byte."""
    from mps_bitsandbytes_b200 import stack as S
    cores = cpu_threads()
    layer = cpu_layer_setup(cfg, M)
    cpu_layer_pass(layer)                                     # warm-up
    best, t_end, reps = float("inf"), time.perf_counter() + budget_s, 0
    while reps < 3 or (time.perf_counter() < t_end and reps < 20):
        t0 = time.perf_counter()
        cpu_layer_pass(layer)
        best = min(best, time.perf_counter() - t0)
        reps += 1
    nbytes = S.algorithmic_bytes(cfg, M, layers=1)           # same byte count per layer as the GPU arm
    return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"1 of {cfg.layers} layers ({nbytes / 1e6:.0f} MB, 7 linears, random codes, absmax already expanded to "
                      f"fp32), best of {reps}, C oracle of functional.py:752-773 with OpenMP"}


def workload_config(cfg, M, layers, world):
    """The `config` object: the same in both arms."""
    from mps_bitsandbytes_b200 import stack as S
    nbytes = S.algorithmic_bytes(cfg, M, layers=layers)
    return {"workload": f"{cfg.name} NF4+DQ decode stack ({layers} layers x 7 Linear4bit), batch {M}, "
                        f"N-sharded over {world} GPU(s)", "batch": M, "layers": layers,
            "l2": f"inputs ({nbytes / 1e9:.2f} GB of weights per step) larger than L2; no flush needed",
            "parallelism": f"n-shard{world}"}


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from mps_bitsandbytes_b200 import stack as S
    cores = cpu_threads()
    layer = cpu_layer_setup(cfg, args.batch)
    for _ in range(max(args.warmup, 1)):
        cpu_layer_pass(layer)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_layer_pass(layer)
    dt = (time.perf_counter() - t0) / args.steps
    nbytes = S.algorithmic_bytes(cfg, args.batch, layers=1)  # same byte count per layer as the GPU arm
    gbs = nbytes / dt / 1e9
    sample = f"each step = 1 of {cfg.layers} layers ({nbytes / 1e6:.0f} MB), C oracle of the reference CPU path, OpenMP"
    print(json.dumps({
        "impl": "reference", "metric": "nf4_decode_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(cfg, args.batch, args.layers or cfg.layers, args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def _rel_err(y, ref):
    """max |y - ref| / max |ref| and max |y - ref| / (|ref| + rms(ref)), the larger one (bound 1e-2)."""
    import numpy as np
    y = np.asarray(y, np.float32); ref = np.asarray(ref, np.float32)
    d = np.abs(y - ref)
    rms = float(np.sqrt(np.mean(np.square(ref.astype(np.float64)))))
    return float(max(d.max() / max(float(np.abs(ref).max()), 1e-30), (d / (np.abs(ref) + max(rms, 1e-30))).max()))


def _event_ms(torch, fn, steps, warmup):
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def prefill_config2(torch, peaks, steps=20, warmup=5):
    """BASELINE config 2: FP4 (double-quantised) 11008 x 4096 weight, x [2048, 4096] fp16.  The weight (45 MB of
    output, 22.5 MB packed, 16.8 MB of x) is touched once per call; calls alternate between two weight/input sets
    so that consecutive timed calls do not find their operands in L2."""
    import numpy as np
    import mps_bitsandbytes_b200 as bnb
    from oracle import oracle_c
    g = torch.Generator(device="cuda"); g.manual_seed(2)
    sets = []
    for _ in range(2):
        w = (torch.randn(11008, 4096, device="cuda", generator=g) * 0.02).half()
        x = torch.randn(2048, 4096, device="cuda", generator=g).half()
        packed, st = bnb.quantize_fp4(w, compress_statistics=True)
        sets.append((x, packed, st))
        del w
    # parity (outside the timed region): 32 sampled rows of x, all 11008 columns, against the C oracle
    x, packed, st = sets[0]
    rows = np.sort(np.random.default_rng(2).choice(2048, 32, replace=False))
    y = bnb.matmul_4bit(x, packed, st)
    am = oracle_c.dequantize_absmax(st.absmax.cpu().numpy(), st.state2.absmax.cpu().numpy())
    ref = oracle_c.matmul_4bit_f16(x.cpu().numpy()[rows], packed.cpu().numpy(), am, 11008, 4096, 64, "fp4")
    parity = _rel_err(y.cpu().numpy()[rows], ref)
    i = [0]

    def call():
        xx, pp, ss = sets[i[0] & 1]; i[0] += 1
        bnb.matmul_4bit(xx, pp, ss)
    ms = _event_ms(torch, call, steps, warmup)
    flops = 2.0 * 2048 * 4096 * 11008
    tf = flops / (ms * 1e-3) / 1e12
    return {"metric": "fp4_prefill_tflops", "value": tf, "unit": "TFLOP/s", "ms": ms, "parity_rel_err": parity,
            "config": {"workload": "FP4+DQ 11008x4096 weight, x [2048,4096] fp16 through matmul_4bit",
                       "l2": "two operand sets alternate (170 MB together, larger than L2)"},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops"], "traffic": None, "peak_source": peaks["source"]}}


def int8_fp8_config4(torch, peaks, steps=10, warmup=3):
    """BASELINE config 4: activations [512, 4096] fp16 with 0.5 % of the columns at magnitude ~20, weight
    4096 x 16384 ~ N(0, 0.02): matmul_int8 (row-wise A, column-wise B), matmul_colrow, matmul_fp8_e4m3 and the
    outlier-aware split (OutlierAwareLinear).  Every figure includes all passes of the call; each case carries its
    parity figure against the numpy oracle (32 sampled rows, all 16384 columns)."""
    import numpy as np
    import mps_bitsandbytes_b200 as bnb
    from oracle import oracle_np as O
    M, K, Nn = 512, 4096, 16384
    g = torch.Generator(device="cuda"); g.manual_seed(4)
    w = (torch.randn(Nn, K, device="cuda", generator=g) * 0.02).half()
    x = torch.randn(M, K, device="cuda", generator=g).half()
    cols = torch.randperm(K, device="cuda", generator=g)[: K // 200]
    x[:, cols] *= 20.0
    w_out = w.clone(); w_out[:, cols] *= 15.0                      # the same columns large in the weight: detected as outliers
    aq, a_s = bnb.quantize_rowwise(x)
    bq_t, b_s = bnb.quantize_rowwise(w)                             # per output column of B = per row of W
    bq = bq_t.t().contiguous()                                      # [K, N], N contiguous
    cq, cr, cc = bnb.quantize_colrow(w)
    f8, f8s = bnb.quantize_fp8_e4m3(w)
    lin = torch.nn.Linear(K, Nn, bias=False, device="cuda", dtype=torch.float16)
    lin.weight.data = w_out
    oal = bnb.OutlierAwareLinear.from_linear(lin)
    del lin, w, w_out, bq_t
    rows = np.sort(np.random.default_rng(4).choice(M, 32, replace=False))
    xs = x.cpu().numpy()[rows]
    n = lambda t: t.cpu().numpy()
    cases = {"matmul_int8": (lambda: bnb.matmul_int8(aq, bq, a_s, b_s),
                             lambda: O.matmul_int8(n(aq)[rows], n(bq), n(a_s)[rows], n(b_s))),
             "matmul_colrow": (lambda: bnb.matmul_colrow(x, cq, cr, cc), lambda: O.matmul_colrow(xs, n(cq), n(cr), n(cc))),
             "matmul_fp8_e4m3": (lambda: bnb.matmul_fp8_e4m3(x, f8, f8s), lambda: O.matmul_fp8_e4m3(xs, n(f8), n(f8s))),
             "outlier_aware_linear": (lambda: oal(x), lambda: O.outlier_linear(xs, n(oal.weight_int8), n(oal.weight_scales),
                                                                                n(oal.outlier_indices), n(oal.outlier_weights),
                                                                                None, "float16"))}
    flops = 2.0 * M * K * Nn
    res = {"config": {"workload": f"x [{M},{K}] fp16 (0.5% outlier columns), weight {K}x{Nn}",
                      "outlier_columns": int(oal.outlier_indices.numel()),
                      "l2": "weight (67 MB) + output (17 MB) + x per call; an L2 flush (256 MB memset) runs between timed calls"},
           "unit": "TFLOP/s", "peak": peaks["bf16_tflops"], "peak_note": "dense bf16 (the MMAs are 16-bit: x stays fp16)"}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name, (fn, ref_fn) in cases.items():
        parity = _rel_err(n(fn())[rows], ref_fn())
        for _ in range(warmup):
            fn()
        tot = 0.0
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        ms = tot / steps
        res[name] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "frac": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
                     "parity_rel_err": parity}
    return res


def quantize_path(torch, peaks, steps=10, warmup=3):
    """The memory-bound ends of the path on BASELINE config 5's largest weight (28672 x 8192 fp16): quantize_4bit
    (NF4 / FP4, plain and double-quantised), dequantize_4bit, and the Embedding4bit / Embedding8bit gathers on a
    128256 x 4096 table with 32768 indices.  GB/s are ALGORITHMIC bytes (16-bit side + packed + scales) over CUDA-event
    time of `steps` calls issued back to back, against the measured HBM copy rate (the median of single calls on an idle
    GPU, which adds the host's time per call, is reported beside it); inputs are larger than L2 and three sets alternate.  Parity is
    bit-exact by construction of the tests; here 64 sampled rows are compared byte for byte with the C oracle."""
    import numpy as np
    import mps_bitsandbytes_b200 as bnb
    from oracle import oracle_c, oracle_np as O
    n, k = 28672, 8192
    g = torch.Generator(device="cuda"); g.manual_seed(5)
    ws = [(torch.randn(n, k, device="cuda", generator=g) * 0.02).half() for _ in range(3)]
    rows = np.sort(np.random.default_rng(5).choice(n, 64, replace=False))
    peak = peaks["hbm_gbs"]
    res = {"config": {"workload": f"weight {n}x{k} fp16, block 64; embeddings 128256x4096, 32768 indices",
                      "l2": "470 MB per weight, three weights alternate: larger than L2"},
           "unit": "GB/s", "peak": peak, "peak_source": peaks.get("source", "measured")}

    def timed(fn, nbytes):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        ts = []
        for i in range(steps):                                      # one call at a time on an idle GPU: the host's
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)   # ~20 us per call show
            e0.record(); fn(i); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        single = sorted(ts)[len(ts) // 2]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):                                      # the same calls back to back (inputs still alternate)
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"ms": ms, "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak, "bytes": nbytes,
                "ms_single_call_idle_gpu": single, "frac_single_call_idle_gpu": nbytes / single / 1e6 / peak}

    nbytes = 2 * n * k + n * k // 2 + 4 * n * k // 64
    for qt in ("nf4", "fp4"):
        o = timed(lambda i: bnb.quantize_4bit(ws[i % 3], quant_type=qt), nbytes)
        p, st = bnb.quantize_4bit(ws[0], quant_type=qt)
        pc, ac = oracle_c.quantize_4bit(ws[0][torch.from_numpy(rows).cuda()].float().cpu().numpy(), 64, qt)
        o["bit_exact"] = bool(np.array_equal(p.view(n, k // 2).cpu().numpy()[rows], pc.reshape(64, k // 2)) and
                              np.array_equal(st.absmax.view(n, k // 64).cpu().numpy()[rows], ac.reshape(64, k // 64)))
        res[f"quantize_4bit_{qt}"] = o
        res[f"quantize_4bit_{qt}_double_quant"] = timed(
            lambda i: bnb.quantize_4bit(ws[i % 3], quant_type=qt, compress_statistics=True), 2 * n * k + n * k // 2 + n * k // 64)
    packs = [bnb.quantize_4bit(w, quant_type="nf4") for w in ws]
    o = timed(lambda i: bnb.dequantize_4bit(*packs[i % 3]), nbytes)
    d = bnb.dequantize_4bit(*packs[0])
    dc = oracle_c.dequantize_4bit(packs[0][0].view(n, k // 2).cpu().numpy()[rows], packs[0][1].absmax.view(n, k // 64).cpu().numpy()[rows],
                                  (64, k), 64, "nf4").astype(np.float16)
    o["bit_exact"] = bool(np.array_equal(d.cpu().numpy()[rows], dc))
    res["dequantize_4bit_nf4"] = o
    del ws, packs, d
    torch.cuda.empty_cache()
    V, D, T = 128256, 4096, 32768
    emb = torch.nn.Embedding(V, D, device="cuda", dtype=torch.float16)
    ids = [torch.randint(0, V, (T,), device="cuda", generator=g) for _ in range(3)]
    for name, mod, rd in (("embedding_4bit", bnb.Embedding4bit.from_embedding(emb), D // 2 + 4 * D // 64),
                          ("embedding_8bit", bnb.Embedding8bit.from_embedding(emb), D + 4)):
        o = timed(lambda i: mod(ids[i % 3]), T * (rd + 2 * D))
        y = mod(ids[0][:64]).cpu().numpy()
        i64 = ids[0][:64].cpu().numpy()
        if name == "embedding_4bit":
            sel = np.unique(i64)
            # the oracle on the looked-up rows only
            ref = O.embedding_4bit(np.searchsorted(sel, i64), mod.weight_packed.cpu().numpy()[sel], mod.weight_absmax.cpu().numpy()[sel], D)
        else:
            ref = O.embedding_8bit(i64, mod.weight_int8.cpu().numpy(), mod.weight_scales.cpu().numpy())
        o["bit_exact"] = bool(np.array_equal(y, np.asarray(ref)))
        res[name] = o
    return res


def oracle_stack_rows(ref_stack, x_rows):
    """The stack's dataflow (stack.py) on the CPU: every linear by the C oracle of the reference's CPU path
    (dequantise the whole weight to fp16, matmul with fp32 accumulation), on the given rows of x, from the packed
    bytes and absmax of an UNSHARDED stack read back from the device.  Checker only; never timed here."""
    import numpy as np
    from oracle import oracle_c
    cfg = ref_stack.cfg
    h = np.ascontiguousarray(x_rows, np.float16)
    for l in range(ref_stack.layers):
        e = np.tile(h, (1, -(-cfg.ffn // cfg.hidden)))[:, :cfg.ffn]
        y = {}
        for pr in ref_stack.proj[l]:
            if pr.name not in ("o", "down"):
                continue                                              # only o and down feed the next layer
            am = pr.absmax.cpu().numpy()
            if pr.absmax2 is not None:
                am = oracle_c.dequantize_absmax(am, pr.absmax2.cpu().numpy())
            xin = e if pr.name == "down" else h
            y[pr.name] = oracle_c.matmul_4bit_f16(xin, pr.packed.cpu().numpy(), am.astype(np.float32), pr.n, pr.k, 64,
                                                  ref_stack.quant_type).astype(np.float32)
        h = (np.float32(ref_stack.alpha) * (y["o"] + y["down"])).astype(np.float16)
    return h


TAGGED = {"auto": None, "tagged": True, "flags": False}


def stack_parity(S, torch, dist, cfg, M, rank, world, local, args, layers=2, sample=4):
    """Reduced-depth instance of the benchmarked stack (same widths, same sharding, same kernels and exchange) run
    once and compared with the C oracle on `sample` rows of the batch.  Returns the parity figure on every rank."""
    import numpy as np
    st = S.LayerStack(cfg, device=f"cuda:{local}", rank=rank, world=world, layers=layers,
                      fused_exchange=args.exchange == "fused", boundary=args.boundary, persistent=not args.per_layer,
                      tagged_exchange=TAGGED[args.handoff])
    st.prepare(M, use_graph=True)
    gen = torch.Generator(device="cpu"); gen.manual_seed(7)
    x = torch.randn(M, cfg.hidden, generator=gen).half()
    h = None
    for _ in range(2):                                                # the second step also checks that state was re-armed
        h = st.step(x.cuda()).float().cpu().numpy()
        torch.cuda.synchronize()
    status = st.check_status()
    err = 0.0
    if rank == 0:
        ref_st = st if world == 1 else S.LayerStack(cfg, device=f"cuda:{local}", rank=0, world=1, layers=layers)
        rows = np.arange(M) if M <= sample else np.sort(np.random.default_rng(M).choice(M, sample, replace=False))
        err = _rel_err(h[rows], oracle_stack_rows(ref_st, x.numpy()[rows]))
        del ref_st
    if world > 1:
        t = torch.tensor([err, float(status)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        err, status = float(t[0]), int(t[1])
    del st
    torch.cuda.empty_cache()
    return err, status


def time_stack(torch, dist, stack, x_dev, steps, warmup, world, min_seconds=1.0, max_blocks=50, profile=False):
    """Blocks of `steps` steps, each block timed with CUDA events on the launching stream, repeated until
    `min_seconds` have been timed; per block the MAX over ranks.  Returns (median, min, max ms per step, blocks)."""
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(max(warmup, 3)):
        stack.step(x_dev)
    barrier()
    blocks = []
    if profile:
        torch.cuda.profiler.start()
    total = 0.0
    # every rank runs the same number of blocks: decided from rank-synchronised times
    while len(blocks) < max_blocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            stack.step()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        blocks.append(ms / steps)
        total += ms * 1e-3
        if total >= min_seconds:
            break
    if profile:
        torch.cuda.profiler.stop()
    return statistics.median(blocks), min(blocks), max(blocks), len(blocks)


def decode_object(S, torch, dist, stack, cfg, M, args, peaks, rank, world, local, main=False):
    """One object of the JSON line: the stack at batch M (prepared here), parity, timing, roofline."""
    parity, pstatus = stack_parity(S, torch, dist, cfg, M, rank, world, local, args)
    stack.prepare(M, use_graph=True)
    gen = torch.Generator(device="cpu"); gen.manual_seed(1)
    x_host = torch.randn(M, cfg.hidden, generator=gen).half().pin_memory()
    x_dev = x_host.cuda()
    steps = args.steps if M <= 32 else max(2, min(args.steps, 5))
    ms, ms_min, ms_max, nblocks = time_stack(torch, dist, stack, x_dev, steps, args.warmup, world,
                                             min_seconds=1.0 if M <= 32 else 0.3, profile=main)
    status = max(pstatus, stack.check_status())
    if world > 1:
        t = torch.tensor([float(status)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        status = int(t[0])
    nbytes = S.algorithmic_bytes(cfg, M, layers=stack.layers)
    gbs = nbytes / (ms * 1e-3) / 1e9
    obj = {"value": gbs, "unit": "GB/s", "ms_per_step": ms, "ms_min": ms_min, "ms_max": ms_max, "blocks": nblocks,
           "steps_per_block": steps, "parity_rel_err": parity, "device_status": status,
           "launches_per_step": stack.launches_per_step()}
    if M <= 32:
        per_gpu = gbs / world
        obj["roofline"] = {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                           "frac": per_gpu / peaks["hbm_gbs"], "peak_source": peaks["source"],
                           "traffic": NCU_TRAFFIC_RATIO_DECODE_B1 * nbytes / world if (M == 1 and stack._persist) else None}
    else:
        flops = 2.0 * M * cfg.params_per_layer() * stack.layers
        tf = flops / (ms * 1e-3) / 1e12
        obj.update({"value": tf, "unit": "TFLOP/s", "gbs": gbs})
        obj["roofline"] = {"bound": "tensor", "achieved": tf / world, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                           "frac": tf / world / peaks["bf16_tflops"], "peak_source": peaks["source"], "traffic": None}
    return obj, x_host, steps * nblocks


def run_gpu(args, cfg):
    import torch
    import torch.distributed as dist
    from mps_bitsandbytes_b200 import stack as S

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = load_peaks()
    M = args.batch
    stack = S.LayerStack(cfg, device=f"cuda:{local}", rank=rank, world=world, layers=args.layers,
                         fused_exchange=args.exchange == "fused", boundary=args.boundary, persistent=not args.per_layer,
                         tagged_exchange=TAGGED[args.handoff])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    obj, x_host, timed_steps = decode_object(S, torch, dist, stack, cfg, M, args, peaks, rank, world, local, main=True)
    # ---- end to end: pinned host input -> device, all layers, result back to host, every step
    y_host = torch.empty(M, cfg.hidden, dtype=torch.float16).pin_memory()
    for _ in range(3):
        stack.step(x_host); y_host.copy_(stack.output(), non_blocking=True); torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        stack.step(x_host)
        y_host.copy_(stack.output(), non_blocking=True)
        torch.cuda.synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0])
    finite = bool(torch.isfinite(stack.output().float()).all())
    nbytes = S.algorithmic_bytes(cfg, M, layers=stack.layers)    # whole model, all ranks together
    e2e_gbs = nbytes / (e2e_ms * 1e-3) / 1e9
    n_gemv = len(stack._plans) if stack._plans is not None else 7 * stack.layers
    kname = ("mpsbnb_decode4_stream_kernel (one cooperative launch per step: all layers)" if stack._persist
             else "decode kernel, one launch per layer (7 linears)" if stack._plans is not None else "one launch per linear")
    out = {
        "metric": "nf4_decode_gbs", "value": obj["value"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": obj["ms_per_step"], "ms_min": obj["ms_min"], "ms_max": obj["ms_max"],
        "timed_blocks": obj["blocks"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(cfg, M, stack.layers, world),
        "parity_rel_err": obj["parity_rel_err"], "parity_check": "2-layer instance of the same stack (same sharding and kernels) "
                                                                  "against the C oracle of the reference CPU path",
        "device_status": obj["device_status"], "outputs_finite": finite,
        "roofline": dict(obj["roofline"], kernel=kname, launches_per_step=n_gemv, bytes_per_launch=nbytes / world / n_gemv,
                         note="achieved = algorithmic bytes of the step / CUDA-event time of the whole step (the decode "
                              "launch plus the small input / counter kernels), per GPU"),
        "e2e": {"value": e2e_gbs, "unit": "GB/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": y_host.numel() * 2},
        "gpu_launches": stack.launches_per_step() * timed_steps,
        "clocks": clocks,
    }
    bad = obj["device_status"] != 0 or not finite
    if not args.skip_extras and args.layers is None:
        # the same stack at the other batch sizes of the configuration (every N)
        for name, m in (("batch32", 32), ("batch512", 512)):
            try:
                o2, _, _ = decode_object(S, torch, dist, stack, cfg, m, args, peaks, rank, world, local)
                o2["config"] = workload_config(cfg, m, stack.layers, world)
                bad = bad or o2["device_status"] != 0
            except Exception as ex:                                  # reported, never hidden
                o2 = {"error": repr(ex)}
            out[name] = o2
    barrier()
    del stack
    torch.cuda.empty_cache()
    if world == 1 and not args.skip_extras and args.layers is None:
        other = S.LLAMA2_7B if cfg.name != "llama2-7b" else None
        if other is not None:
            st7 = S.LayerStack(other, device=f"cuda:{local}")
            for name, m in (("decode_7b", 1), ("decode_7b_batch16", 16)):
                try:
                    o2, _, _ = decode_object(S, torch, dist, st7, other, m, args, peaks, rank, world, local)
                    o2["config"] = workload_config(other, m, st7.layers, world)
                    bad = bad or o2["device_status"] != 0
                except Exception as ex:
                    o2 = {"error": repr(ex)}
                out[name] = o2
            del st7
            torch.cuda.empty_cache()
        try:
            out["prefill"] = prefill_config2(torch, peaks)
        except Exception as ex:
            out["prefill"] = {"error": repr(ex)}
        try:
            out["int8_fp8"] = int8_fp8_config4(torch, peaks)
        except Exception as ex:
            out["int8_fp8"] = {"error": repr(ex)}
        try:
            out["quantize_path"] = quantize_path(torch, peaks)
        except Exception as ex:
            out["quantize_path"] = {"error": repr(ex)}
        out["cpu_baseline"] = cpu_baseline(cfg, M)
    if rank == 0:
        print(json.dumps(out), flush=True)
    rc = 1 if bad else 0
    if world > 1:
        # The captured step may hold NCCL kernels; tearing the communicator down under a live graph can block.
        # Every rank is past the last collective (barrier above), so leave without the teardown.
        sys.stdout.flush(); sys.stderr.flush()
        os._exit(rc)
    if rc:
        sys.exit(rc)

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--model", default="llama-70b", choices=["llama2-7b", "llama-70b"])
    ap.add_argument("--layers", type=int, default=None, help="reduced depth, for profiler captures")
    ap.add_argument("--skip-extras", action="store_true", help="no prefill object, no CPU baseline")
    ap.add_argument("--prefill-only", action="store_true", help="only the prefill GEMM object (BASELINE config 2)")
    ap.add_argument("--int8-only", action="store_true", help="only the INT8 / FP8 / outlier-split object (BASELINE config 4)")
    ap.add_argument("--quant-only", action="store_true", help="only the quantise / dequantise / embedding object")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1: layer boundary by peer stores + flags (default) or by an NCCL all-gather")
    ap.add_argument("--handoff", default="auto", choices=["auto", "tagged", "flags"],
                    help="N > 1, one launch per step: how a layer learns that its input is complete - tagged {values, tag} "
                         "entries, or per-rank counts of closed tiles (auto: counts)")
    ap.add_argument("--boundary", default=None, choices=["kernel", "inline", "stream"],
                    help="layer boundary: its own small kernel, the closing step of the GEMV launch, or streamed tile "
                         "by tile from inside the launch (default)")
    ap.add_argument("--per-layer", action="store_true", help="one GEMV launch per layer instead of one per step")
    args = ap.parse_args()
    from mps_bitsandbytes_b200 import stack as S
    cfg = S.LLAMA2_7B if args.model == "llama2-7b" else S.LLAMA_70B
    if args.prefill_only:
        import torch
        print(json.dumps(prefill_config2(torch, load_peaks(), steps=args.steps, warmup=max(args.warmup, 3))))
    elif args.int8_only:
        import torch
        print(json.dumps(int8_fp8_config4(torch, load_peaks(), steps=args.steps, warmup=max(args.warmup, 3))))
    elif args.quant_only:
        import torch
        print(json.dumps(quantize_path(torch, load_peaks(), steps=args.steps, warmup=max(args.warmup, 3))))
    elif args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_gpu(args, cfg)


if __name__ == "__main__":
    main()
