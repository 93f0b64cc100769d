"""Benchmark of the fused dequantise-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch M]
                    [--layers L] [--skip-extras] [--prefill-only] [--int8-only]

Workload (N = 1): the Llama-2-7B-shaped NF4 decode stack of BASELINE config 3 — 32 layers x
{q,k,v,o 4096x4096, gate/up 11008x4096, down 4096x11008}, double-quantised absmax, fp16,
batch 1 — one "step" = one pass over all 224 linears (3.34 GB of packed weights and absmax,
far larger than the 126 MB L2, so every step streams from HBM), by default ONE cooperative
kernel launch.  For N > 1 (launched by torchrun, one rank per GPU) the stack is N-sharded over
the ranks; at each layer boundary every rank stores its shard of the next input into all ranks'
buffers over NVLink and raises flags (--exchange nccl: an NCCL all-gather instead); the per-GPU
work shrinks with N (strong scaling of a fixed model).

Prints ONE JSON line: metric nf4_decode_gbs = algorithmic bytes per step / step time, with
the HBM roofline, an end-to-end figure through the public LayerStack API with host buffers,
a CPU baseline (the C oracle of the reference's CPU path on this host's cores), and, at
N = 1, the prefill GEMM of BASELINE config 2 (FP4, 2048 x 4096 x 11008) as a second object and
the INT8 / FP8 / outlier-split matmuls of BASELINE config 4 (512 x 4096 x 16384) as a third.

--layers L runs a stack of only L layers (a reduced workload for profiler captures; the JSON
line names it) and --skip-extras leaves out the prefill object and the CPU baseline.  The timed
region is bracketed by cudaProfilerStart/Stop so that a profiler started with
--profile-from-start off sees exactly the timed launches.

--prefill-only runs just the prefill GEMM of BASELINE config 2 and prints its object (used for
profiler captures of the tcgen05 GEMM).

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


# dram__bytes_read.sum + dram__bytes_write.sum of ONE gemv4_stream_kernel launch (one Llama-2-7B layer, batch 1,
# whole layer on one GPU), from the ncu capture summarised in profiles/gemv4_stream_kernel_llama7b_one_layer_per_launch.md;
# a launch that covers all layers moves layers x this (the two-layer one-launch capture reads 213.5 MB for 2 layers)
NCU_TRAFFIC_7B_LAYER_BYTES = 108.5e6


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
def prefill_config2(torch, peaks, steps=20, warmup=5):
    """BASELINE config 2: FP4 (double-quantised) 11008 x 4096 weight, x [2048, 4096] fp16."""
    import mps_bitsandbytes_b200 as bnb
    g = torch.Generator(device="cuda"); g.manual_seed(2)
    w = (torch.randn(11008, 4096, device="cuda", generator=g) * 0.02).half()
    x = torch.randn(2048, 4096, device="cuda", generator=g).half()
    packed, st = bnb.quantize_fp4(w, compress_statistics=True)
    del w
    for _ in range(warmup):
        y = bnb.matmul_4bit(x, packed, st)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        y = bnb.matmul_4bit(x, packed, st)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    flops = 2.0 * 2048 * 4096 * 11008
    tf = flops / (ms * 1e-3) / 1e12
    return {"metric": "fp4_prefill_tflops", "value": tf, "unit": "TFLOP/s", "ms": ms,
            "config": {"workload": "FP4+DQ 11008x4096 weight, x [2048,4096] fp16 (dequantise + tcgen05 GEMM)"},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops"], "traffic": None, "peak_source": peaks["source"]}}


def int8_fp8_config4(torch, peaks, steps=10, warmup=3):
    """BASELINE config 4: activations [512, 4096] fp16 with 0.5 % of the columns at magnitude ~20, weight
    4096 x 16384 ~ N(0, 0.02): matmul_int8 (row-wise A, column-wise B), matmul_colrow, matmul_fp8_e4m3 and the
    outlier-aware split (OutlierAwareLinear).  Every figure includes the operand-preparation passes."""
    import mps_bitsandbytes_b200 as bnb
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
    cases = {"matmul_int8": lambda: bnb.matmul_int8(aq, bq, a_s, b_s),
             "matmul_colrow": lambda: bnb.matmul_colrow(x, cq, cr, cc),
             "matmul_fp8_e4m3": lambda: bnb.matmul_fp8_e4m3(x, f8, f8s),
             "outlier_aware_linear": lambda: oal(x)}
    flops = 2.0 * M * K * Nn
    res = {"config": {"workload": f"x [{M},{K}] fp16 (0.5% outlier columns), weight {K}x{Nn}; dequantise/requantise passes + tcgen05 GEMM",
                      "outlier_columns": int(oal.outlier_indices.numel())}, "unit": "TFLOP/s", "peak": peaks["bf16_tflops"]}
    for name, fn in cases.items():
        for _ in range(warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        res[name] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "frac": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    return res


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
                         fused_exchange=args.exchange == "fused", boundary=args.boundary, persistent=not args.per_layer, mid_batch_tcgen05=not args.no_mid_tc)
    stack.prepare(M, use_graph=True)
    gen = torch.Generator(device="cpu"); gen.manual_seed(1)
    x_host = torch.randn(M, cfg.hidden, generator=gen).half().pin_memory()
    y_host = torch.empty(M, cfg.hidden, dtype=torch.float16).pin_memory()
    x_dev = x_host.cuda()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for _ in range(max(args.warmup, 3)):
        stack.step(x_dev)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.profiler.start()
    e0.record()
    for _ in range(args.steps):
        stack.step()
    e1.record()
    barrier()
    torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    # ---- end to end: pinned host input -> device, all layers, result back to host, every step
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
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    finite = bool(torch.isfinite(stack.output().float()).all())

    nbytes = S.algorithmic_bytes(cfg, M, layers=stack.layers)    # whole model, all ranks together
    gbs = nbytes / (ms * 1e-3) / 1e9
    e2e_gbs = nbytes / (e2e_ms * 1e-3) / 1e9
    out = None
    if rank == 0:
        per_gpu = gbs / world
        grouped = stack._plans is not None
        n_gemv = len(stack._plans) if grouped else 7 * stack.layers
        kname = ("gemv4_stream_kernel (one cooperative launch per step: all layers)" if grouped and n_gemv == 1 and stack.layers > 1
                 else "gemv4_stream_kernel (one launch per layer: 7 linears)" if grouped else "gemv4_kernel (one launch per linear)")
        out = {
            "metric": "nf4_decode_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": dict(workload_config(cfg, M, stack.layers, world), outputs_finite=finite),
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": per_gpu / peaks["hbm_gbs"],
                         "traffic": NCU_TRAFFIC_7B_LAYER_BYTES * (stack.layers if n_gemv == 1 else 1)
                         if (grouped and world == 1 and M == 1 and cfg.name == "llama2-7b") else None,
                         "peak_source": peaks["source"],
                         "kernel": kname, "launches_per_step": n_gemv,
                         "bytes_per_launch": nbytes / world / n_gemv,
                         "note": "achieved = algorithmic bytes of the step / CUDA-event time of the whole step "
                                 "(the GEMV launch(es) plus the small input / boundary / counter kernels), per GPU"},
            "e2e": {"value": e2e_gbs, "unit": "GB/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": y_host.numel() * 2},
            "gpu_launches": stack.launches_per_step() * args.steps,
            "clocks": clocks,
        }
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    if rank == 0:
        if world == 1 and not args.skip_extras:
            del stack
            torch.cuda.empty_cache()
            try:
                out["prefill"] = prefill_config2(torch, peaks)
            except Exception as ex:                                  # reported, never hidden
                out["prefill"] = {"error": repr(ex)}
            try:
                out["int8_fp8"] = int8_fp8_config4(torch, peaks)
            except Exception as ex:
                out["int8_fp8"] = {"error": repr(ex)}
            out["cpu_baseline"] = cpu_baseline(cfg, M)
        print(json.dumps(out), flush=True)
    if world > 1:
        # The captured step holds NCCL kernels; tearing the communicator down under a live graph can block.
        # Every rank is past the last collective (barrier above), so leave without the teardown.
        sys.stdout.flush(); sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--model", default="llama2-7b", choices=["llama2-7b", "llama-70b"])
    ap.add_argument("--layers", type=int, default=None, help="reduced depth, for profiler captures")
    ap.add_argument("--skip-extras", action="store_true", help="no prefill object, no CPU baseline")
    ap.add_argument("--prefill-only", action="store_true", help="only the prefill GEMM object (BASELINE config 2)")
    ap.add_argument("--int8-only", action="store_true", help="only the INT8 / FP8 / outlier-split object (BASELINE config 4)")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1: layer boundary by peer stores + flags (default) or by an NCCL all-gather")
    ap.add_argument("--boundary", default=None, choices=["kernel", "inline", "stream"],
                    help="layer boundary: its own small kernel, the closing step of the GEMV launch, or streamed tile "
                         "by tile from inside the launch (default)")
    ap.add_argument("--per-layer", action="store_true", help="one GEMV launch per layer instead of one per step")
    ap.add_argument("--no-mid-tc", action="store_true", help="batch 9..32: per-linear launches of the older kernel instead of tcgen05")
    args = ap.parse_args()
    from mps_bitsandbytes_b200 import stack as S
    cfg = S.LLAMA2_7B if args.model == "llama2-7b" else S.LLAMA_70B
    if args.prefill_only:
        import torch
        print(json.dumps(prefill_config2(torch, load_peaks(), steps=args.steps, warmup=max(args.warmup, 3))))
    elif args.int8_only:
        import torch
        print(json.dumps(int8_fp8_config4(torch, load_peaks(), steps=args.steps, warmup=max(args.warmup, 3))))
    elif args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_gpu(args, cfg)


if __name__ == "__main__":
    main()
