"""Synthetic decoder-layer stacks of Linear4bit layers (Llama-2-7B and Llama-70B shaped), the
workload of the decode / prefill benchmarks, single-GPU or N-sharded over the GPUs of one box.

The reference ships linear layers, not a model, so the dataflow between them is defined
here.  Layer l takes a replicated activation h [M, H]:

    q, k, v, o, gate, up = W_* . h          (six projections, all reading h)
    down                 = W_down . e       (e [M, F]: h tiled along features, e[m, j] = h[m, j mod H])
    h_next               = alpha * (o + down)        alpha keeps activations at unit scale

Every projection is column (N) sharded over the ranks: rank r owns rows [r N/g, (r+1) N/g) of
each packed weight and of its absmax — pure slices of the reference layout.  The only exchange
is an all-gather of the [M, H/g] shard of h_next at the layer boundary.  q, k, v, gate, up are
outputs of the layer (they stay sharded).

One ``step`` runs all layers; it is captured once into a CUDA graph and replayed.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _native as N
from .functional import QuantState, _expand_absmax, quantize_4bit


@dataclass
class StackConfig:
    name: str
    hidden: int
    ffn: int
    kv: int          # output width of the k / v projections (GQA)
    layers: int

    def projections(self):
        """(name, out_features, in_features) of the seven linears of one layer."""
        H, F, KV = self.hidden, self.ffn, self.kv
        return [("q", H, H), ("k", KV, H), ("v", KV, H), ("o", H, H), ("gate", F, H), ("up", F, H), ("down", H, F)]

    def params_per_layer(self) -> int:
        return sum(n * k for _, n, k in self.projections())

    def alpha(self) -> float:
        # std of (o + down) for unit-variance h and weights ~ N(0, 0.02)
        return 1.0 / math.sqrt(0.02 ** 2 * (self.hidden + self.ffn))


LLAMA2_7B = StackConfig("llama2-7b", 4096, 11008, 4096, 32)
LLAMA_70B = StackConfig("llama-70b", 8192, 28672, 1024, 80)


def weight_bytes(cfg: StackConfig, double_quant: bool = True, layers: Optional[int] = None) -> int:
    """Packed + absmax bytes of the stack: 0.5 B per weight + absmax (fp32 per 64, or int8 per 64
    plus fp32 per 16384 when double-quantised)."""
    L = cfg.layers if layers is None else layers
    total = 0
    for _, n, k in cfg.projections():
        nb = n * (k // 64)
        total += n * k // 2 + (nb + 4 * ((nb + 255) // 256) if double_quant else 4 * nb)
    return total * L


def algorithmic_bytes(cfg: StackConfig, M: int, double_quant: bool = True, layers: Optional[int] = None) -> int:
    """Bytes one step must move: every weight byte and absmax once, plus x and y of each linear (fp16)."""
    L = cfg.layers if layers is None else layers
    act = sum(2 * M * (n + k) for _, n, k in cfg.projections())
    return weight_bytes(cfg, double_quant, layers) + act * L


def shard_rows(n: int, rank: int, world: int):
    """Row range [lo, hi) of an [n, k] weight (and of its packed bytes / absmax rows) owned by ``rank``."""
    if n % world:
        raise ValueError(f"{n} rows do not divide over {world} ranks")
    ns = n // world
    return rank * ns, (rank + 1) * ns


def gathered_to_full(gathered: torch.Tensor) -> torch.Tensor:
    """[g, M, H/g] (what all_gather_into_tensor returns for per-rank [M, H/g] shards) -> [M, H].
    The device path does this inside mpsbnb_stack_expand; this is its host-side statement."""
    g, M, hs = gathered.shape
    return gathered.permute(1, 0, 2).reshape(M, g * hs)


class _Proj:
    __slots__ = ("name", "n", "k", "packed", "absmax", "absmax2", "state")


class LayerStack:
    """N-sharded stack of 4-bit linears.  ``rank`` / ``world`` select the shard (world = 1: whole)."""

    def __init__(self, cfg: StackConfig, device, quant_type: str = "nf4", double_quant: bool = True,
                 layers: Optional[int] = None, rank: int = 0, world: int = 1, seed: int = 1000,
                 dtype: torch.dtype = torch.float16, group=None, use_pdl: bool = True, fused_exchange: bool = True, boundary: Optional[str] = None, persistent: bool = True, mid_batch_tcgen05: bool = True, emulate_peers: bool = False,
                 tagged_exchange: Optional[bool] = None):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.layers = cfg.layers if layers is None else layers
        self.rank, self.world, self.group = rank, world, group
        # timing aid: run ONE rank's shard of a `world`-way split on this GPU alone, every peer pointer aimed at this
        # GPU's own buffers (the per-GPU work of the sharded stack without NVLink; the result is not the model's)
        self.emulate_peers = emulate_peers and world > 1
        # one-launch step: True = h travels as {values, tag} entries (no flag, fence or acquire on the layer boundary's
        # path, and a linear starts as soon as ITS columns have arrived; the loaders pay for it by examining tags, 8 % of
        # a single GPU's streaming rate).  Off unless asked for: per-rank counts of closed tiles are the measured default.
        self.tagged_exchange = tagged_exchange
        # programmatic dependent launch between the per-layer kernels (single GPU: no NCCL kernel in between)
        self.use_pdl = use_pdl and world == 1
        # world > 1, batch <= 8: the layer boundary stores its shard of h into every rank's buffer over NVLink and
        # raises flags (csrc/exchange.cu) instead of calling an NCCL all-gather; decided in prepare()
        self.fused_exchange = fused_exchange and world > 1
        # layer boundary (h' = alpha (o + down)) of the grouped path: "kernel" = its own small kernel after the GEMV
        # launch; "inline" = closing step of the GEMV launch (last CTA); "stream" = tile by tile inside the GEMV
        # launch as soon as a tile's o and down contributions are complete (h rotates over three buffers, or has one
        # per layer when the whole step is one launch)
        # Measured (7B step, one GPU): stream 1.167 ms, kernel 1.229 ms, inline 1.306 ms; across GPUs streaming also
        # hides the exchange.  With NCCL as the exchange the boundary has to be its own kernel.
        if boundary is None:
            boundary = "stream" if (world == 1 or fused_exchange) else "kernel"
        if boundary not in ("kernel", "inline", "stream"):
            raise ValueError("boundary must be 'kernel', 'inline' or 'stream'")
        self.boundary = boundary
        self.mid_batch_tcgen05 = mid_batch_tcgen05
        # with the streamed boundary, ONE cooperative launch per step covers all layers (segment = layer): the
        # weight stream never drains at a layer boundary
        self.persistent = persistent and boundary == "stream"
        self.in_kernel_boundary = boundary != "kernel"
        self._fused = self._stream = self._persist = self._inline = False
        self._nbuf = 2
        self._peer_bases = []
        self.quant_type, self.double_quant = quant_type, double_quant
        self.alpha = cfg.alpha()
        if cfg.hidden % world or cfg.ffn % world or cfg.kv % world:
            raise ValueError("layer widths must divide by the number of ranks")
        self.proj: List[List[_Proj]] = []
        gen = torch.Generator(device=self.device)
        for l in range(self.layers):
            row = []
            for i, (name, n, k) in enumerate(cfg.projections()):
                lo, hi = shard_rows(n, rank, world)
                ns = hi - lo
                if (ns * (k // 64)) % 256 and double_quant and world > 1:
                    raise ValueError("shard does not align with the 256-block groups of double quantisation")
                # the whole weight is drawn from the (layer, projection) seed, N(0, 0.02), and this
                # rank keeps its rows: the model is the same for every world size
                gen.manual_seed(seed + 7 * l + i)
                full = torch.randn(n, k, device=self.device, generator=gen, dtype=torch.float32)
                w = (full[lo:hi] * 0.02).to(dtype)
                del full
                packed, st = quantize_4bit(w, blocksize=64, compress_statistics=double_quant, quant_type=quant_type)
                del w
                pr = _Proj()
                pr.name, pr.n, pr.k, pr.packed, pr.state = name, ns, k, packed, st
                pr.absmax, pr.absmax2 = _expand_absmax(st.absmax, st.state2)
                row.append(pr)
            self.proj.append(row)
        self._graph = None
        self._M = None

    # ------------------------------------------------------------------ buffers
    def _alloc(self, M: int):
        cfg, dev, dt, g = self.cfg, self.device, self.dtype, self.world
        self.h = torch.zeros(M, cfg.hidden, dtype=dt, device=dev)
        self.e = torch.zeros(M, cfg.ffn, dtype=dt, device=dev)
        self.out = {name: torch.zeros(M, n // g, dtype=dt, device=dev) for name, n, _ in cfg.projections()}
        self.h_shard = torch.zeros(M, cfg.hidden // g, dtype=dt, device=dev)
        self.gathered = torch.zeros(g, M, cfg.hidden // g, dtype=dt, device=dev) if g > 1 else None
        self.acc = torch.zeros(M, cfg.hidden // g, dtype=torch.float32, device=dev)
        self._M = M
        self._plans = None
        self._fused = self.fused_exchange and M <= 8
        self._stream = self.boundary == "stream" and M <= 8 and (g == 1 or self._fused)
        self._persist = self.persistent and self._stream
        # h buffers a step rotates over.  One launch per step: one per layer plus the result.  Nothing in THIS stack waits
        # for a CTA's q / k / v / gate / up units (down reads h, not gate * up), so such a CTA may fall layers behind the
        # o / down chain; with a buffer per layer none is rewritten while a late reader still wants it, and the step's end
        # (the kernel's end; across GPUs the acknowledgement counts) separates the steps.
        self._nbuf = (self.layers + 1) if self._persist else (3 if self._stream else 2)
        self._inline = self.in_kernel_boundary and M <= 8         # closing step inside the GEMV launch (default kernel only)
        if self._fused or self._persist:
            self._setup_exchange(M)
        elif self._stream:
            self.hbuf = torch.zeros(self._nbuf, M, cfg.hidden, dtype=dt, device=dev)
        if self._persist:
            self._build_persistent_plan(M)
        elif M <= 8:
            self._build_plans(M)
        elif M <= 32 and self.mid_batch_tcgen05:
            # batch 9 .. 32: grouped launches of the tensor-memory decode kernel (its MMAs are 16 or 32 columns wide),
            # one per layer, with the boundary as its own kernel
            self._build_plans(M)

    # ------------------------------------------------------------------ fused exchange (world > 1, batch <= 8)
    def _setup_exchange(self, M: int):
        """One exported buffer per rank: h double-buffered by layer parity [2, M, H], flags int32[g] (raised by the
        boundary kernels of all ranks), acks int32[g] (raised at the end of a step).  Peers map it with CUDA IPC."""
        cfg, dev, g, lib = self.cfg, self.device, self.world, N.lib()
        self._close_exchange()
        esz = torch.empty(0, dtype=self.dtype).element_size()
        # the one-launch-per-step form exchanges h in TAGGED form: 8-byte entries {two values, tag} (twice the bytes; no
        # flags or fences on the way, see mpsbnb_tagged_write in the header)
        self._tagged = self._persist and cfg.hidden % 2 == 0 and bool(self.tagged_exchange)
        if self._tagged:
            esz *= 2
        nb = self._nbuf
        h_bytes = (nb * M * cfg.hidden * esz + 255) // 256 * 256
        self._xbuf = torch.zeros(h_bytes + 512, dtype=torch.uint8, device=dev)
        if self._tagged:
            self.hbuf = self._xbuf[:nb * M * cfg.hidden * esz].view(torch.int64).view(nb, M, cfg.hidden // 2)
        else:
            self.hbuf = self._xbuf[:nb * M * cfg.hidden * esz].view(self.dtype).view(nb, M, cfg.hidden)
        self.flags = self._xbuf[h_bytes:h_bytes + 4 * g].view(torch.int32)
        self.acks = self._xbuf[h_bytes + 256:h_bytes + 256 + 4 * g].view(torch.int32)
        self.step_ctr = torch.zeros(1, dtype=torch.int32, device=dev)
        self.h_out = torch.zeros(M, cfg.hidden, dtype=self.dtype, device=dev)
        everyone = [None] * g
        if self.emulate_peers:
            base = self._xbuf.data_ptr()
            one = M * cfg.hidden * esz
            # tagged form: no flags to fake, so "peer" r's copy of this rank's columns is aimed at rank r's columns of the
            # same buffer - every column then receives a (meaningless but correctly tagged) value, as on g real GPUs
            shift = (cfg.hidden // g) * esz if self._tagged else 0
            self._peer_h = [torch.tensor([base + p * one + (r - self.rank) * shift for r in range(g)], dtype=torch.int64, device=dev)
                            for p in range(nb)]
            # the kernels write flag pointer[r] + own rank: aim pointer r at flags[r - rank] so that slot r is raised
            self._peer_flags = torch.tensor([base + h_bytes + 4 * (r - self.rank) for r in range(g)], dtype=torch.int64, device=dev)
            self._peer_acks = torch.tensor([base + h_bytes + 256 + 4 * (r - self.rank) for r in range(g)], dtype=torch.int64, device=dev)
            self._peer_h_all = torch.cat(self._peer_h)
            torch.cuda.synchronize()
            return
        if g > 1:
            handle = (C.c_ubyte * 64)()
            off = C.c_int64(0)
            N.check(lib.mpsbnb_ipc_export(N.ptr(self._xbuf), handle, C.byref(off)), "ipc_export")
            mine = (bytes(handle), int(off.value))
            torch.cuda.synchronize()
            torch.distributed.all_gather_object(everyone, mine, group=self.group)
        bases = []
        for r in range(g):
            if r == self.rank:
                bases.append(self._xbuf.data_ptr())
                continue
            hb = (C.c_ubyte * 64).from_buffer_copy(everyone[r][0])
            base = C.c_void_p(0)
            N.check(lib.mpsbnb_ipc_open(hb, C.byref(base)), "ipc_open")
            self._peer_bases.append(base.value)
            bases.append(base.value + everyone[r][1])
        one = M * cfg.hidden * esz
        self._peer_h = [torch.tensor([b + p * one for b in bases], dtype=torch.int64, device=dev) for p in range(nb)]
        self._peer_flags = torch.tensor([b + h_bytes for b in bases], dtype=torch.int64, device=dev)
        self._peer_acks = torch.tensor([b + h_bytes + 256 for b in bases], dtype=torch.int64, device=dev)
        self._peer_h_all = torch.cat(self._peer_h)                # [buffer][rank]
        torch.cuda.synchronize()
        if g > 1:
            torch.distributed.barrier(group=self.group)          # every rank has mapped every buffer (all zero)

    def _close_exchange(self):
        for b in self._peer_bases:
            N.lib().mpsbnb_ipc_close(C.c_void_p(b))
        self._peer_bases = []

    def _x_of_layer(self, l: int) -> torch.Tensor:
        """Input h of layer l: the parity buffer in the fused exchange, else the one h."""
        return self.hbuf[l % self._nbuf] if (self._fused or self._stream or self._persist) else self.h

    def _build_plans(self, M: int):
        """One grouped-launch plan per layer: q, k, v, gate, up store their outputs; o and down add
        into the fp32 accumulator ``acc`` (their sum is what the boundary needs); down reads h with
        its column index wrapped at H, which is the tiled input e without materialising it."""
        cfg, lib, g = self.cfg, N.lib(), self.world
        self._plans, self._plan_mem = [], []
        self._ep_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._own_h = torch.tensor([self.h.data_ptr()], dtype=torch.int64, device=self.device)
        if self._stream:
            self._tile_cnt = torch.zeros((cfg.hidden // g + 31) // 32, dtype=torch.int32, device=self.device)
            if not self._fused:
                self._own_hbuf = [torch.tensor([self.hbuf[p].data_ptr()], dtype=torch.int64, device=self.device)
                                  for p in range(self._nbuf)]
        for l in range(self.layers):
            descs = (N.Linear4Desc * 7)()
            for i, pr in enumerate(self.proj[l]):
                d = descs[i]
                d.x, d.x_ld = self._x_of_layer(l).data_ptr(), cfg.hidden
                d.x_period = cfg.hidden if pr.name == "down" else 0
                d.packed, d.absmax = pr.packed.data_ptr(), pr.absmax.data_ptr()
                d.absmax2 = None if pr.absmax2 is None else pr.absmax2.data_ptr()
                d.bias = None
                if pr.name in ("o", "down"):
                    d.y, d.acc = None, self.acc.data_ptr()
                else:
                    d.y, d.acc = self.out[pr.name].data_ptr(), None
                d.N, d.K = pr.n, pr.k
            nbytes = lib.mpsbnb_gemv_4bit_group_plan_bytes(descs, C.c_int(7))
            mem = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            plan = N.GroupPlan()
            N.check(lib.mpsbnb_gemv_4bit_group_plan(descs, C.c_int(7), N.i64(M), N.dt(self.dtype), N.dt(self.dtype),
                                                    C.c_int(N.qt(self.quant_type)), N.ptr(mem), C.c_size_t(nbytes),
                                                    C.byref(plan), N.stream()), "gemv_4bit_group_plan")
            plan.flags = N.GROUP_PDL if (self.use_pdl or self._fused) else 0
            if self._inline and (g == 1 or self._fused):
                # the CTA that finishes last writes alpha * (o + down) as the next layer's h (into every rank's
                # buffer when fused) and re-arms the accumulator: no boundary kernel
                ep = plan.ep
                ep.acc, ep.alpha, ep.counter = self.acc.data_ptr(), self.alpha, self._ep_counter.data_ptr()
                ep.M, ep.hs, ep.H, ep.rank, ep.nranks = M, cfg.hidden // g, cfg.hidden, self.rank, g
                nxt = (l + 1) % self._nbuf
                if self._fused:
                    ep.peer_h, ep.peer_flags = self._peer_h[nxt].data_ptr(), self._peer_flags.data_ptr()
                    ep.step, ep.mul, ep.add = self.step_ctr.data_ptr(), self.layers, l + 1
                else:
                    ep.peer_h = self._own_hbuf[nxt].data_ptr() if self._stream else self._own_h.data_ptr()
                if self._stream:
                    ep.tile_cnt, ep.tile_expect = self._tile_cnt.data_ptr(), plan.acc_parts
            if self._fused:
                # layer 0 waits for the acks of the previous step (every rank has copied its result out), the
                # others for the boundary flags of the layer before
                src = self.acks if l == 0 else self.flags
                plan.wait_flags, plan.wait_step = src.data_ptr(), self.step_ctr.data_ptr()
                plan.wait_n = g
                plan.wait_mul, plan.wait_add = (1, 0) if l == 0 else (self.layers, l)
            self._plans.append(plan)
            self._plan_mem.append(mem)

    def _build_persistent_plan(self, M: int):
        """One plan for the whole stack: 7 L linears, segment = layer.  Layer l reads h from buffer l (one buffer per
        layer plus the result); the closing step of segment l (streamed, by tiles) writes buffer l + 1 on every rank and
        either adds to the per-rank counts of closed tiles - linears of layer l wait for counts >= (step L + l) T - or,
        with the tagged exchange, writes entries that carry the tag step (L + 1) + l + 1, which layer l + 1 looks for."""
        cfg, lib, g, L = self.cfg, N.lib(), self.world, self.layers
        n = 7 * L
        if self._tagged:
            self.acc2 = torch.zeros(2, M, cfg.hidden // g, dtype=torch.float32, device=self.device)
        descs = (N.Linear4Desc * n)()
        self.out_layers = []
        for l in range(L):
            outs = {name: torch.zeros(M, nn // g, dtype=self.dtype, device=self.device) for name, nn, _ in cfg.projections()}
            self.out_layers.append(outs)
            for i, pr in enumerate(self.proj[l]):
                d = descs[7 * l + i]
                d.x, d.x_ld = self.hbuf[l % self._nbuf].data_ptr(), cfg.hidden
                d.x_period = cfg.hidden if pr.name == "down" else 0
                d.packed, d.absmax = pr.packed.data_ptr(), pr.absmax.data_ptr()
                d.absmax2 = None if pr.absmax2 is None else pr.absmax2.data_ptr()
                d.bias = None
                if pr.name in ("o", "down"):
                    d.y, d.acc = None, (self.acc2[l & 1] if self._tagged else self.acc).data_ptr()
                else:
                    d.y, d.acc = outs[pr.name].data_ptr(), None
                d.N, d.K, d.segment = pr.n, pr.k, l
        self.out = self.out_layers[-1]
        nbytes = lib.mpsbnb_gemv_4bit_group_plan_bytes(descs, C.c_int(n))
        self._plan_mem = [torch.empty(nbytes, dtype=torch.uint8, device=self.device)]
        plan = N.GroupPlan()
        N.check(lib.mpsbnb_gemv_4bit_group_plan(descs, C.c_int(n), N.i64(M), N.dt(self.dtype), N.dt(self.dtype),
                                                C.c_int(N.qt(self.quant_type)), N.ptr(self._plan_mem[0]), C.c_size_t(nbytes),
                                                C.byref(plan), N.stream()), "gemv_4bit_group_plan")
        self._ep_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        # tagged exchange: accumulators and tile counts by layer parity (see the closer warp of the kernel)
        self._tile_cnt = torch.zeros((2 if self._tagged else 1) * ((cfg.hidden // g + 31) // 32), dtype=torch.int32, device=self.device)
        ep = plan.ep
        ep.acc, ep.alpha, ep.counter = (self.acc2 if self._tagged else self.acc).data_ptr(), self.alpha, self._ep_counter.data_ptr()
        ep.M, ep.hs, ep.H, ep.rank, ep.nranks = M, cfg.hidden // g, cfg.hidden, self.rank, g
        ep.peer_h, ep.nbuf, ep.peer_flags = self._peer_h_all.data_ptr(), self._nbuf, self._peer_flags.data_ptr()
        ep.step, ep.mul, ep.add = self.step_ctr.data_ptr(), L, 1
        ep.tile_cnt, ep.tile_expect = self._tile_cnt.data_ptr(), plan.acc_parts
        # flags[r] counts the 32-row tiles of h that rank r has closed and stored here since the start (every closed
        # tile adds 1 on every rank): the input of layer l of step s is complete when every count is (s L + l) T
        if self._tagged:
            # tagged exchange: the input of layer l of step s carries the tag s (L + 1) + l; nothing else is waited for
            ep.count_tiles, ep.mul, ep.add = 2, L + 1, 1
            plan.wait_flags, plan.wait_step = None, self.step_ctr.data_ptr()
            plan.wait_n, plan.wait_mul, plan.wait_add, plan.wait_seg_mul = 0, L + 1, 0, 1
        else:
            # flags[r] counts the 32-row tiles of h that rank r has closed and stored here since the start
            T = self._tiles_per_shard = (cfg.hidden // g + 31) // 32
            ep.count_tiles = 1
            plan.wait_flags, plan.wait_step = self.flags.data_ptr(), self.step_ctr.data_ptr()
            plan.wait_n, plan.wait_mul, plan.wait_add, plan.wait_seg_mul = g, L * T, 0, T
        self._plans = [plan]

    def _gemv(self, pr: _Proj, x: torch.Tensor, y: torch.Tensor, M: int):
        lib = N.lib()
        if M <= lib.mpsbnb_gemv_4bit_max_m():
            N.check(lib.mpsbnb_gemv_4bit(N.ptr(x), N.dt(self.dtype), N.i64(M), N.ptr(pr.packed), N.ptr(pr.absmax),
                                         N.ptr(pr.absmax2), N.i64(pr.n), N.i64(pr.k), C.c_int(64),
                                         C.c_int(N.qt(self.quant_type)), None, N.ptr(y), N.dt(self.dtype), N.stream()),
                    "gemv_4bit")
        else:
            N.check(lib.mpsbnb_gemm_4bit(N.ptr(x), N.dt(self.dtype), N.i64(M), N.ptr(pr.packed), N.ptr(pr.absmax),
                                         N.ptr(pr.absmax2), N.i64(pr.n), N.i64(pr.k), C.c_int(64),
                                         C.c_int(N.qt(self.quant_type)), None, N.ptr(y), N.dt(self.dtype),
                                         N.ptr(self._ws), C.c_size_t(self._ws.numel()), N.stream()), "gemm_4bit")

    def _run_layers(self, M: int):
        """Enqueue one step (all layers) on the current stream."""
        cfg, lib, g = self.cfg, N.lib(), self.world
        if self._persist:
            L = self.layers
            if g > 1:     # every rank has copied the previous step's result out of its h buffers
                N.check(lib.mpsbnb_flags_wait(N.ptr(self.acks), C.c_int(g), N.ptr(self.step_ctr), C.c_int(1), C.c_int(0),
                                              C.c_int(0), N.stream()), "flags_wait")
            N.check(lib.mpsbnb_gemv_4bit_group_run(C.byref(self._plans[0]), N.stream()), "gemv_4bit_group_run")
            if self._tagged:   # the result is complete when every entry carries the tag of "layer L"
                N.check(lib.mpsbnb_tagged_read(N.ptr(self.hbuf[L % self._nbuf]), N.i64(M), N.i64(cfg.hidden), N.ptr(self.h_out),
                                               N.ptr(self.step_ctr), C.c_int(L + 1), C.c_int(L), N.stream()), "tagged_read")
            else:
                if g > 1:     # ... and every rank's last shard has landed here
                    T = self._tiles_per_shard
                    N.check(lib.mpsbnb_flags_wait(N.ptr(self.flags), C.c_int(g), N.ptr(self.step_ctr), C.c_int(L * T), C.c_int(L * T),
                                                  C.c_int(0), N.stream()), "flags_wait")
                self.h_out.copy_(self.hbuf[L % self._nbuf])
            N.check(lib.mpsbnb_counter_add(N.ptr(self.step_ctr), C.c_int(1), N.stream()), "counter_add")
            if g > 1:
                N.check(lib.mpsbnb_flags_push(N.ptr(self._peer_acks), C.c_int(self.rank), C.c_int(g), N.ptr(self.step_ctr),
                                              C.c_int(1), C.c_int(0), N.stream()), "flags_push")
            return
        if self._plans is not None and self._fused:
            hs, L = cfg.hidden // g, self.layers
            for l in range(L):
                N.check(lib.mpsbnb_gemv_4bit_group_run(C.byref(self._plans[l]), N.stream()), "gemv_4bit_group_run")
                if self._inline:
                    continue
                N.check(lib.mpsbnb_stack_boundary_push(N.ptr(self.acc), C.c_float(self.alpha), N.i64(M), N.i64(hs),
                                                       N.i64(cfg.hidden), C.c_int(self.rank), C.c_int(g),
                                                       N.ptr(self._peer_h[(l + 1) % self._nbuf]), N.ptr(self._peer_flags),
                                                       N.ptr(self.step_ctr), C.c_int(L), C.c_int(l + 1), N.dt(self.dtype),
                                                       C.c_int(N.GROUP_PDL), N.stream()), "stack_boundary_push")
            # the step is complete here once every rank's last shard has landed; keep the result in a buffer no
            # peer writes, then tell the peers (acks) that this rank's h buffers may be overwritten again
            N.check(lib.mpsbnb_flags_wait(N.ptr(self.flags), C.c_int(g), N.ptr(self.step_ctr), C.c_int(L), C.c_int(L),
                                          C.c_int(1), N.stream()), "flags_wait")
            self.h_out.copy_(self.hbuf[L % self._nbuf])
            N.check(lib.mpsbnb_counter_add(N.ptr(self.step_ctr), C.c_int(1), N.stream()), "counter_add")
            N.check(lib.mpsbnb_flags_push(N.ptr(self._peer_acks), C.c_int(self.rank), C.c_int(g), N.ptr(self.step_ctr),
                                          C.c_int(1), C.c_int(0), N.stream()), "flags_push")
            return
        if self._plans is not None:
            hs = cfg.hidden // g
            for l in range(self.layers):
                N.check(lib.mpsbnb_gemv_4bit_group_run(C.byref(self._plans[l]), N.stream()), "gemv_4bit_group_run")
                if self._inline and g == 1:
                    continue
                dst = self.h if g == 1 else self.h_shard
                N.check(lib.mpsbnb_stack_boundary_acc(N.ptr(self.acc), C.c_float(self.alpha), N.i64(M * hs), N.ptr(dst),
                                                      N.dt(self.dtype), C.c_int(N.GROUP_PDL if self.use_pdl else 0),
                                                      N.stream()), "stack_boundary_acc")
                if g > 1:
                    torch.distributed.all_gather_into_tensor(self.gathered.view(g * M, -1), self.h_shard, group=self.group)
                    N.check(lib.mpsbnb_stack_expand(N.ptr(self.gathered), N.dt(self.dtype), N.i64(g), N.i64(M),
                                                    N.i64(cfg.hidden), N.i64(cfg.hidden), N.ptr(self.h), None,
                                                    N.stream()), "stack_expand")
            return
        for l in range(self.layers):
            for pr in self.proj[l]:
                self._gemv(pr, self.e if pr.name == "down" else self.h, self.out[pr.name], M)
            if g == 1:
                N.check(lib.mpsbnb_stack_boundary(N.ptr(self.out["o"]), N.ptr(self.out["down"]), N.dt(self.dtype),
                                                  C.c_float(self.alpha), N.i64(M), N.i64(cfg.hidden), N.i64(cfg.ffn),
                                                  N.ptr(self.h), N.ptr(self.e), N.stream()), "stack_boundary")
            else:
                hs = cfg.hidden // g
                N.check(lib.mpsbnb_stack_boundary(N.ptr(self.out["o"]), N.ptr(self.out["down"]), N.dt(self.dtype),
                                                  C.c_float(self.alpha), N.i64(M), N.i64(hs), N.i64(hs),
                                                  N.ptr(self.h_shard), None, N.stream()), "stack_boundary")
                torch.distributed.all_gather_into_tensor(self.gathered.view(g * M, -1), self.h_shard, group=self.group)
                N.check(lib.mpsbnb_stack_expand(N.ptr(self.gathered), N.dt(self.dtype), N.i64(g), N.i64(M),
                                                N.i64(cfg.hidden), N.i64(cfg.ffn), N.ptr(self.h), N.ptr(self.e),
                                                N.stream()), "stack_expand")

    # ------------------------------------------------------------------ public
    def prepare(self, M: int, use_graph: bool = True):
        """Allocate activations for batch M, and capture the step into a CUDA graph."""
        with torch.cuda.device(self.device):
            self._alloc(M)
            lib = N.lib()
            if M > lib.mpsbnb_gemv_4bit_max_m():
                big = max(lib.mpsbnb_gemm_4bit_workspace_bytes(N.i64(M), N.i64(p.n), N.i64(p.k), C.c_int(64))
                          for p in self.proj[0])
                self._ws = torch.empty(big, dtype=torch.uint8, device=self.device)
            self.x_in = torch.zeros(M, self.cfg.hidden, dtype=self.dtype, device=self.device)
            self._graph = None
            if use_graph:
                s = torch.cuda.Stream(device=self.device)
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._load_input()
                    self._run_layers(M)             # warm-up outside capture (function attributes, NCCL)
                torch.cuda.current_stream().wait_stream(s)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self._load_input()
                    self._run_layers(M)
                self._graph = graph

    def _load_input(self):
        """h = x_in, e = tile(x_in): the stack's input stage (uses the expand kernel with one rank)."""
        cfg = self.cfg
        if self._persist and getattr(self, "_tagged", False):
            N.check(N.lib().mpsbnb_tagged_write(N.ptr(self.x_in), N.i64(self._M), N.i64(cfg.hidden), N.ptr(self.hbuf[0]),
                                                N.ptr(self.step_ctr), C.c_int(self.layers + 1), C.c_int(0), N.stream()), "tagged_write")
            return
        N.check(N.lib().mpsbnb_stack_expand(N.ptr(self.x_in), N.dt(self.dtype), N.i64(1), N.i64(self._M),
                                            N.i64(cfg.hidden), N.i64(cfg.ffn), N.ptr(self._x_of_layer(0)), N.ptr(self.e),
                                            N.stream()), "stack_expand")

    def step(self, x: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One pass of all layers.  ``x`` [M, H] (device) replaces the input; returns h of the last layer."""
        if self._M is None:
            raise RuntimeError("call prepare(M) first")
        with torch.cuda.device(self.device):
            if x is not None:
                self.x_in.copy_(x, non_blocking=True)
            if self._graph is not None:
                self._graph.replay()
            else:
                self._load_input()
                self._run_layers(self._M)
        return self._result()

    def _result(self) -> torch.Tensor:
        if self._fused or self._persist:
            return self.h_out
        return self.hbuf[self.layers % self._nbuf] if self._stream else self.h

    def check_status(self, reset: bool = True) -> int:
        """Device status word of this stack's GPU: 0, or the code a kernel recorded when one of its bounded waits ran
        out (a peer that never raised its flag, a stage that never arrived).  A step whose status is not 0 returned
        with a wrong result; callers that need to know must poll this (it synchronises the device)."""
        with torch.cuda.device(self.device):
            st = C.c_int(0)
            N.check(N.lib().mpsbnb_device_status(C.byref(st), C.c_int(1 if reset else 0)), "device_status")
        return int(st.value)

    def output(self) -> torch.Tensor:
        """h after the last layer of the latest step."""
        return self._result()

    def launches_per_step(self) -> int:
        """Kernels of this library launched per step (NCCL's own kernels not counted)."""
        if self._persist:
            return 3 + (3 if self.world > 1 else 0)                  # input stage, the one GEMV launch, step counter (+ waits, acks)
        if self._plans is not None and self._fused:
            return 1 + self.layers * (1 if self._inline else 2) + 3                          # + flags_wait, counter_add, flags_push (the copy is torch's)
        if self._plans is not None and self.world == 1 and self._inline:
            return 1 + self.layers
        if self._plans is not None:
            return 1 + self.layers * (2 if self.world == 1 else 3)
        return 1 + self.layers * (7 + (1 if self.world == 1 else 2))
