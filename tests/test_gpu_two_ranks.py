"""The N-sharded layer stack on two real GPUs (NCCL all-gather at every layer boundary) against the same
stack run whole on one GPU.  Skipped on a box with fewer than two GPUs; the host-side logic of the
sharding is covered on CPU (gloo) in test_sharding_cpu.py."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, M, fused, boundary, persistent, tagged=None):
    import torch.distributed as dist
    from mps_bitsandbytes_b200 import stack as S
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    cfg = S.StackConfig("tiny2", hidden=512, ffn=1024, kv=128, layers=3)
    x = torch.from_numpy(np.random.default_rng(7).standard_normal((M, cfg.hidden)).astype(np.float16)).cuda()
    whole = S.LayerStack(cfg, device=f"cuda:{rank}", seed=21)                   # the same model on every rank
    whole.prepare(M, use_graph=False)
    ref = whole.step(x).float().clone()
    part = S.LayerStack(cfg, device=f"cuda:{rank}", seed=21, rank=rank, world=world, fused_exchange=fused, boundary=boundary, persistent=persistent,
                        tagged_exchange=tagged)
    ok = True
    for use_graph in (False, True):
        part.prepare(M, use_graph=use_graph)
        for _ in range(2):
            h = part.step(x).float()
            torch.cuda.synchronize()
            err = float((h - ref).abs().max() / ref.abs().max())
            ok = ok and err <= 2e-3
    import ctypes as C
    from mps_bitsandbytes_b200 import _native
    code = C.c_int(0)
    ok = ok and _native.lib().mpsbnb_device_status(C.byref(code), C.c_int(1)) == 0 and code.value == 0
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    dist.barrier()
    # leave without tearing NCCL down under the captured graph
    os._exit(0 if int(flag.item()) == 1 else 1)


@pytest.mark.parametrize("M,fused,boundary,persistent,tagged", [
    (1, True, "kernel", False, None), (4, True, "inline", False, None), (1, True, "stream", False, None),
    (8, True, "stream", False, None), (1, True, "stream", True, None), (5, True, "stream", True, None),
    (1, True, "stream", True, True), (2, True, "stream", True, True),
    (1, False, "kernel", False, None), (16, True, "kernel", False, None)])
def test_two_rank_stack_matches_single_gpu(M, fused, boundary, persistent, tagged):
    """fused: peer stores at the layer boundary (batch <= 8) - with flags, or (one launch per step)
    as tagged entries when asked for; otherwise NCCL all-gather."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.spawn(_worker, args=(2, port, M, fused, boundary, persistent, tagged), nprocs=2, join=False)
    # bounded: a rank that never joins must not hold the suite
    for p in ctx.processes:
        p.join(timeout=180)
    alive = [p for p in ctx.processes if p.is_alive()]
    for p in alive:
        p.kill()
    assert not alive, "a rank did not finish within 180 s"
    assert all(p.exitcode == 0 for p in ctx.processes), [p.exitcode for p in ctx.processes]
