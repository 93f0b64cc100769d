"""Host-side logic of the N-sharded stack on CPU: shard arithmetic, byte accounting, and — as two
gloo ranks — that all-gathered [M, H/g] shards re-assemble into the replicated [M, H] activation
in the layout the device-side expand kernel assumes."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mps_bitsandbytes_b200 import stack as S


def test_shard_rows_and_byte_accounting():
    assert S.shard_rows(4096, 0, 8) == (0, 512) and S.shard_rows(4096, 7, 8) == (3584, 4096)
    with pytest.raises(ValueError):
        S.shard_rows(10, 0, 3)
    assert S.LLAMA2_7B.params_per_layer() == 202375168
    assert S.LLAMA_70B.params_per_layer() == 855638016
    assert S.weight_bytes(S.LLAMA2_7B) == 3340771328
    # every shard of every projection keeps double-quant groups (256 blocks) whole, up to 8 ranks
    for cfg in (S.LLAMA2_7B, S.LLAMA_70B):
        for world in (2, 4, 8):
            for _, n, k in cfg.projections():
                assert (n // world * (k // 64)) % 256 == 0
    assert abs(S.LLAMA2_7B.alpha() - 1 / (0.02 * (4096 + 11008) ** 0.5)) < 1e-12


def _worker(rank, world, port, M, H):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = torch.arange(M * H, dtype=torch.float32).view(M, H)
    lo, hi = S.shard_rows(H, rank, world)
    shard = full[:, lo:hi].contiguous()                     # this rank's columns of h
    gathered = torch.empty(world, M, H // world)
    dist.all_gather_into_tensor(gathered.view(world * M, H // world), shard)   # gloo wants rank-major rows
    assert torch.equal(S.gathered_to_full(gathered), full)
    dist.barrier()
    dist.destroy_process_group()


def test_all_gather_layout_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, 3, 8), nprocs=2, join=True)
