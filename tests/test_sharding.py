"""Multi-GPU partitioning logic, on CPU: pure functions plus a world_size-2 gloo run that
checks the shards of two ranks reassemble to the single-process result bit for bit."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_attn_triton_b200 import sharding as sh

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_covers_everything():
    for n in (0, 1, 7, 256, 257):
        for world in (1, 2, 3, 8):
            spans = [sh.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sh.shard_range(4, 2, 2)


def test_causal_pairs():
    assert sh.causal_pairs(4) == 10
    assert sh.causal_pairs(5, window_left=1) == 1 + 2 + 2 + 2 + 2
    # brute force
    for L in (1, 9, 40):
        for w in (-1, 0, 3, 100):
            brute = sum(1 for i in range(L) for j in range(L) if j <= i and (w < 0 or j >= i - w))
            assert sh.causal_pairs(L, w) == brute


def test_balance_sequences():
    lens = [4096, 256, 256, 3000, 1024, 512, 2048, 64]
    for world in (1, 2, 4, 8):
        owned = sh.balance_sequences(lens, world, window_left=1024)
        assert sorted(i for o in owned for i in o) == list(range(len(lens)))
        loads = [sum(sh.causal_pairs(lens[i], 1024) for i in o) for o in owned]
        assert max(loads) <= sum(loads) / world + max(sh.causal_pairs(l, 1024) for l in lens)


def _unit_tensor(seed, unit):
    g = torch.Generator().manual_seed(sh.unit_seed(seed, unit))
    return torch.randn(8, 4, generator=g)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_units = 10
    lo, hi = sh.shard_range(n_units, rank, world)
    mine = torch.stack([_unit_tensor(3, u) * 2 + 1 for u in range(lo, hi)])  # stand-in "kernel"
    sizes = [sh.shard_range(n_units, r, world) for r in range(world)]
    bufs = [torch.empty(b - a, 8, 4) for a, b in sizes]
    dist.all_gather(bufs, mine)
    if rank == 0:
        torch.save(torch.cat(bufs), os.path.join(out_dir, "gathered.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reassemble(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(os.path.join(tmp_path, "gathered.pt"))
    want = torch.stack([_unit_tensor(3, u) * 2 + 1 for u in range(10)])
    assert torch.equal(got, want)
