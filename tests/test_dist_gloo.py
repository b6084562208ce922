"""CPU, world_size 2, gloo: the host-side sharding used for N > 1 and the max-over-ranks timing rule."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kda_b200.inputs import cu_seqlens_from_lengths, varlen_lengths
from kda_b200.shard import balance_sequences, batch_slice, take_sequences


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lengths = varlen_lengths(16, 128, 4096, seed=3)
    cu = cu_seqlens_from_lengths(lengths)
    owners = balance_sequences(lengths, world)
    x = torch.arange(int(cu[-1]), dtype=torch.float32).view(1, -1, 1)
    mine, my_cu = take_sequences(x, cu, owners[rank])
    # every rank reports (tokens, checksum); the union must be the whole batch exactly once
    stat = torch.tensor([float(mine.shape[1]), float(mine.sum())], dtype=torch.float64)
    allstat = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(allstat, stat)
    # timing rule: the reported time is the max over ranks
    t = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ret["tokens"] = [int(s[0]) for s in allstat]
        ret["sum"] = float(sum(s[1] for s in allstat))
        ret["total"] = int(cu[-1])
        ret["expect_sum"] = float(x.sum())
        ret["tmax"] = float(t)
        ret["my_cu_last"] = int(my_cu[-1])
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_and_timing():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert sum(ret["tokens"]) == ret["total"]
    assert ret["sum"] == ret["expect_sum"]
    assert max(ret["tokens"]) - min(ret["tokens"]) <= 4096          # balanced within one longest sequence
    assert ret["tmax"] == 11.0
    assert ret["my_cu_last"] == ret["tokens"][0]


def test_batch_slices_partition():
    for B in (1, 7, 8):
        for world in (1, 2, 4, 8):
            got = []
            for r in range(world):
                s = batch_slice(B, r, world)
                got.extend(range(B)[s])
            assert got == list(range(B))


def test_balance_is_a_partition_and_deterministic():
    lengths = varlen_lengths(64, 128, 16384, seed=0)
    a = balance_sequences(lengths, 8)
    assert sorted(i for o in a for i in o) == list(range(64))
    assert a == balance_sequences(lengths, 8)
    loads = [sum(lengths[i] for i in o) for o in a]
    assert max(loads) - min(loads) <= max(lengths)
