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


def test_batch_head_blocks_partition_the_units():
    from kda_b200.shard import batch_head_block
    for B, H in ((8, 32), (4, 32), (1, 32)):
        for world in (1, 2, 4, 8):
            if world > B and (world % B or H % (world // B)):
                continue
            seen = set()
            for r in range(world):
                b0, b1, h0, h1 = batch_head_block(B, H, r, world)
                block = {(b, h) for b in range(b0, b1) for h in range(h0, h1)}
                assert block and not (block & seen)
                seen |= block
            assert len(seen) == B * H
    assert batch_head_block(4, 32, 5, 8) == (2, 3, 16, 32)          # two ranks per batch row: the second takes heads 16..31


def _bench_shard_worker(rank, world, port, ret):
    """The benchmark's own sharding of the headline workload (bench.shard_inputs), shrunk: the union of the ranks' batch
    rows is the batch a single rank would generate, row for row."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import argparse
    import dataclasses
    import bench
    from kda_b200.inputs import WORKLOADS
    w = dataclasses.replace(WORKLOADS["train_bf16"], B=4, T=16, H=2)
    args = argparse.Namespace(workload="train_bf16", weak=False, scale_down=1)
    mine, cu, job_tokens = bench.shard_inputs(args, w, rank, world, None)
    whole, _, _ = bench.shard_inputs(args, w, 0, 1, None)
    sl = batch_slice(4, rank, world)
    ok = all(torch.equal(mine[n], whole[n][sl]) for n in mine) and cu is None and job_tokens == 4 * 16
    flags = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(flags, torch.tensor([1.0 if ok else 0.0]))
    if rank == 0:
        ret["ok"] = [bool(f.item()) for f in flags]
        ret["rows"] = mine["q"].shape[0]
    dist.barrier()
    dist.destroy_process_group()


def test_bench_shards_the_headline_batch_over_two_ranks():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_bench_shard_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret["ok"] == [True, True] and ret["rows"] == 2
