"""Host-side sharding of the independent (sequence, head) recurrences over the GPUs of one box.

There is no exchange step in KDA's forward or backward when value heads == key heads, so every rank
works on a disjoint shard and the only cross-rank traffic is the barrier / timing reduction of a
benchmark.  Equal-length batches are split along the batch axis (contiguous slices); packed
variable-length batches are split by whole sequences, balanced by token count (longest first).
"""
from __future__ import annotations

import torch


def batch_slice(B: int, rank: int, world: int) -> slice:
    """Contiguous batch slice of `rank`; sizes differ by at most one."""
    base, rem = divmod(B, world)
    start = rank * base + min(rank, rem)
    return slice(start, start + base + (1 if rank < rem else 0))


def batch_head_block(B: int, H: int, rank: int, world: int) -> tuple[int, int, int, int]:
    """Contiguous block of the B*H flattened (batch, head) units for `rank`, as (b0, b1, h0, h1): whole batch rows
    while there are at least as many rows as ranks, otherwise a head range of one row (world must then be a multiple
    of B and H a multiple of world // B), so that every rank's slice stays a dense sub-tensor."""
    if world <= B:
        sl = batch_slice(B, rank, world)
        return sl.start, sl.stop, 0, H
    if world % B or H % (world // B):
        raise ValueError(f"cannot cut {B} x {H} (batch, head) units into {world} dense blocks")
    per = world // B
    hs = H // per
    b, j = divmod(rank, per)
    return b, b + 1, j * hs, (j + 1) * hs


def balance_sequences(lengths, world: int) -> list[list[int]]:
    """Longest-processing-time assignment of whole sequences to ranks; returns per-rank sequence ids
    (each list in ascending id order so that a rank's packed tensor keeps the original order)."""
    loads = [0] * world
    owners: list[list[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i)):
        r = min(range(world), key=lambda r: (loads[r], r))
        owners[r].append(i)
        loads[r] += int(lengths[i])
    return [sorted(o) for o in owners]


def take_sequences(x: torch.Tensor, cu_seqlens, seq_ids):
    """Packs the chosen sequences of a [1, T, ...] tensor; returns (packed, rebased int32 cu_seqlens)."""
    cu = [int(c) for c in cu_seqlens]
    parts = [x[:, cu[i]:cu[i + 1]] for i in seq_ids]
    new_cu = [0]
    for i in seq_ids:
        new_cu.append(new_cu[-1] + cu[i + 1] - cu[i])
    packed = torch.cat(parts, dim=1) if parts else x[:, :0]
    return packed, torch.tensor(new_cu, dtype=torch.int32)
