"""Head (and batch) sharding of one prefill call across the GPUs of a node.

Every (batch, query head) of the path is independent end to end -- own importance scores,
permutation, block mask and attention (reference: pbs_attn/src/permute_states.py:44-56, grid of
pbs_attn/src/pbs.py:221-222) -- so ranks take disjoint query heads and exchange nothing while
computing.  This is also how the reference is deployed: Hugging Face tensor parallelism gives each
rank a slice of the heads and the patch derives the local head counts from the projection widths
(pbs_attn/patch/huggingface.py:194-199).  The only collective is an all-gather of the outputs when
the caller wants the full (B, Hq, S, D) tensor on every rank.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    q_start: int      # first query head of this rank
    q_count: int
    kv_start: int     # first KV head this rank reads
    kv_count: int

    @property
    def q_slice(self):
        return slice(self.q_start, self.q_start + self.q_count)

    @property
    def kv_slice(self):
        return slice(self.kv_start, self.kv_start + self.kv_count)


def shard_heads(q_heads: int, kv_heads: int, rank: int, world: int) -> HeadShard:
    """KV-head groups are dealt out whole while there are enough of them (world <= Hkv, world
    divides Hkv); with more ranks than KV heads (world a multiple of Hkv) the query heads inside a
    group are split as evenly as possible and the ranks of a group all read its one KV head."""
    assert q_heads % kv_heads == 0 and 0 <= rank < world
    group = q_heads // kv_heads
    if world <= kv_heads:
        if kv_heads % world:
            raise ValueError(f"{world} ranks do not divide {kv_heads} KV heads")
        per = kv_heads // world
        return HeadShard(rank * per * group, per * group, rank * per, per)
    if world % kv_heads:
        raise ValueError(f"{world} ranks is not a multiple of {kv_heads} KV heads")
    ways = world // kv_heads                    # ranks per KV group
    if ways > group:
        raise ValueError(f"{world} ranks exceed the {q_heads} query heads")
    kv, part = divmod(rank, ways)
    base, extra = divmod(group, ways)           # e.g. 7 query heads over 2 ranks -> 4 + 3
    start = part * base + min(part, extra)
    count = base + (1 if part < extra else 0)
    return HeadShard(kv * group + start, count, kv, 1)


def shard_batch(batch: int, rank: int, world: int) -> slice:
    """Multi-sequence prefill: whole sequences per rank, as evenly as possible (the first
    ``batch % world`` ranks take one more); sequences are independent, so nothing is exchanged
    while computing.  Ranks beyond the batch get an empty slice."""
    assert 0 <= rank < world
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def gather_batch(local_out: torch.Tensor, batch: int, group=None) -> torch.Tensor:
    """All-gathers per-rank (B_local, Hq, S, D) outputs of ``shard_batch`` into (batch, Hq, S, D)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    _, H, S, D = local_out.shape
    parts = [shard_batch(batch, r, world) for r in range(world)]
    bmax = max(p.stop - p.start for p in parts)
    send = torch.zeros(bmax, H, S, D, dtype=local_out.dtype, device=local_out.device)
    send[: local_out.shape[0]] = local_out
    recv = torch.empty(world, bmax, H, S, D, dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(recv.view(-1), send.view(-1), group=group)
    full = torch.empty(batch, H, S, D, dtype=local_out.dtype, device=local_out.device)
    for r, p in enumerate(parts):
        full[p] = recv[r, : p.stop - p.start]
    return full


def all_shards(q_heads: int, kv_heads: int, world: int):
    return [shard_heads(q_heads, kv_heads, r, world) for r in range(world)]


def gather_heads(local_out: torch.Tensor, q_heads: int, kv_heads: int, group=None) -> torch.Tensor:
    """All-gathers the per-rank (B, Hq_local, S, D) outputs into (B, Hq, S, D) on every rank.

    Equal shards with batch 1 go through one ``all_gather_into_tensor`` straight into the result;
    otherwise every rank sends a buffer padded to the largest shard (collectives need equal sizes)
    and each shard is copied to its head range.
    """
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    shards = all_shards(q_heads, kv_heads, world)
    B, _, S, D = local_out.shape
    local_out = local_out.contiguous()
    even = len({s.q_count for s in shards}) == 1
    if even and B == 1:
        full = torch.empty(B, q_heads, S, D, dtype=local_out.dtype, device=local_out.device)
        dist.all_gather_into_tensor(full.view(-1), local_out.view(-1), group=group)
        return full
    hmax = max(s.q_count for s in shards)
    send = local_out
    if local_out.shape[1] != hmax:
        send = torch.zeros(B, hmax, S, D, dtype=local_out.dtype, device=local_out.device)
        send[:, : local_out.shape[1]] = local_out
    recv = torch.empty(world, B, hmax, S, D, dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(recv.view(-1), send.view(-1), group=group)
    full = torch.empty(B, q_heads, S, D, dtype=local_out.dtype, device=local_out.device)
    for r, s in enumerate(shards):
        full[:, s.q_slice] = recv[r, :, : s.q_count]
    return full
