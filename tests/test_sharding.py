"""Head sharding: shard arithmetic, and the output all-gather on two CPU ranks over gloo."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pbs_attn_b200.sharding import all_shards, gather_heads, shard_heads


@pytest.mark.parametrize("hq,hkv,world", [(32, 8, 1), (32, 8, 2), (32, 8, 4), (32, 8, 8), (28, 4, 4), (28, 4, 8), (4, 1, 2)])
def test_shards_partition_the_heads(hq, hkv, world):
    shards = all_shards(hq, hkv, world)
    seen = []
    for s in shards:
        seen += list(range(s.q_start, s.q_start + s.q_count))
        group = hq // hkv
        # every query head of the shard maps onto a KV head the shard holds
        for h in range(s.q_start, s.q_start + s.q_count):
            assert s.kv_start <= h // group < s.kv_start + s.kv_count
    assert seen == list(range(hq))


def test_qwen_heads_over_eight_ranks_split_4_3():
    counts = [s.q_count for s in all_shards(28, 4, 8)]
    assert counts == [4, 3] * 4


def test_bad_world_sizes():
    with pytest.raises(ValueError):
        shard_heads(32, 8, 0, 3)
    with pytest.raises(ValueError):
        shard_heads(4, 4, 0, 8)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, hq, hkv, batch, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = shard_heads(hq, hkv, rank, world)
        full = torch.arange(batch * hq * 6 * 4, dtype=torch.float32).view(batch, hq, 6, 4)
        got = gather_heads(full[:, sh.q_slice].clone(), hq, hkv)
        q.put((rank, bool(torch.equal(got, full))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("hq,hkv,batch", [(8, 2, 1), (7, 1, 1), (8, 2, 2)])
def test_gather_heads_two_ranks_gloo(hq, hkv, batch):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, hq, hkv, batch, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == [(0, True), (1, True)]


def test_batch_shards_partition_the_sequences():
    from pbs_attn_b200.sharding import shard_batch
    for batch, world in [(8, 8), (8, 2), (5, 2), (3, 4), (1, 2)]:
        parts = [shard_batch(batch, r, world) for r in range(world)]
        assert [i for p in parts for i in range(p.start, p.stop)] == list(range(batch))
        sizes = [p.stop - p.start for p in parts]
        assert max(sizes) - min(sizes) <= 1


def _batch_worker(rank, world, port, batch, q):
    from pbs_attn_b200.sharding import gather_batch, shard_batch
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(batch * 2 * 6 * 4, dtype=torch.float32).view(batch, 2, 6, 4)
        got = gather_batch(full[shard_batch(batch, rank, world)].clone(), batch)
        q.put((rank, bool(torch.equal(got, full))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [4, 3, 1])
def test_gather_batch_two_ranks_gloo(batch):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_batch_worker, args=(r, 2, port, batch, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == [(0, True), (1, True)]
