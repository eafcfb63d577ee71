"""Head-sharded call on two GPUs of one node (skipped with fewer): the attention kernel of every rank
stores its heads into both ranks' full result tensors (plain peer stores, pbs_attn_b200.peer_gather), and the
result must equal the NCCL all-gather of the same shards and a one-GPU run of all heads, bit for bit.
Also one small case with tensors on cuda:1 while cuda:0 is the current device."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q_heads, kv_heads, result):
    import torch.distributed as dist
    from pbs_attn_b200.peer_gather import FusedHeadGather, permuted_block_sparse_attn_fwd_gathered
    from pbs_attn_b200.prefill import permuted_block_sparse_attn_fwd
    from pbs_attn_b200.sharding import gather_heads, shard_heads
    from pbs_attn_b200.synth import Workload, make_qkv_heads
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        w = Workload("multi", 2, q_heads, kv_heads, 128, 4096, "bf16", 128, 256, 0.9, 5e5, sinks=4)
        sh = shard_heads(w.q_heads, w.kv_heads, rank, world)
        q, k, v = make_qkv_heads(w, 3, sh.kv_start, sh.kv_count, sh.q_start, sh.q_count, device=dev)
        fq, fk, fv = make_qkv_heads(w, 3, 0, w.kv_heads, device=dev)
        want = permuted_block_sparse_attn_fwd(fq, fk, fv, w.block_size, w.segment_size, w.threshold, True)
        gather = FusedHeadGather(w.batch, w.q_heads, w.kv_heads, w.seq_len, w.head_dim, q.dtype, dev)
        ok = True
        for _ in range(3):                                  # three calls: both result buffers get reused
            full = permuted_block_sparse_attn_fwd_gathered(gather, q, k, v, w.block_size, w.segment_size, w.threshold)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(full, want))
        local = permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, w.threshold, True)
        nccl = gather_heads(local, w.q_heads, w.kv_heads)
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(nccl, want))
        flag = torch.tensor([int(ok)], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        gather.close()
        if rank == 0:
            result.put(int(flag.item()))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("q_heads,kv_heads", [(8, 2), (7, 1)])     # whole KV groups per rank; query heads split 4 + 3
def test_fused_head_gather_on_two_gpus(q_heads, kv_heads):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    mp.spawn(_worker, args=(2, _free_port(), q_heads, kv_heads, result), nprocs=2, join=True)
    assert result.get(timeout=10) == 1


def test_tensors_on_another_device_than_the_current_one():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from pbs_attn_b200.prefill import key_importance_static, permuted_block_sparse_attn_fwd
    from pbs_attn_b200.synth import Workload, make_qkv
    w = Workload("dev1", 1, 4, 1, 128, 2048, "bf16", 128, 256, 0.9, 5e5, sinks=4)
    q, k, v = make_qkv(w, seed=9)
    want = permuted_block_sparse_attn_fwd(q.cuda(0), k.cuda(0), v.cuda(0), w.block_size, w.segment_size, w.threshold, True)
    imp0 = key_importance_static(q.cuda(0), k.cuda(0), w.block_size, w.segment_size)
    torch.cuda.set_device(0)
    got = permuted_block_sparse_attn_fwd(q.cuda(1), k.cuda(1), v.cuda(1), w.block_size, w.segment_size, w.threshold, True)
    imp1 = key_importance_static(q.cuda(1), k.cuda(1), w.block_size, w.segment_size)
    torch.cuda.synchronize(1)
    assert got.device.index == 1 and torch.equal(got.cpu(), want.cpu())
    assert imp1.device.index == 1 and torch.equal(imp1.cpu(), imp0.cpu())
