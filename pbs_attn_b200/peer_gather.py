"""Head-sharded prefill whose outputs land in every rank's full tensor from the attention kernel itself.

``sharding.gather_heads`` runs an NCCL all-gather after the call: the transfer starts when the last
head is done and nothing hides it.  Here every rank allocates the full (B, Hq, S, D) result, the
ranks exchange CUDA IPC handles of those buffers once, and the epilogue of the tcgen05 attention
kernel stores each finished output tile into its own buffer AND, with plain stores over NVLink, into
the same place of every peer's buffer (``pbs_out_replicas_t`` in include/pbs_b200.h).  The transfer is
spread over the whole kernel; what remains after it is one tiny all-reduce that tells every rank
that all peers' kernels (hence their stores into its buffer) have completed.

Only plain peer stores are used: no multicast, no TMA access to peer memory, and no library kernel
is handed a peer pointer.  One process per GPU, all GPUs of one node.  In a Hugging Face
tensor-parallel deployment (what the reference runs, pbs_attn/patch/huggingface.py:194-199) no gather
is needed at all; this is for callers that want the whole (B, Hq, S, D) tensor on every rank.
"""
from __future__ import annotations

import ctypes as C
from typing import List

import torch
import torch.distributed as dist

from . import _cabi
from .sharding import HeadShard, shard_heads


class FusedHeadGather:
    """Full-result buffers of one shape on every rank, mapped into each other's address space.

    ``buffers`` full tensors are kept and used in turn, so that a consumer may still read the result
    of call i while call i + 1 is being written (call i + 2 reuses call i's buffer).
    """

    def __init__(self, batch: int, q_heads: int, kv_heads: int, seq_len: int, head_dim: int, dtype: torch.dtype,
                 device, group=None, buffers: int = 2):
        if not dist.is_initialized():
            raise RuntimeError("FusedHeadGather needs an initialised process group (one process per GPU)")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.shard: HeadShard = shard_heads(q_heads, kv_heads, self.rank, self.world)
        if self.world - 1 > _cabi.MAX_OUT_REPLICAS:
            raise ValueError(f"{self.world} ranks: at most {_cabi.MAX_OUT_REPLICAS + 1} are supported")
        self.lib = _cabi.load()
        self.full: List[torch.Tensor] = [torch.empty(batch, q_heads, seq_len, head_dim, dtype=dtype, device=self.device)
                                         for _ in range(buffers)]
        self._mapped = {}                 # handle bytes -> base pointer of the mapping in this process
        self._replicas: List[_cabi.OutReplicas] = []
        ok, err = 1, ""
        try:
            self._exchange()
        except Exception as e:            # every rank must learn of a failure, or the others would hang
            ok, err = 0, f"{type(e).__name__}: {e}"
        flag = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            self.close()
            raise RuntimeError("peer mapping of the result buffers failed on some rank" + (f" (here: {err})" if err else ""))
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._calls = 0

    def _exchange(self):
        mine = []
        with torch.cuda.device(self.device):
            for t in self.full:
                handle = (C.c_ubyte * 64)()
                off = C.c_int64(0)
                _cabi.check(self.lib.pbs_ipc_export(C.c_void_p(t.data_ptr()), C.byref(handle), C.byref(off)), "pbs_ipc_export")
                mine.append((bytes(handle), int(off.value)))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, (self.device.index, mine), group=self.group)
        sl = self.shard.q_slice
        ref = self.full[0]
        # byte offset of this rank's head range inside a full tensor (identical layout on every rank)
        slice_off = ref[:, sl].data_ptr() - ref.data_ptr()
        reps = [_cabi.OutReplicas() for _ in self.full]
        with torch.cuda.device(self.device):
            for r, (peer_dev, descs) in enumerate(everyone):
                if r == self.rank:
                    continue
                _cabi.check(self.lib.pbs_enable_peer_access(int(peer_dev)), "pbs_enable_peer_access")
                for i, (handle, off) in enumerate(descs):
                    base = self._mapped.get(handle)
                    if base is None:
                        hbuf = (C.c_ubyte * 64).from_buffer_copy(handle)
                        p = C.c_void_p()
                        _cabi.check(self.lib.pbs_ipc_import(C.byref(hbuf), C.byref(p)), "pbs_ipc_import")
                        base = self._mapped[handle] = int(p.value)
                    rep = reps[i]
                    rep.out[rep.count] = base + off + slice_off
                    rep.count += 1
        self._replicas = reps

    def close(self):
        """Unmaps the peers' buffers (the tensors of this rank stay valid)."""
        with torch.cuda.device(self.device):
            for base in self._mapped.values():
                self.lib.pbs_ipc_release(C.c_void_p(base))
        self._mapped = {}
        self._replicas = []

    def next_slot(self):
        """(local output view, replicas struct, full tensor) of the next call."""
        i = self._calls % len(self.full)
        self._calls += 1
        return self.full[i][:, self.shard.q_slice], self._replicas[i], self.full[i]

    def complete(self):
        """Enqueues the cross-rank completion point on the current stream: after it, every rank's
        heads have arrived in this rank's full tensor."""
        dist.all_reduce(self._flag, group=self.group)


def permuted_block_sparse_attn_fwd_gathered(gather: FusedHeadGather, q_local, k_local, v_local, block_size, segment_size,
                                            threshold, **kwargs) -> torch.Tensor:
    """One head-sharded call: this rank's query heads (and the KV heads they read) in, the FULL
    (B, Hq, S, D) result out, valid on every rank once the current stream has passed this call.
    Only shapes the tcgen05 attention kernel covers (bf16/fp16, head_dim 64/128, block 64/128)."""
    from .prefill import permuted_block_sparse_attn_fwd
    out_view, replicas, full = gather.next_slot()
    permuted_block_sparse_attn_fwd(q_local, k_local, v_local, block_size, segment_size, threshold, True,
                                   attn_impl="tcgen05", out=out_view, out_replicas=replicas, **kwargs)
    gather.complete()
    return full
