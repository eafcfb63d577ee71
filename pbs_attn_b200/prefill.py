"""Host side of the prefill path: shapes, scratch memory and the calls into libpbs_b200.so.

``permuted_block_sparse_attn_fwd`` has the signature and argument meaning of the
reference's function of the same name (pbs_attn/src/pbs.py:132-146).  PyTorch is used
for device memory and streams only; all arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional, Union

import torch

from . import _cabi

_DTYPES = {torch.bfloat16: _cabi.BF16, torch.float16: _cabi.FP16, torch.float32: _cabi.FP32}
_STATUS_SLOTS = 16      # whole-path calls whose status words may be in flight to the host at once


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _strides(t: torch.Tensor):
    return _cabi.Strides4(*t.stride())


def _readable(t: torch.Tensor, need_distinct_heads: bool = False) -> torch.Tensor:
    """Returns ``t`` if the kernels can read it in place (unit head-dim stride, 16-byte aligned
    rows), else a contiguous copy."""
    e = t.element_size()
    ok = (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and t.stride(2) > 0
          and all((s * e) % 16 == 0 and s >= 0 for s in t.stride()[:3]))
    if ok and need_distinct_heads:
        # the TMA descriptor of the query tensor cannot describe broadcast (stride-0) batch / head dims
        ok = all(st > 0 or n == 1 for st, n in zip(t.stride()[:2], t.shape[:2]))
    return t if ok else t.contiguous()


class Plan:
    """Shape, scratch buffers and stage calls for one (shape, device).

    Scratch lives in torch tensors (the library never allocates).  The stage methods map
    one-to-one onto the C entry points; ``run`` is the whole path.
    """

    def __init__(self, batch, q_heads, kv_heads, seq_len, head_dim, block_size, segment_size,
                 dtype: torch.dtype, device):
        if dtype not in _DTYPES:
            raise TypeError(f"unsupported dtype {dtype}: need bfloat16, float16 or float32")
        self.lib = _cabi.load()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("pbs_attn_b200 runs on CUDA devices only; there is no CPU path")
        self.dtype = dtype
        self.shape = _cabi.Shape(batch, q_heads, kv_heads, seq_len, head_dim, block_size, segment_size, _DTYPES[dtype])
        sizes = _cabi.ScratchSizes()
        _cabi.check(self.lib.pbs_scratch_sizes(C.byref(self.shape), C.byref(sizes)), "pbs_scratch_sizes")
        self.dense = seq_len <= segment_size
        self.nb = -(-seq_len // block_size)
        self.n_complete = (seq_len // segment_size) * segment_size
        dev = self.device

        def buf(n, dt):
            return torch.empty(max(int(n), 1), dtype=dt, device=dev)

        B, H, S, D = batch, q_heads, seq_len, head_dim
        self.logits = None                 # optional inspection output of stage 1a, allocated on demand
        self._logits_numel = int(sizes.logits)
        self.partials = buf(0 if self.dense else 2 * sizes.partials, torch.float32)
        self.rowstats = buf(2 * sizes.rowstats, torch.float32)
        self.importance = buf(sizes.importance, torch.float32)
        self.key_indices = buf(sizes.key_indices, torch.int32).view(B, H, S)
        self.perm_k = buf(sizes.perm_kv, dtype).view(B, H, S, D)
        self.perm_v = buf(sizes.perm_kv, dtype).view(B, H, S, D)
        self.pooled_q = buf(sizes.pooled, dtype).view(B, H, self.nb, D)
        self.pooled_k = buf(sizes.pooled, dtype).view(B, H, self.nb, D)
        self.first_block = torch.zeros(max(int(sizes.first_block), 1), dtype=torch.int32, device=dev)
        self.block_mask = buf(sizes.block_mask, torch.uint8).view(B, H, self.nb, self.nb)
        self.tile_list = buf(sizes.tile_list, torch.int32)
        self.tile_count = buf(sizes.tile_count, torch.int32)
        self.status = torch.zeros(int(sizes.status), dtype=torch.int32, device=dev)
        self.scratch = _cabi.Scratch(None, *[t.data_ptr() for t in (
            self.partials, self.rowstats, self.importance, self.key_indices, self.perm_k,
            self.perm_v, self.pooled_q, self.pooled_k, self.first_block, self.block_mask, self.tile_list,
            self.tile_count, self.status)])
        self._thr_dev = None
        # deferred status check: after every whole-path call the 8 status words are copied to pinned
        # host memory (asynchronously); the copies that have landed are inspected on entry to the next call
        self._status_ring = torch.zeros(_STATUS_SLOTS, 8, dtype=torch.int32).pin_memory()
        self._status_pending = []          # [(event, slot)], oldest first
        self._status_next = 0

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _on_device(self):
        """The library launches on the CURRENT device: make this plan's device current around every call."""
        return torch.cuda.device(self.device)

    def _raise_status(self, words):
        raise _cabi.PbsError(f"device-side error flags {list(words)}: a bounded wait in the attention kernel ran out "
                             f"(code {int(words[0])}); the output of that call is invalid")

    def _inspect_landed_status(self, wait_all: bool = False):
        while self._status_pending:
            ev, slot = self._status_pending[0]
            if wait_all or len(self._status_pending) >= _STATUS_SLOTS:
                ev.synchronize()
            elif not ev.query():
                break
            self._status_pending.pop(0)
            words = self._status_ring[slot].tolist()
            if words[0] != 0:
                self._status_pending.clear()
                self._raise_status(words)

    def _queue_status_copy(self):
        slot = self._status_next
        self._status_next = (slot + 1) % _STATUS_SLOTS
        self._status_ring[slot].copy_(self.status, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._status_pending.append((ev, slot))

    def options(self, threshold, force_select_first_block=True, query_pool_mode="mean", key_pool_mode="mean",
                attn_impl="auto", no_permutation=False, diagonal_candidates=False, no_own_segment=False,
                out_replicas: Optional[_cabi.OutReplicas] = None) -> _cabi.Options:
        for m in (query_pool_mode, key_pool_mode):
            if m not in _cabi.POOL:
                raise ValueError(f"Invalid pool mode: {m}")
        thr_ptr, thr, select_all = None, 0.0, 0
        if isinstance(threshold, torch.Tensor):
            self._thr_dev = threshold.detach().to(device=self.device, dtype=torch.float32).reshape(-1).contiguous()
            if self._thr_dev.numel() != self.shape.q_heads:
                raise ValueError("a tensor threshold must hold one value per query head")
            thr_ptr = self._thr_dev.data_ptr()
        elif isinstance(threshold, int) and not isinstance(threshold, bool) and threshold == 1:
            select_all = 1          # the reference takes every candidate block for the int 1
        else:
            thr = float(threshold)
        opt = _cabi.Options(thr_ptr, thr, select_all, int(bool(force_select_first_block)),
                            _cabi.POOL[query_pool_mode], _cabi.POOL[key_pool_mode], _cabi.ATTN_IMPL[attn_impl],
                            int(bool(no_permutation)), int(bool(diagonal_candidates)), int(bool(no_own_segment)),
                            C.pointer(out_replicas) if out_replicas is not None else None)
        opt._keep = out_replicas            # the struct must outlive the call
        return opt

    def check_status(self):
        """Synchronises and raises if a kernel reported a device-side error (in the last call or in an
        earlier whole-path call whose status has not been inspected yet)."""
        self._inspect_landed_status(wait_all=True)
        st = self.status.cpu()
        if int(st[0]) != 0:
            self._raise_status(st.tolist())

    # ------------------------------------------------------------------ stages
    def key_importance(self, q, k, want_logits: bool = False):
        """Returns the (B, Hq, L) importance; with ``want_logits`` also the (B, Hq, block_size, L)
        rounded scoring logits (for inspection and tests)."""
        if want_logits and self.logits is None:
            self.logits = torch.empty(max(self._logits_numel, 1), dtype=self.dtype, device=self.device)
        with self._on_device():
            _cabi.check(self.lib.pbs_key_importance(C.byref(self.shape), _ptr(q), _strides(q), _ptr(k), _strides(k),
                                                    _ptr(self.logits if want_logits else None), _ptr(self.partials),
                                                    _ptr(self.rowstats), _ptr(self.importance), self._stream()),
                        "pbs_key_importance")
        B, H, L = self.shape.batch, self.shape.q_heads, self.n_complete
        imp = self.importance[: B * H * L].view(B, H, L)
        if want_logits:
            return imp, self.logits[: B * H * self.shape.block_size * L].view(B, H, self.shape.block_size, L)
        return imp

    def segment_permute(self, k, v, key_pool_mode="mean", identity=False):
        imp = None if identity else _ptr(self.importance)
        with self._on_device():
            _cabi.check(self.lib.pbs_segment_permute(C.byref(self.shape), imp, _ptr(k), _strides(k), _ptr(v), _strides(v),
                                                     _ptr(self.key_indices), _ptr(self.perm_k), _ptr(self.perm_v),
                                                     _ptr(self.pooled_k), _cabi.POOL[key_pool_mode],
                                                     _ptr(self.first_block), self._stream()), "pbs_segment_permute")

    def pool_queries(self, q, query_pool_mode="mean"):
        with self._on_device():
            _cabi.check(self.lib.pbs_pool_queries(C.byref(self.shape), _ptr(q), _strides(q), _ptr(self.pooled_q),
                                                  _cabi.POOL[query_pool_mode], self._stream()), "pbs_pool_queries")

    def select_blocks(self, opt: _cabi.Options, want_scores: bool = False):
        """Returns the (B, Hq, nb, nb) fp32 pooled scores when ``want_scores`` (else None)."""
        scores = None
        if want_scores:
            scores = torch.empty(self.block_mask.shape, dtype=torch.float32, device=self.device)
        with self._on_device():
            _cabi.check(self.lib.pbs_select_blocks(C.byref(self.shape), _ptr(self.pooled_q), _ptr(self.pooled_k),
                                                   _ptr(self.first_block), C.byref(opt), _ptr(self.block_mask),
                                                   _ptr(scores), self._stream()), "pbs_select_blocks")
        return scores

    def build_tile_lists(self):
        with self._on_device():
            _cabi.check(self.lib.pbs_build_tile_lists(C.byref(self.shape), _ptr(self.block_mask), _ptr(self.tile_list),
                                                      _ptr(self.tile_count), self._stream()), "pbs_build_tile_lists")

    def attn_fwd(self, q, out, attn_impl="auto"):
        self.status.zero_()
        with self._on_device():
            _cabi.check(self.lib.pbs_attn_fwd(C.byref(self.shape), _ptr(q), _strides(q), _ptr(self.perm_k), _ptr(self.perm_v),
                                              _ptr(self.key_indices), _ptr(self.block_mask), _ptr(self.tile_list),
                                              _ptr(self.tile_count), _ptr(out), _strides(out), _cabi.ATTN_IMPL[attn_impl],
                                              _ptr(self.status), None, self._stream()), "pbs_attn_fwd")

    # ------------------------------------------------------------------ whole path
    def run(self, q, k, v, out, opt: _cabi.Options):
        """The whole path.  Never synchronises: a device-side error of an EARLIER call (its status words
        have reached the host by now) is raised here; this call's own status is queued for the next."""
        self._inspect_landed_status()
        with self._on_device():
            _cabi.check(self.lib.pbs_prefill_fwd(C.byref(self.shape), _ptr(q), _strides(q), _ptr(k), _strides(k),
                                                 _ptr(v), _strides(v), _ptr(out), _strides(out), C.byref(opt),
                                                 C.byref(self.scratch), self._stream()), "pbs_prefill_fwd")
            self._queue_status_copy()
        return out


def key_importance_static(q: torch.Tensor, k: torch.Tensor, block_size: int, segment_size: int) -> torch.Tensor:
    """Key importance (B, Hq, L) through ``pbs_key_importance_static``: only q, k and the result are
    passed, the stage's scratch is the array built into the library (see include/pbs_b200.h for who
    needs this and its 64 MiB limit).  The result tensor is the caller's; the call allocates nothing
    on the C side."""
    lib = _cabi.load()
    B, Hq, S, D = q.shape
    shape = _cabi.Shape(B, Hq, k.shape[1], S, D, block_size, segment_size, _DTYPES[q.dtype])
    L = (S // segment_size) * segment_size
    out = torch.empty(B, Hq, L, dtype=torch.float32, device=q.device)
    stream = C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
    with torch.cuda.device(q.device):       # the built-in array is looked up on, and used by, the current device
        _cabi.check(lib.pbs_key_importance_static(C.byref(shape), _ptr(q), _strides(q), _ptr(k), _strides(k),
                                                  _ptr(out), stream), "pbs_key_importance_static")
    return out


_PLANS: dict = {}
_MAX_PLANS = 2


def apply_rope_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary position embedding of (B, H, S, D) queries or keys IN PLACE, in one pass on the CUDA
    library: x <- x * cos + rotate_half(x) * sin with the roundings of the separate tensor operations
    of pbs_attn/patch/huggingface.py:14-26.  cos / sin: (B or 1, S, D), same dtype as x."""
    if not x.is_cuda:
        raise RuntimeError("pbs_attn_b200 runs on CUDA devices only; there is no CPU path")
    B, H, S, D = x.shape
    if cos.dim() != 3 or cos.shape[-2:] != (S, D) or sin.shape != cos.shape or cos.dtype != x.dtype or sin.dtype != x.dtype:
        raise ValueError("cos / sin must be (B or 1, S, D) tables of x's dtype")
    if x.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {x.dtype}: need bfloat16, float16 or float32")
    e = x.element_size()
    if not all(t.stride(2) == 1 and t.data_ptr() % 16 == 0 and (t.stride(1) * e) % 16 == 0 and (t.stride(0) * e) % 16 == 0
               for t in (cos, sin)) or sin.stride() != cos.stride():
        cos, sin = cos.contiguous(), sin.contiguous()
    cs = (C.c_int64 * 3)(cos.stride(0) if cos.shape[0] > 1 else 0, cos.stride(1), 1)
    lib = _cabi.load()
    with torch.cuda.device(x.device):
        _cabi.check(lib.pbs_apply_rope(_DTYPES[x.dtype], B, H, S, D, _ptr(x), _strides(x), _ptr(cos), _ptr(sin), cs,
                                       C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)), "pbs_apply_rope")
    return x


def get_plan(q: torch.Tensor, kv_heads: int, block_size: int, segment_size: int) -> Plan:
    """Scratch is reused between calls of the same shape on the same device (e.g. the layers
    of one model); at most two shapes stay cached."""
    B, Hq, S, D = q.shape
    key = (B, Hq, kv_heads, S, D, block_size, segment_size, q.dtype, q.device.index)
    plan = _PLANS.get(key)
    if plan is None:
        while len(_PLANS) >= _MAX_PLANS:
            _PLANS.pop(next(iter(_PLANS)))
        plan = _PLANS[key] = Plan(B, Hq, kv_heads, S, D, block_size, segment_size, q.dtype, q.device)
    return plan


def release_plans():
    _PLANS.clear()


def permuted_block_sparse_attn_fwd(
    query_states: torch.Tensor,
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    block_size: int,
    segment_size: int,
    threshold: Union[float, torch.Tensor],
    causal: bool,
    force_select_first_block: bool = True,
    use_triton: bool = True,
    query_pool_mode: str = "mean",
    key_pool_mode: str = "mean",
    attn_impl: str = "auto",
    intermediates: Optional[dict] = None,
    out: Optional[torch.Tensor] = None,
    out_replicas: Optional[_cabi.OutReplicas] = None,
):
    """Permuted block-sparse attention forward (prefill, causal) on the CUDA library.

    Same arguments and result as the reference (pbs_attn/src/pbs.py:132-257): q is
    (B, Hq, S, D); the result has q's shape, dtype and memory layout, in original token
    order.  Differences, all additive:
      * k/v may have Hkv < Hq heads (Hkv divides Hq); query head h uses KV head
        h // (Hq // Hkv), which equals the reference result on ``repeat_kv``-ed tensors;
      * ``use_triton`` is accepted and ignored (there is one backend);
      * ``attn_impl`` picks the attention kernel ("auto", "tcgen05", "simt");
      * ``intermediates``: a dict that receives the permutation, block mask and plan
        (used by the parity tests);
      * ``out``: a preallocated result tensor of q's shape and dtype (any strides the kernels can
        write: unit head-dim stride, 16-byte aligned rows), e.g. a head slice of a larger tensor;
      * ``out_replicas``: further destinations with ``out``'s strides that the attention kernel
        writes as well (buffers on peer GPUs of a head-sharded call, see ``peer_gather``).
    Runs on the current CUDA stream without synchronising.
    """
    batch_size, num_q_heads, q_len, head_dim = query_states.shape
    _, num_kv_heads, kv_len, _ = key_states.shape
    assert num_q_heads % num_kv_heads == 0
    assert causal
    assert q_len == kv_len
    assert value_states.shape == key_states.shape
    if not query_states.is_cuda:
        raise RuntimeError("pbs_attn_b200 runs on CUDA devices only; there is no CPU path")
    assert segment_size % block_size == 0, "segment_size must be a multiple of block_size"

    q = _readable(query_states, need_distinct_heads=True)
    k = _readable(key_states)
    v = _readable(value_states)
    plan = get_plan(q, num_kv_heads, block_size, segment_size)
    opt = plan.options(threshold, force_select_first_block, query_pool_mode, key_pool_mode, attn_impl,
                       out_replicas=out_replicas)
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or out.device != q.device:
        raise ValueError("out must have the shape, dtype and device of query_states")
    plan.run(q, k, v, out, opt)
    if intermediates is not None:
        intermediates["plan"] = plan
        intermediates["key_indices"] = plan.key_indices
        intermediates["block_mask"] = plan.block_mask
    if os.environ.get("PBS_B200_CHECK_STATUS") == "1":
        plan.check_status()
    return out


def MeanPooling_prefill(
    query_states: torch.Tensor,
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    block_size: int = 128,
    segment_size: int = 1024,
    threshold: float = 0.9,
    causal: bool = True,
    force_select_first_block: bool = True,
    force_select_current_block: bool = True,
    attn_impl: str = "auto",
    intermediates: Optional[dict] = None,
):
    """The reference's mean-pooling block selection WITHOUT key permutation, on the same kernels.

    Same arguments and result as pbs_attn/baselines/MeanPooling.py:7-111: every q block scores
    all kv blocks up to and including its own, keeps the top blocks reaching ``threshold``, always
    keeps kv block 0 (``force_select_first_block``) and its own block, and attends causally.
    ``segment_size`` is accepted and unused, as in the reference.  Implemented as the permuted
    pipeline with identity key order, one block per segment and the diagonal block among the
    candidates.  With ``force_select_current_block=False`` the q block's own kv block is an ordinary
    candidate (MeanPooling.py:55-58 skipped): a q block that does not select it does not attend it,
    and a q block that selects nothing outputs zeros.  Additive: batch > 1 and Hkv < Hq are accepted.
    ``causal=False`` fails with the reference's own assertion: its ``select_blocks`` only supports
    causal selection (pbs_attn/src/utils.py:54), so the baseline never ran non-causally there either.
    """
    batch_size, num_q_heads, q_len, head_dim = query_states.shape
    _, num_kv_heads, kv_len, _ = key_states.shape
    assert num_q_heads % num_kv_heads == 0
    assert q_len == kv_len, "Only support prefilling for now, q_len: {}, kv_len: {}".format(q_len, kv_len)
    # the reference accepts causal=False here but then fails in select_blocks (pbs_attn/src/utils.py:54)
    assert causal == True, "This implementation variant strictly supports causal=True."  # noqa: E712
    if not query_states.is_cuda:
        raise RuntimeError("pbs_attn_b200 runs on CUDA devices only; there is no CPU path")
    q = _readable(query_states, need_distinct_heads=True)
    k = _readable(key_states)
    v = _readable(value_states)
    plan = get_plan(q, num_kv_heads, block_size, block_size)
    if not isinstance(threshold, torch.Tensor):
        threshold = float(threshold)        # the baseline has no "int 1 selects everything" rule
    opt = plan.options(threshold, force_select_first_block, "mean", "mean", attn_impl,
                       no_permutation=True, diagonal_candidates=True, no_own_segment=not force_select_current_block)
    out = torch.empty_like(q)
    plan.run(q, k, v, out, opt)
    if intermediates is not None:
        intermediates["plan"] = plan
        intermediates["key_indices"] = plan.key_indices
        intermediates["block_mask"] = plan.block_mask
    if os.environ.get("PBS_B200_CHECK_STATUS") == "1":
        plan.check_status()
    return out


class _HostPipeline:
    """Streams and device staging buffers of ``permuted_block_sparse_attn_fwd_host`` for one shape."""

    def __init__(self, B, hq_c, hkv_c, S, D, dtype, device):
        self.copy_in = torch.cuda.Stream(device)
        self.copy_out = torch.cuda.Stream(device)
        mk = lambda h: [torch.empty(B, h, S, D, dtype=dtype, device=device) for _ in range(2)]
        self.q, self.k, self.v, self.o = mk(hq_c), mk(hkv_c), mk(hkv_c), mk(hq_c)


_HOST_PIPES: dict = {}


def _host_chunks(Hq: int, Hkv: int, chunks: Optional[int]):
    """Query heads per chunk and KV heads per chunk.  Default: one KV head (with its query heads) per
    chunk; with a single KV head, one query head per chunk (the KV head is then uploaded once)."""
    group = Hq // Hkv
    if chunks is None:
        chunks = Hkv if Hkv > 1 else Hq
    if Hq % chunks:
        raise ValueError(f"chunks={chunks} does not divide the {Hq} query heads")
    hq_c = Hq // chunks
    if hq_c % group == 0:
        return chunks, hq_c, hq_c // group          # whole KV heads per chunk
    if group % hq_c == 0:
        return chunks, hq_c, 1                      # several chunks share one KV head
    raise ValueError(f"chunks={chunks}: a chunk of {hq_c} query heads neither holds nor divides a KV group of {group}")


def permuted_block_sparse_attn_fwd_host(
    query_states: torch.Tensor,
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    block_size: int,
    segment_size: int,
    threshold,
    causal: bool = True,
    force_select_first_block: bool = True,
    query_pool_mode: str = "mean",
    key_pool_mode: str = "mean",
    out: Optional[torch.Tensor] = None,
    device=None,
    chunks: Optional[int] = None,
) -> torch.Tensor:
    """The same call for HOST tensors (ideally pinned): q (B, Hq, S, D), k/v (B, Hkv, S, D) in CPU
    memory, result in CPU memory.

    Query heads are independent, so the call is cut into ``chunks`` groups of query heads (by default
    one KV head with its query heads per group) and pipelined over three streams: while group g is
    computed, group g+1 is copied in and group g-1 is copied out (PCIe is full duplex), with two device
    staging buffers per operand.  A KV head shared by consecutive groups is uploaded once.  Only the
    first group's upload and the last group's download are exposed.  Returns after enqueueing
    everything; synchronise (``torch.cuda.synchronize``) before reading ``out``.
    """
    assert causal and not query_states.is_cuda
    B, Hq, S, D = query_states.shape
    Hkv = key_states.shape[1]
    assert Hq % Hkv == 0 and key_states.shape == value_states.shape and key_states.shape[2] == S
    group = Hq // Hkv
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    if dev.type != "cuda":
        dev = torch.device("cuda", torch.cuda.current_device())
    chunks, hq_c, hkv_c = _host_chunks(Hq, Hkv, chunks)
    if out is None:
        out = torch.empty(B, Hq, S, D, dtype=query_states.dtype).pin_memory()
    key = (B, hq_c, hkv_c, S, D, query_states.dtype, dev.index)
    pipe = _HOST_PIPES.get(key)
    if pipe is None:
        _HOST_PIPES.clear()
        pipe = _HOST_PIPES[key] = _HostPipeline(B, hq_c, hkv_c, S, D, query_states.dtype, dev)
    plan = get_plan(pipe.q[0], hkv_c, block_size, segment_size)
    opt = plan.options(threshold, force_select_first_block, query_pool_mode, key_pool_mode)
    main = torch.cuda.current_stream(dev)
    start = torch.cuda.Event()
    start.record(main)
    pipe.copy_in.wait_event(start)
    pipe.copy_out.wait_event(start)
    q_read = [None, None]            # last compute that read q/o staging slot s
    kv_read = [None, None]           # last compute that read k/v staging slot s
    o_read = [None, None]            # last download that read output slot s
    kv_slot, kv_loaded, n_kv = 0, None, 0
    for c in range(chunks):
        s = c & 1
        qs = slice(c * hq_c, (c + 1) * hq_c)
        kv0 = (c * hq_c) // group
        ks = slice(kv0, kv0 + hkv_c)
        with torch.cuda.stream(pipe.copy_in):
            if q_read[s] is not None:
                pipe.copy_in.wait_event(q_read[s])
            copies = [(pipe.q[s], query_states[:, qs])]
            if kv_loaded != kv0:                       # a KV head shared with the previous chunk stays
                kv_slot = n_kv & 1
                n_kv += 1
                kv_loaded = kv0
                if kv_read[kv_slot] is not None:
                    pipe.copy_in.wait_event(kv_read[kv_slot])
                copies += [(pipe.k[kv_slot], key_states[:, ks]), (pipe.v[kv_slot], value_states[:, ks])]
            for dst, src in copies:
                for b in range(B):
                    dst[b].copy_(src[b], non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(pipe.copy_in)
        main.wait_event(ev_in)
        if o_read[s] is not None:
            main.wait_event(o_read[s])
        plan.run(pipe.q[s], pipe.k[kv_slot], pipe.v[kv_slot], pipe.o[s], opt)
        done = torch.cuda.Event()
        done.record(main)
        q_read[s] = done
        kv_read[kv_slot] = done
        with torch.cuda.stream(pipe.copy_out):
            pipe.copy_out.wait_event(done)
            for b in range(B):
                out[b, qs].copy_(pipe.o[s][b], non_blocking=True)
            o_read[s] = torch.cuda.Event()
            o_read[s].record(pipe.copy_out)
    for ev in o_read:
        if ev is not None:
            main.wait_event(ev)
    return out
