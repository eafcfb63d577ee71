"""CPU oracle for permuted block-sparse attention (prefill, causal).

TEST INFRASTRUCTURE ONLY -- never imported by the product path.

This is a restatement, in plain PyTorch CPU ops, of the algorithm of the
reference project (xinghaow99/pbs-attn).  Each function cites the reference
lines it follows (paths are relative to the reference project root).  The
reference is itself PyTorch, so the restatement uses the same ATen operators at
the same rounding points: a bf16 call rounds the importance logits and the
pooled-block logits to bf16 exactly where the reference does.

Differences from the reference, on purpose:
  * ``stable=True`` (default) makes both sorts stable, so ties are broken by
    the lower original position / lower kv-block id.  The reference calls the
    non-stable ``torch.argsort`` / ``torch.sort`` whose tie order is
    implementation defined; ``stable=False`` reproduces that call exactly.
  * K/V may arrive with fewer heads than Q (grouped-query attention); they are
    repeated here the way the reference's patch layer does before its call
    (pbs_attn/patch/huggingface.py:28-37,209-211).
  * every intermediate (permutation, block scores, block mask) is returned.

Parity pinning: the reference ships no tests or golden vectors.  This oracle is
pinned against outputs of the unmodified reference run on seeded inputs; those
outputs are the fixtures under tests/golden/ (made by tests/golden/make_golden.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Union

import torch
import torch.nn.functional as F


@dataclass
class OracleResult:
    out: torch.Tensor                 # (B, Hq, S, D), input dtype, original token order
    key_indices: Optional[torch.Tensor]   # (B, Hq, S) int64, original position of permuted slot
    block_mask: Optional[torch.Tensor]    # (B, Hq, nb, nb) bool, final mask the kernel consumes
    block_scores: Optional[torch.Tensor]  # (B, Hq, nb, nb) fp32 pooled softmax scores
    importance: Optional[torch.Tensor]    # (B, Hq, nseg*seg) fp32 per-key importance


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """pbs_attn/patch/huggingface.py:28-37 -- head h of the result is KV head h // n_rep."""
    return x if n_rep == 1 else x.repeat_interleave(n_rep, dim=1)


# --------------------------------------------------------------------------- stage 1
def key_importance(q: torch.Tensor, k: torch.Tensor, block_size: int, segment_size: int) -> torch.Tensor:
    """Mean attention of the last query block to every key of the complete segments.

    pbs_attn/src/permute_states.py:44-50.  The matmul and the division by sqrt(D)
    run in the input dtype (two bf16 roundings for bf16 inputs); the softmax runs
    in fp32 over ALL complete-segment keys with no causal mask; the mean over the
    block's query rows is fp32.
    """
    S, D = k.shape[-2], k.shape[-1]
    L = (S // segment_size) * segment_size
    logits = torch.matmul(q[:, :, -block_size:, :], k[:, :, :L, :].transpose(-1, -2)) / math.sqrt(D)
    probs = F.softmax(logits, dim=-1, dtype=torch.float32)
    return probs.mean(dim=-2)


def segment_permutation(importance: torch.Tensor, seq_len: int, segment_size: int, stable: bool = True) -> torch.Tensor:
    """Per-segment descending argsort of the importance, as global positions.

    pbs_attn/src/permute_states.py:52-56,71-81.  The tail ``S % segment_size`` keeps
    its place.  Returns int64 (B, H, S).
    """
    B, H, L = importance.shape
    nseg = L // segment_size
    order = torch.argsort(importance.view(B, H, nseg, segment_size), dim=-1, descending=True, stable=stable)
    order = order + torch.arange(0, L, segment_size).view(1, 1, nseg, 1)
    idx = order.reshape(B, H, L)
    if L < seq_len:
        tail = torch.arange(L, seq_len).view(1, 1, -1).expand(B, H, -1)
        idx = torch.cat([idx, tail], dim=2)
    return idx


def gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """x[b, h, idx[b, h, s], :]  (permute_states.py:59-62 for K, pbs.py:213-215 for V)."""
    return torch.gather(x, 2, idx.unsqueeze(-1).expand(-1, -1, -1, x.shape[-1]))


def permute_keys(q, k, block_size, segment_size, stable=True):
    """pbs_attn/src/permute_states.py:6-83 incl. the no-op cases (:36-38)."""
    B, H, S, _ = k.shape
    nseg, rem = divmod(S, segment_size)
    if nseg == 0 or (nseg == 1 and rem == 0):
        return k, torch.arange(S).view(1, 1, S).expand(B, H, S), None
    imp = key_importance(q, k, block_size, segment_size)
    idx = segment_permutation(imp, S, segment_size, stable)
    return gather_rows(k, idx), idx, imp


# --------------------------------------------------------------------------- stage 2
def _pool(x: torch.Tensor, block_size: int, mode: str) -> torch.Tensor:
    B, H, S, D = x.shape
    x5 = x.reshape(B, H, S // block_size, block_size, D)
    if mode == "mean":
        return x5.mean(dim=-2)
    if mode == "max":
        return x5.max(dim=-2).values
    raise ValueError(f"Invalid pool mode: {mode}")


def _pad_to_block(x: torch.Tensor, block_size: int) -> torch.Tensor:
    pad = (-x.shape[2]) % block_size
    return F.pad(x, (0, 0, 0, pad), value=0) if pad else x


def candidate_block_mask(nb: int, blocks_per_segment: int):
    """(candidates, same_segment), both (nb, nb) bool.  pbs_attn/src/pbs.py:95-107.

    A kv block is a selection candidate for a q block iff it is causal at block
    level and NOT in the q block's own segment, i.e. it lies in an earlier segment.
    """
    qb = torch.arange(nb).unsqueeze(1)
    kb = torch.arange(nb).unsqueeze(0)
    same = (qb // blocks_per_segment) == (kb // blocks_per_segment)
    return (kb <= qb) & ~same, same


def pooled_block_scores(q, perm_k, block_size, candidates, query_pool_mode="mean", key_pool_mode="mean"):
    """pbs_attn/src/pbs.py:67-92 (zero padding) + pbs_attn/src/utils.py:6-34.

    Pooling, the einsum and the in-place division run in the input dtype; masked
    logits are -inf; the softmax over kv blocks is fp32.  Rows without a candidate
    come out NaN, exactly as in the reference.
    """
    D = q.shape[-1]
    pq = _pool(_pad_to_block(q, block_size), block_size, query_pool_mode)
    pk = _pool(_pad_to_block(perm_k, block_size), block_size, key_pool_mode)
    logits = torch.einsum("bhqd,bhkd->bhqk", pq, pk)
    logits /= math.sqrt(D)
    logits = logits.masked_fill(~candidates, float("-inf"))
    return F.softmax(logits, dim=-1, dtype=torch.float32)


def select_blocks(scores: torch.Tensor, threshold: Union[float, torch.Tensor], stable: bool = True) -> torch.Tensor:
    """Smallest top-ranked set of kv blocks whose cumulative score reaches the threshold.

    pbs_attn/src/utils.py:38-86: NaN -> 0, sort descending, running sum (CPU torch
    accumulates an fp32 cumsum in double and rounds each element to fp32), compare
    ``>=`` against the threshold (a Python float is compared as fp32), keep ranks up
    to and including the first one that reaches it -- or nothing when none does --
    and scatter back to kv-block positions.
    """
    scores = torch.nan_to_num(scores, nan=0.0)
    nb_k = scores.shape[-1]
    if scores.shape[-2] == 0 or nb_k == 0:
        return torch.zeros_like(scores, dtype=torch.bool)
    vals, order = torch.sort(scores, dim=-1, descending=True, stable=stable)
    cum = torch.cumsum(vals, dim=-1)
    if isinstance(threshold, torch.Tensor):
        threshold = threshold.view(-1, 1, 1)          # per head
    reached = cum >= threshold
    first = torch.argmax(reached.int(), dim=-1, keepdim=True)
    keep_sorted = (torch.arange(nb_k).view(1, 1, 1, nb_k) <= first) & reached.any(dim=-1, keepdim=True)
    mask = torch.empty_like(scores, dtype=torch.bool)
    mask.scatter_(-1, order, keep_sorted)
    return mask


def first_token_blocks(idx: torch.Tensor, seq_len: int, block_size: int) -> torch.Tensor:
    """(B, H, 1, nb) bool: the permuted kv block holding original token 0.  pbs.py:10-25,78-92."""
    B, H, _ = idx.shape
    pad = (-seq_len) % block_size
    if pad:
        idx = torch.cat([idx, torch.arange(seq_len, seq_len + pad).view(1, 1, -1).expand(B, H, -1)], dim=-1)
    return (idx.reshape(B, H, -1, block_size) == 0).any(dim=-1)[:, :, None, :]


def block_selection(q, perm_k, idx, block_size, segment_size, threshold,
                    force_select_first_block=True, query_pool_mode="mean", key_pool_mode="mean", stable=True):
    """Final block mask and the pooled scores.  pbs.py:29-130 followed by pbs.py:209.

    ``threshold`` given as the Python int 1 selects every candidate (pbs.py:120-121).
    The result always contains every kv block of the q block's own segment.
    """
    S = q.shape[2]
    assert segment_size % block_size == 0, "segment_size must be a multiple of block_size"
    nb = (S + block_size - 1) // block_size
    cand, same = candidate_block_mask(nb, segment_size // block_size)
    scores = pooled_block_scores(q, perm_k, block_size, cand, query_pool_mode, key_pool_mode)
    if isinstance(threshold, int) and not isinstance(threshold, bool) and threshold == 1:
        mask = cand.view(1, 1, nb, nb).expand_as(scores).clone()
    else:
        mask = select_blocks(scores, threshold, stable)
    if force_select_first_block:
        mask = mask | first_token_blocks(idx, S, block_size)
    return mask | same[None, None], scores


# --------------------------------------------------------------------------- stage 3
def sparse_attention(q, perm_k, perm_v, idx, block_mask, block_size, empty_rows_zero=False):
    """Attention of every q block over its selected permuted kv blocks.

    pbs_attn/src/kernels/permuted_block_sparse_attention.py:314-384: logits / sqrt(D)
    in the input dtype, -inf where the key's original position is after the query's
    (query positions are the identity, pbs.py:191-193), fp32 softmax cast back to
    the input dtype, then P @ V in the input dtype.
    """
    B, H, S, D = q.shape
    out = torch.zeros_like(q)
    nb = block_mask.shape[-1]
    for b in range(B):
        for h in range(H):
            kk = perm_k[b, h]
            vv = perm_v[b, h]
            pos = idx[b, h]
            for qb in range(nb):
                r0, r1 = qb * block_size, min((qb + 1) * block_size, S)
                sel = torch.nonzero(block_mask[b, h, qb]).flatten()
                if sel.numel() == 0:
                    continue
                cols = (sel[:, None] * block_size + torch.arange(block_size)[None, :]).flatten()
                cols = cols[cols < S]
                s = torch.matmul(q[b, h, r0:r1], kk[cols].transpose(0, 1)) / math.sqrt(D)
                visible = torch.arange(r0, r1)[:, None] >= pos[cols][None, :]
                s = s.masked_fill(~visible, float("-inf"))
                p = torch.softmax(s, dim=-1, dtype=torch.float32)
                if empty_rows_zero:              # a row whose selected blocks hold no visible key attends nothing
                    p = torch.nan_to_num(p, nan=0.0)
                p = p.to(q.dtype)
                out[b, h, r0:r1] = torch.matmul(p, vv[cols])
    return out


# --------------------------------------------------------------------------- whole path
def permuted_block_sparse_attn_fwd(q, k, v, block_size, segment_size, threshold, causal=True,
                                   force_select_first_block=True, query_pool_mode="mean",
                                   key_pool_mode="mean", stable=True) -> OracleResult:
    """pbs_attn/src/pbs.py:132-257 with ``use_triton=False``."""
    assert causal
    B, Hq, S, D = q.shape
    assert k.shape[2] == S and v.shape[2] == S
    n_rep = Hq // k.shape[1]
    k, v = repeat_kv(k, n_rep), repeat_kv(v, n_rep)
    if S <= segment_size:                                            # pbs.py:175-182
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return OracleResult(out, None, None, None, None)
    perm_k, idx, imp = permute_keys(q, k, block_size, segment_size, stable)
    mask, scores = block_selection(q, perm_k, idx, block_size, segment_size, threshold,
                                   force_select_first_block, query_pool_mode, key_pool_mode, stable)
    perm_v = gather_rows(v, idx)
    out = sparse_attention(q, perm_k, perm_v, idx, mask, block_size)
    return OracleResult(out, idx, mask, scores, imp)


# --------------------------------------------------------------------------- MeanPooling baseline
def meanpooling_block_mask(q, k, block_size, threshold, force_select_first_block=True,
                           force_select_current_block=True, stable=True):
    """Block mask and pooled scores of the reference's MeanPooling baseline.

    pbs_attn/baselines/MeanPooling.py:24-58: zero padding to a block multiple, a
    block-level causal mask that INCLUDES the diagonal, pooled-score softmax and
    threshold selection (pbs_attn/src/utils.py:6-86), then kv block 0 and the
    diagonal block forced on.  Keys are not permuted.
    """
    S = q.shape[2]
    nb = (S + block_size - 1) // block_size
    causal_blocks = torch.tril(torch.ones(nb, nb, dtype=torch.bool))
    scores = pooled_block_scores(q, k, block_size, causal_blocks)
    mask = select_blocks(scores, threshold, stable)
    if force_select_first_block:
        mask[..., 0] = True
    if force_select_current_block:
        mask = mask | torch.eye(nb, dtype=torch.bool)[None, None]
    return mask, scores


def meanpooling_prefill(q, k, v, block_size=128, threshold=0.9, force_select_first_block=True,
                        force_select_current_block=True, stable=True) -> OracleResult:
    """pbs_attn/baselines/MeanPooling.py:7-111 with ``causal=True``.

    The reference hands its block mask to an external block-sparse flash-attention
    library with ``is_causal=True`` (MeanPooling.py:92-106): every selected block is
    attended, element-causally on the diagonal.  That library is not part of the
    reference project, so the attention itself is restated from its contract:
    softmax over the selected blocks' visible keys, the same arithmetic as
    ``sparse_attention`` with the identity permutation.  Without the forced diagonal block a query
    row may have no visible key among its selected blocks (or no selected block at all); block-sparse
    flash-attention kernels return zeros for such rows, and so does this restatement.
    """
    B, Hq, S, D = q.shape
    n_rep = Hq // k.shape[1]
    k, v = repeat_kv(k, n_rep), repeat_kv(v, n_rep)        # the baseline asserts Hq == Hkv (MeanPooling.py:21)
    mask, scores = meanpooling_block_mask(q, k, block_size, threshold, force_select_first_block,
                                          force_select_current_block, stable)
    idx = torch.arange(S).view(1, 1, S).expand(B, Hq, S)
    out = sparse_attention(q, k, v, idx, mask, block_size, empty_rows_zero=True)
    return OracleResult(out, idx, mask, scores, None)
