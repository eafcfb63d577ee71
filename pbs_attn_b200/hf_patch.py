"""Hugging Face boundary: the prefill-function factory and the attention monkey patch.

Mirrors the public surface of the reference's pbs_attn/patch/huggingface.py for the PBS path:
``get_permuted_block_sparse_attn_fwd`` (:141-167), ``patched_attention_forward`` (:169-241),
``apply_patch_with_prefill`` (:243-307), ``get_supported_model_types`` / ``is_model_supported``
(:309-316).  The factories of the competitor baselines (:43-138) are not part of this path.
"""
from __future__ import annotations

import types
from functools import partial
from typing import Callable, Optional

import torch

SUPPORTED_MODEL_TYPES = ("LlamaForCausalLM", "Qwen2ForCausalLM")


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    """Rotate-half RoPE on (B, H, S, D) tensors with (B, S, D) tables (huggingface.py:14-26)."""
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    """(B, Hkv, S, D) -> (B, Hkv * n_rep, S, D), head h taken from KV head h // n_rep (huggingface.py:28-37)."""
    if n_rep == 1:
        return hidden_states
    b, hkv, s, d = hidden_states.shape
    return hidden_states[:, :, None].expand(b, hkv, n_rep, s, d).reshape(b, hkv * n_rep, s, d)


def get_permuted_block_sparse_attn_fwd(
    block_size=128,
    segment_size=256,
    threshold=0.9,
    causal=True,
    force_select_first_block=True,
    use_triton=True,
    query_pool_mode: str = "mean",
    key_pool_mode: str = "mean",
):
    """A ``functools.partial`` over ``permuted_block_sparse_attn_fwd`` with the given settings,
    to hand to ``apply_patch_with_prefill``.  Raises RuntimeError("PBS unavailable.") when the
    CUDA library cannot be loaded."""
    try:
        from . import _cabi
        from .prefill import permuted_block_sparse_attn_fwd as impl
        _cabi.load()
    except Exception as e:  # same contract as the reference factory
        raise RuntimeError("PBS unavailable.") from e
    return partial(impl, block_size=block_size, segment_size=segment_size, threshold=threshold, causal=causal,
                   force_select_first_block=force_select_first_block, use_triton=use_triton,
                   query_pool_mode=query_pool_mode, key_pool_mode=key_pool_mode)


def get_meanpooling_prefill(block_size=128, segment_size=1024, threshold=0.9,
                            force_select_first_block=True, force_select_current_block=True):
    """A ``functools.partial`` over ``MeanPooling_prefill`` (block selection without permutation), the
    counterpart of the reference factory of the same name (pbs_attn/patch/huggingface.py:43-58)."""
    try:
        from . import _cabi
        from .prefill import MeanPooling_prefill as impl
        _cabi.load()
    except Exception as e:
        raise RuntimeError("MeanPooling unavailable.") from e
    return partial(impl, block_size=block_size, segment_size=segment_size, threshold=threshold, causal=True,
                   force_select_first_block=force_select_first_block,
                   force_select_current_block=force_select_current_block)


def _fused_rope_applies(q, k, cos, sin) -> bool:
    """The CUDA library's in-place rotary kernel replaces the five tensor operations of
    ``apply_rotary_pos_emb`` when the tensors are on a GPU, share a supported dtype and nothing needs
    gradients (the projections' outputs are fresh tensors, so writing in place is safe)."""
    if not (q.is_cuda and k.is_cuda and cos.is_cuda) or torch.is_grad_enabled() and (q.requires_grad or k.requires_grad):
        return False
    if q.dtype not in (torch.bfloat16, torch.float16, torch.float32) or not (k.dtype == cos.dtype == sin.dtype == q.dtype):
        return False
    d = q.shape[-1]
    if cos.dim() != 3 or cos.shape[-1] != d or cos.shape[-2] != q.shape[-2] or (d // 2 * q.element_size()) % 16 or d % 2:
        return False
    e = q.element_size()
    return all(t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all((st * e) % 16 == 0 for st in t.stride()[:3]) for t in (q, k))


def _kernel_of(prefill_fn):
    return prefill_fn.func if isinstance(prefill_fn, partial) else prefill_fn


def _takes_grouped_kv(prefill_fn) -> bool:
    """True for this package's own prefill functions, which map query heads onto fewer KV heads
    themselves (and for a callable that says so with a ``takes_grouped_kv = True`` attribute); any
    other callable gets K/V repeated to the query head count like the reference does."""
    from .prefill import MeanPooling_prefill, permuted_block_sparse_attn_fwd
    kern = _kernel_of(prefill_fn)
    return kern in (permuted_block_sparse_attn_fwd, MeanPooling_prefill) or bool(getattr(kern, "takes_grouped_kv", False))


def patched_attention_forward(
    self,
    hidden_states: torch.Tensor,
    position_embeddings: tuple,
    attention_mask: Optional[torch.Tensor],
    past_key_values=None,
    cache_position: Optional[torch.LongTensor] = None,
    prefill_fn: Optional[Callable] = None,
    **kwargs,
):
    """Replacement for ``LlamaAttention.forward`` / ``Qwen2Attention.forward``.

    Prompts (q_len > 1) go through ``prefill_fn(query, key, value)`` on (B, H, S, D) tensors after
    projection, RoPE and the KV-cache update; single-token decode goes to the layer's original
    forward.  Head counts are derived from the projection widths, so a tensor-parallel shard works
    unchanged.  Returns ``(attn_output, None)``.
    """
    bsz, q_len, _ = hidden_states.size()
    if q_len <= 1:
        return self.original_forward(hidden_states=hidden_states, position_embeddings=position_embeddings,
                                     attention_mask=attention_mask, past_key_values=past_key_values,
                                     cache_position=cache_position, **kwargs)
    if prefill_fn is None:
        raise RuntimeError("prefill_fn required.")
    d = self.head_dim
    q = self.q_proj(hidden_states)
    k = self.k_proj(hidden_states)
    v = self.v_proj(hidden_states)
    n_q, n_kv = q.shape[-1] // d, k.shape[-1] // d
    q = q.view(bsz, q_len, n_q, d).transpose(1, 2)
    k = k.view(bsz, q_len, n_kv, d).transpose(1, 2)
    v = v.view(bsz, q_len, n_kv, d).transpose(1, 2)
    cos, sin = position_embeddings
    if _fused_rope_applies(q, k, cos, sin):
        from .prefill import apply_rope_
        q, k = apply_rope_(q, cos, sin), apply_rope_(k, cos, sin)     # one pass each, in place
    else:
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
    if past_key_values is not None:
        past_key_values.update(k, v, self.layer_idx, {"sin": sin, "cos": cos, "cache_position": cache_position})
    if not _takes_grouped_kv(prefill_fn):
        n_rep = max(1, n_q // max(1, n_kv))
        k, v = repeat_kv(k, n_rep), repeat_kv(v, n_rep)
    if "layer_idx" in _kernel_of(prefill_fn).__code__.co_varnames:
        o = prefill_fn(q, k, v, layer_idx=self.layer_idx)
    else:
        o = prefill_fn(q, k, v)
    o = o.transpose(1, 2).reshape(bsz, q_len, n_q * d)
    return self.o_proj(o), None


def get_supported_model_types():
    return list(SUPPORTED_MODEL_TYPES)


def is_model_supported(model) -> bool:
    return type(model).__name__ in SUPPORTED_MODEL_TYPES


def apply_patch_with_prefill(model, prefill_fn: Optional[Callable] = None, skip_layers: Optional[list] = None):
    """Rebinds ``self_attn.forward`` of every decoder layer (except ``skip_layers``) to route
    prompts through ``prefill_fn``; the original method is kept as ``self_attn.original_forward``.
    Only LlamaForCausalLM and Qwen2ForCausalLM are accepted (ValueError otherwise)."""
    skip = set(skip_layers or [])
    if not is_model_supported(model):
        raise ValueError(f"Model type {type(model).__name__} is not supported. "
                         f"Supported types: {get_supported_model_types()}")
    layers = model.model.layers
    name = getattr(_kernel_of(prefill_fn), "__name__", "None") if prefill_fn is not None else "None"
    print(f"Patching {type(model).__name__}: prefill function {name}, skipping layers {sorted(skip)}")

    def make_forward(fn):
        def new_forward(self, hidden_states, position_embeddings, attention_mask=None, past_key_values=None,
                        cache_position=None, **kwargs):
            return patched_attention_forward(self, hidden_states=hidden_states,
                                             position_embeddings=position_embeddings,
                                             attention_mask=attention_mask, past_key_values=past_key_values,
                                             cache_position=cache_position, prefill_fn=fn, **kwargs)
        return new_forward

    patched = 0
    for i, layer in enumerate(layers):
        if i in skip:
            continue
        attn = layer.self_attn
        attn.original_forward = attn.forward
        attn.forward = types.MethodType(make_forward(prefill_fn), attn)
        patched += 1
    print(f"Patched {patched}/{len(layers)} attention layers.")
    return model


def remove_patch(model):
    """Undoes ``apply_patch_with_prefill``: every patched layer gets its original forward back.
    (The reference has no such call; re-patching a patched model there would keep the patched method
    as ``original_forward``.  Used to time one model with several prefill functions.)"""
    for layer in model.model.layers:
        attn = layer.self_attn
        if "original_forward" in attn.__dict__:
            attn.forward = attn.__dict__.pop("original_forward")
    return model
