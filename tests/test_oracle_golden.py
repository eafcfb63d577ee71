"""Pins the CPU oracle against outputs of the unmodified reference (tests/golden/*.npz)."""
import numpy as np
import pytest
import torch

from cases import CASES, MEANPOOLING_CASES
from oracle import pbs_oracle
from parity import assert_close_out, golden_mask, golden_out, load_case


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_equals_stable_reference(name):
    """stable=True oracle == reference run with stable sorts: bit-exact everywhere."""
    w, kwargs, stride, (q, k, v), g = load_case(name)
    r = pbs_oracle.permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, w.threshold,
                                                  stable=True, **kwargs)
    out = r.out[:, :, ::stride, :]
    assert torch.equal(out.float(), golden_out(g, "stable", w.torch_dtype).float())
    if "idx_stable" in g:
        nb = -(-w.seq_len // w.block_size)
        assert np.array_equal(r.key_indices.numpy().astype(np.int32), g["idx_stable"])
        assert torch.equal(r.block_mask, golden_mask(g, "stable", nb))
        assert np.array_equal(torch.nan_to_num(r.block_scores, nan=-1.0).numpy(), g["scores"])
    else:
        assert r.key_indices is None


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_vs_unmodified_reference(name):
    """Against the reference exactly as shipped (non-stable sorts): outputs within the
    stated tolerance; permutation and mask equal except where its sort broke a tie
    differently (the two reference runs themselves differ only there)."""
    w, kwargs, stride, (q, k, v), g = load_case(name)
    r = pbs_oracle.permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, w.threshold,
                                                  stable=False, **kwargs)
    assert_close_out(r.out[:, :, ::stride, :], golden_out(g, "ref", w.torch_dtype), w.torch_dtype, name)
    if "idx_ref" in g:
        nb = -(-w.seq_len // w.block_size)
        assert np.array_equal(r.key_indices.numpy().astype(np.int32), g["idx_ref"])
        assert torch.equal(r.block_mask, golden_mask(g, "ref", nb))


def test_oracle_dense_threshold_is_causal_sdpa():
    """threshold == int 1 without the forced first block selects every causal block, so the
    result is dense causal attention (property of the reference, pbs.py:120-121)."""
    w, kwargs, stride, (q, k, v), g = load_case("dense_int_threshold")
    r = pbs_oracle.permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, 1, **kwargs)
    kr = k.repeat_interleave(w.q_heads // w.kv_heads, 1)
    vr = v.repeat_interleave(w.q_heads // w.kv_heads, 1)
    dense = torch.nn.functional.scaled_dot_product_attention(q, kr, vr, is_causal=True)
    assert (r.out - dense).abs().max() < 1e-5


def test_oracle_first_segment_rows_select_nothing_by_score():
    w, kwargs, stride, (q, k, v), g = load_case("no_first_block")
    r = pbs_oracle.permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, w.threshold, **kwargs)
    bps = w.segment_size // w.block_size
    first = r.block_mask[:, :, :bps]
    assert first[..., :bps].all() and not first[..., bps:].any()


def test_oracle_threshold_never_reached_keeps_only_forced_blocks():
    w, kwargs, stride, (q, k, v), g = load_case("threshold_never_reached")
    r = pbs_oracle.permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, w.threshold, **kwargs)
    nb = r.block_mask.shape[-1]
    bps = w.segment_size // w.block_size
    qb = torch.arange(nb)[:, None]
    kb = torch.arange(nb)[None, :]
    same = (qb // bps) == (kb // bps)
    forced = same[None, None] | pbs_oracle.first_token_blocks(r.key_indices, w.seq_len, w.block_size)
    assert torch.equal(r.block_mask, forced.expand_as(r.block_mask))


@pytest.mark.parametrize("name", list(MEANPOOLING_CASES))
def test_meanpooling_oracle_equals_reference(name):
    """The MeanPooling restatement against the reference's own MeanPooling_prefill (run with a stub
    for the external attention library it imports): block mask and pooled scores bit-exact, output
    within tolerance of the stub's fp32 attention."""
    w, kwargs, stride, (q, k, v), g = load_case(name)
    r = pbs_oracle.meanpooling_prefill(q, k, v, w.block_size, w.threshold, stable=True, **kwargs)
    nb = -(-w.seq_len // w.block_size)
    assert torch.equal(r.block_mask, golden_mask(g, "stable", nb))
    assert torch.equal(r.block_mask, golden_mask(g, "ref", nb))
    assert np.array_equal(r.block_scores.numpy(), g["scores"])
    assert_close_out(r.out[:, :, ::stride, :], golden_out(g, "stable", w.torch_dtype), w.torch_dtype, name)
    eye = torch.eye(nb, dtype=torch.bool)
    if kwargs.get("force_select_current_block", True):
        assert (r.block_mask & eye).sum() == eye.sum() * w.batch * w.q_heads    # the diagonal is always on
    else:
        assert (r.block_mask & eye).sum() < eye.sum() * w.batch * w.q_heads     # ... an ordinary candidate otherwise
    assert not torch.triu(r.block_mask, diagonal=1).any()                        # nothing above it


@pytest.mark.parametrize("name", ["rope_bf16", "rope_fp16", "rope_fp32"])
def test_rotary_helper_equals_reference_fixture(name):
    """The host-side rotary helper of the patch layer (used for CPU tensors and as the check of the CUDA
    rotary kernel) against outputs of the reference's own function: bit-exact."""
    import os
    from cases import ROPE_CASES, rope_inputs
    from pbs_attn.patch.huggingface import apply_rotary_pos_emb
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rope.npz"))
    q, k, cos, sin = rope_inputs(ROPE_CASES[name])
    qe, ke = apply_rotary_pos_emb(q, k, cos, sin)
    for got, want in ((qe, g[f"{name}_q"]), (ke, g[f"{name}_k"])):
        got = got.contiguous()
        raw = got.view(torch.int16).numpy().view(np.uint16) if got.dtype != torch.float32 else got.numpy()
        assert np.array_equal(raw, want)
