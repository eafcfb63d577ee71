"""Full-size GPU checks (task configurations 2 and 3) through size-independent properties: the CPU
oracle would need minutes to hours at these sizes."""
import pytest
import torch

from pbs_attn_b200.synth import LLAMA8B_128K, LLAMA8B_32K, make_qkv

pytestmark = pytest.mark.gpu


def _run(w, q, k, v, **kw):
    from pbs_attn_b200.prefill import permuted_block_sparse_attn_fwd
    inter = {}
    out = permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, kw.pop("threshold", w.threshold), True,
                                         intermediates=inter, **kw)
    torch.cuda.synchronize()
    inter["plan"].check_status()
    return out, inter


def _structure_checks(w, inter):
    idx = inter["key_indices"]
    B, H, S = idx.shape
    L = (S // w.segment_size) * w.segment_size
    srt = torch.sort(idx[..., :L].reshape(B, H, -1, w.segment_size), dim=-1).values
    base = torch.arange(L, device=idx.device, dtype=idx.dtype).view(1, 1, -1, w.segment_size)
    assert torch.equal(srt, base.expand_as(srt)), "a segment is not a permutation of itself"
    mask = inter["block_mask"].bool()
    nb = mask.shape[-1]
    bps = w.segment_size // w.block_size
    qb = torch.arange(nb, device=mask.device)[:, None]
    kb = torch.arange(nb, device=mask.device)[None, :]
    same = (qb // bps) == (kb // bps)
    future = (kb // bps) > (qb // bps)
    assert bool(mask[..., same].all()), "own-segment blocks must always be on"
    assert not bool(mask[..., future].any()), "a block of a later segment is on"
    first = inter["plan"].first_block[: B * H].long().view(B, H)
    hit = torch.gather(mask, 3, first[:, :, None, None].expand(B, H, nb, 1))
    assert bool(hit.all()), "the block holding token 0 must be on for every query block"
    # token 0 really sits in that block
    pos0 = (idx == 0).float().argmax(-1) // w.block_size
    assert torch.equal(pos0, first)


@pytest.fixture(scope="module")
def cfg2():
    w = LLAMA8B_32K
    q, k, v = make_qkv(w, seed=2, device="cuda")
    return w, q, k, v


def test_cfg2_structure_and_kernel_agreement(cfg2):
    """Llama-3.1-8B heads at 32768 tokens: structural invariants of permutation and mask; the
    tcgen05 kernel agrees with the generic CUDA-core kernel on identical inputs; two runs are
    bitwise identical."""
    w, q, k, v = cfg2
    out, inter = _run(w, q, k, v)
    _structure_checks(w, inter)
    assert torch.isfinite(out.float()).all()
    plan = inter["plan"]
    ref = torch.empty_like(q)
    plan.attn_fwd(q, ref, "simt")
    torch.cuda.synchronize()
    d = (out.float() - ref.float()).abs()
    assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3, (d.max().item(), d.mean().item())
    out2, _ = _run(w, q, k, v)
    assert torch.equal(out, out2)


def test_cfg2_select_all_equals_dense_causal_attention(cfg2):
    """threshold == int 1 without the forced first block selects every causal block (reference,
    pbs_attn/src/pbs.py:120-121), so the path must equal dense causal attention."""
    w, q, k, v = cfg2
    out, _ = _run(w, q, k, v, threshold=1, force_select_first_block=False)
    n_rep = w.q_heads // w.kv_heads
    dense = torch.nn.functional.scaled_dot_product_attention(q, k.repeat_interleave(n_rep, 1), v.repeat_interleave(n_rep, 1), is_causal=True)
    d = (out.float() - dense.float()).abs()
    assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3, (d.max().item(), d.mean().item())


def test_cfg2_linearity_in_values(cfg2):
    """Permutation and mask depend on Q and K only, so the output is linear in V."""
    w, q, k, v = cfg2
    v2 = torch.randn_like(v)
    a, _ = _run(w, q, k, v)
    b, _ = _run(w, q, k, v2)
    c, _ = _run(w, q, k, (v.float() + v2.float()).to(v.dtype))
    d = (c.float() - (a.float() + b.float())).abs()
    assert d.max().item() <= 6e-2 and d.mean().item() <= 4e-3, (d.max().item(), d.mean().item())


def test_cfg3_one_kv_group_at_131072():
    """One GPU's shard of the 128K configuration (4 query heads, 1 KV head): invariants, finiteness,
    and agreement with dense attention in select-all mode."""
    w = LLAMA8B_128K.with_(q_heads=4, kv_heads=1)
    q, k, v = make_qkv(w, seed=3, device="cuda")
    out, inter = _run(w, q, k, v)
    _structure_checks(w, inter)
    assert torch.isfinite(out.float()).all()
    dense_out, _ = _run(w, q, k, v, threshold=1, force_select_first_block=False)
    dense = torch.nn.functional.scaled_dot_product_attention(q, k.expand(-1, 4, -1, -1), v.expand(-1, 4, -1, -1), is_causal=True)
    d = (dense_out.float() - dense.float()).abs()
    assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3, (d.max().item(), d.mean().item())


@pytest.mark.parametrize("hq,hkv,d,s,dt,bs,seg,batch", [
    (28, 4, 128, 8192, "bf16", 64, 128, 1),     # Qwen2.5-7B heads, small blocks and segments
    (28, 4, 128, 8192, "bf16", 128, 512, 1),    # Qwen2.5-7B heads, long segments
    (8, 2, 64, 6000, "fp16", 64, 256, 2),       # head_dim 64, fp16, ragged length, batch 2
    (4, 4, 128, 5000, "bf16", 128, 128, 1),     # one block per segment, no GQA, ragged length
])
def test_sweep_shapes_tcgen05_agrees_with_generic_kernel(hq, hkv, d, s, dt, bs, seg, batch):
    """Shapes of the Qwen sweep (task configuration 5) and the corner cases of the tcgen05 kernel:
    structure of permutation and mask, and agreement of the two attention kernels on the same
    permuted inputs."""
    from pbs_attn_b200.synth import Workload
    w = Workload("sweep", batch, hq, hkv, d, s, dt, bs, seg, 0.9, 1e6, density=0.08, sinks=4)
    q, k, v = make_qkv(w, seed=11, device="cuda")
    out, inter = _run(w, q, k, v)
    _structure_checks(w, inter)
    assert torch.isfinite(out.float()).all()
    ref = torch.empty_like(q)
    inter["plan"].attn_fwd(q, ref, "simt")
    torch.cuda.synchronize()
    dd = (out.float() - ref.float()).abs()
    assert dd.max().item() <= 2e-2 and dd.mean().item() <= 2e-3, (dd.max().item(), dd.mean().item())


def test_one_head_pair_at_524288_tokens():
    """The longest context of the reference's efficiency sweep (512K, run there over 8 GPUs: this is a
    2-query-head slice of one rank's share).  Index arithmetic at that size: structure invariants on the
    sparse call, and the select-all call against dense causal attention."""
    w = LLAMA8B_128K.with_(q_heads=2, kv_heads=1, seq_len=524288, name="llama8b_heads_s524288_h2")
    q, k, v = make_qkv(w, seed=11, device="cuda")
    out, inter = _run(w, q, k, v)
    _structure_checks(w, inter)
    assert torch.isfinite(out.float()).all()
    del out, inter
    dense_out, _ = _run(w, q, k, v, threshold=1, force_select_first_block=False)
    dense = torch.nn.functional.scaled_dot_product_attention(q, k.expand(-1, 2, -1, -1), v.expand(-1, 2, -1, -1), is_causal=True)
    d = (dense_out.float() - dense.float()).abs()
    assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3, (d.max().item(), d.mean().item())
