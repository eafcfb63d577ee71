"""GPU parity of MeanPooling_prefill (block selection without key permutation) against the CPU
oracle and the fixtures made from the reference's own MeanPooling_prefill.

Bars as for the permuted path: block masks bit-exact up to explained near-ties of the fp32 scores
(exactly equal for fp32 inputs); outputs within max-abs 2e-2 / mean-abs 2e-3 for bf16 (2e-4 / 2e-5
for fp32).
"""
import pytest
import torch

from cases import MEANPOOLING_CASES
from oracle import pbs_oracle
from parity import assert_close_out, classify_mask, golden_mask, golden_out, load_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("impl", ["auto", "simt"])
@pytest.mark.parametrize("name", list(MEANPOOLING_CASES))
def test_meanpooling_against_reference_fixtures(name, impl):
    from pbs_attn_b200.prefill import MeanPooling_prefill
    w, kwargs, stride, (q, k, v), g = load_case(name)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    inter = {}
    out = MeanPooling_prefill(qd, kd, vd, block_size=w.block_size, threshold=w.threshold, attn_impl=impl,
                              intermediates=inter, **kwargs)
    torch.cuda.synchronize()
    plan = inter["plan"]
    plan.check_status()
    assert out.shape == q.shape and out.dtype == q.dtype
    # keys stay in place
    idx = inter["key_indices"].cpu().long()
    assert torch.equal(idx, torch.arange(w.seq_len).view(1, 1, -1).expand_as(idx))
    nb = -(-w.seq_len // w.block_size)
    mask = inter["block_mask"].cpu().bool()
    r = pbs_oracle.meanpooling_prefill(q, k, v, w.block_size, w.threshold, stable=True, **kwargs)
    rows, bad = classify_mask(mask, r.block_mask, r.block_scores, float(w.threshold), 1)
    assert bad == 0, f"{bad}/{rows} mask rows unexplained"
    # the reference's selection run on OUR pooled scores must give our mask
    force = kwargs.get("force_select_first_block", True)
    current = kwargs.get("force_select_current_block", True)
    opt = plan.options(float(w.threshold), force, no_permutation=True, diagonal_candidates=True, no_own_segment=not current)
    scores = plan.select_blocks(opt, want_scores=True).cpu()
    expect = pbs_oracle.select_blocks(scores, float(w.threshold), stable=True)
    if force:
        expect[..., 0] = True
    if current:
        expect = expect | torch.eye(nb, dtype=torch.bool)[None, None]
    rows2, bad2 = classify_mask(mask, expect, scores, float(w.threshold), 1)
    assert bad2 == 0, f"{bad2}/{rows2} rows differ from select_blocks run on our own scores"
    if w.dtype == "fp32":
        assert torch.equal(mask, golden_mask(g, "stable", nb))
        assert torch.allclose(scores, torch.from_numpy(g["scores"]), rtol=1e-5, atol=1e-7)   # fp32 dot-product order differs
    sub = out.cpu()[:, :, ::stride, :]
    assert_close_out(sub, r.out[:, :, ::stride, :], w.torch_dtype, name + " vs oracle")
    if rows == 0:
        assert_close_out(sub, golden_out(g, "stable", w.torch_dtype), w.torch_dtype, name + " vs reference fixture")


def test_meanpooling_unreachable_threshold_is_sink_plus_diagonal():
    """With a threshold no running sum reaches, every q block attends kv block 0 and its own
    block only; checked at S=16384 against that attention written with torch ops on the GPU."""
    from pbs_attn_b200.prefill import MeanPooling_prefill
    torch.manual_seed(5)
    H, S, D, bs = 4, 16384, 128, 128
    q = torch.randn(1, H, S, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 2, S, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(1, 2, S, D, device="cuda", dtype=torch.bfloat16)
    inter = {}
    out = MeanPooling_prefill(q, k, v, block_size=bs, threshold=2.0, intermediates=inter)
    torch.cuda.synchronize()
    inter["plan"].check_status()
    nb = S // bs
    mask = inter["block_mask"].bool()
    want_mask = torch.eye(nb, dtype=torch.bool, device="cuda")
    want_mask[:, 0] = True
    assert torch.equal(mask, want_mask[None, None].expand_as(mask))
    kr, vr = k.repeat_interleave(2, 1).float(), v.repeat_interleave(2, 1).float()
    qb = q.float().view(1, H, nb, bs, D)
    kd, vd = kr.view(1, H, nb, bs, D), vr.view(1, H, nb, bs, D)
    s_diag = torch.einsum("bhnqd,bhnkd->bhnqk", qb, kd) / D ** 0.5
    s_diag = s_diag.masked_fill(~torch.tril(torch.ones(bs, bs, dtype=torch.bool, device="cuda")), float("-inf"))
    s_sink = torch.einsum("bhnqd,bhkd->bhnqk", qb, kd[:, :, 0]) / D ** 0.5
    s_sink[:, :, 0] = float("-inf")                       # block 0's diagonal IS the sink block: count it once
    p = torch.softmax(torch.cat([s_sink, s_diag], dim=-1), dim=-1)
    want = torch.einsum("bhnqk,bhkd->bhnqd", p[..., :bs], vd[:, :, 0]) + torch.einsum("bhnqk,bhnkd->bhnqd", p[..., bs:], vd)
    assert_close_out(out.cpu(), want.reshape(1, H, S, D).cpu(), torch.bfloat16, "sink + diagonal")


def test_meanpooling_factory_and_patch_probe():
    from functools import partial
    from pbs_attn.patch.huggingface import get_meanpooling_prefill
    from pbs_attn.baselines.MeanPooling import MeanPooling_prefill
    fn = get_meanpooling_prefill(block_size=64, threshold=0.8)
    assert isinstance(fn, partial) and fn.func is MeanPooling_prefill
    assert "layer_idx" not in fn.func.__code__.co_varnames
    with pytest.raises(AssertionError, match="causal=True"):      # the reference's select_blocks asserts the same
        MeanPooling_prefill(torch.zeros(1, 1, 128, 64, device="cuda"), torch.zeros(1, 1, 128, 64, device="cuda"),
                            torch.zeros(1, 1, 128, 64, device="cuda"), causal=False)
