"""The efficiency harness (time to first token of a patched random-init model, the reference's
eval/efficiency protocol) run end to end on a tiny architecture: it must patch, warm up, time with CUDA
events, report the attention share and write its result line."""
import json

import pytest
import torch

pytestmark = pytest.mark.gpu

TINY = dict(kind="llama", vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=10000.0,
            max_position_embeddings=4096, rms_norm_eps=1e-5)


@pytest.mark.parametrize("method", ["pbs", "meanpooling"])
def test_harness_runs_patched_prefill_and_reports(tmp_path, capsys, method):
    from pbs_attn_b200 import efficiency
    efficiency.ARCHS["tiny-llama"] = dict(TINY)
    out = tmp_path / "result.jsonl"
    try:
        efficiency.main(["--arch", "tiny-llama", "--method", method, "--lens", "1024,2048", "--block-size", "64",
                         "--segment-size", "128", "--warmup", "1", "--iters", "2", "--attention-share", "--out", str(out)])
    finally:
        efficiency.ARCHS.pop("tiny-llama", None)
    recs = [json.loads(l) for l in out.read_text().splitlines()]
    assert [r["len"] for r in recs] == [1024, 2048]
    for r in recs:
        assert r["method"] == method and r["layers"] == 2 and r["batch"] == 1
        assert r["mean_s"] > 0 and r["without_attention_s"] > 0 and r["tokens_per_s"] > 0
        assert 0.0 < r["last_layer_density"] <= 1.3
        assert -1.0 < r["attention_share"] < 1.0
    printed = [l for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert len(printed) == 2


def test_patched_model_logits_match_dense_attention_in_select_all_mode():
    """With every causal block selected the patched model must reproduce the unpatched model's
    next-token logits (the reference's own smoke check, pbs_attn/patch/huggingface.py:322-406, compares
    generations before and after patching)."""
    from pbs_attn_b200 import efficiency
    from pbs_attn_b200.hf_patch import apply_patch_with_prefill, get_permuted_block_sparse_attn_fwd, remove_patch
    efficiency.ARCHS["tiny-llama"] = dict(TINY)
    try:
        model = efficiency.build_model("tiny-llama", device="cuda")
    finally:
        efficiency.ARCHS.pop("tiny-llama", None)
    ids = torch.randint(0, 512, (1, 1536), device="cuda")
    with torch.no_grad():
        want = model(ids, logits_to_keep=1).logits.float()
        apply_patch_with_prefill(model, get_permuted_block_sparse_attn_fwd(block_size=64, segment_size=128, threshold=1,
                                                                           force_select_first_block=False))
        got = model(ids, logits_to_keep=1).logits.float()
        remove_patch(model)
        again = model(ids, logits_to_keep=1).logits.float()
    assert torch.equal(again, want)
    assert (got - want).abs().max().item() <= 5e-2 * max(1.0, want.abs().max().item())
