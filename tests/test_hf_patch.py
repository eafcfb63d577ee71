"""The Hugging Face boundary: factory, monkey patch and patched forward (mirrors of the reference's
pbs_attn/patch/huggingface.py:141-307).  CPU tests use a plain-PyTorch stand-in prefill function to
exercise the plumbing; the GPU test runs tiny random Llama/Qwen2 models through the CUDA path."""
from functools import partial

import pytest
import torch

from pbs_attn.patch.huggingface import (apply_patch_with_prefill, get_permuted_block_sparse_attn_fwd,
                                        get_supported_model_types, is_model_supported)


def _tiny(kind, dtype=torch.float32, layers=2):
    from transformers import LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM
    kw = dict(vocab_size=128, hidden_size=128, intermediate_size=256, num_hidden_layers=layers,
              num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=2048)
    torch.manual_seed(0)
    if kind == "llama":
        m = LlamaForCausalLM(LlamaConfig(head_dim=32, **kw))
    else:
        m = Qwen2ForCausalLM(Qwen2Config(**kw))
    return m.to(dtype).eval()


def dense_prefill(query_states, key_states, value_states):
    """Stand-in with the prefill-function contract: (B, H, S, D) in, (B, H, S, D) out."""
    return torch.nn.functional.scaled_dot_product_attention(query_states, key_states, value_states, is_causal=True)


def dense_prefill_with_layer(query_states, key_states, value_states, layer_idx=None, seen=None):
    seen.append(layer_idx)
    return dense_prefill(query_states, key_states, value_states)


@pytest.mark.parametrize("kind", ["llama", "qwen2"])
def test_patched_prefill_matches_unpatched_model_and_decode_uses_original_forward(kind):
    model = _tiny(kind)
    ids = torch.randint(0, 128, (2, 48))
    with torch.no_grad():
        want = model(ids).logits
        gen_want = model.generate(ids[:1], max_new_tokens=4, do_sample=False)
    apply_patch_with_prefill(model, dense_prefill)
    assert all(hasattr(l.self_attn, "original_forward") for l in model.model.layers)
    with torch.no_grad():
        got = model(ids).logits
        gen_got = model.generate(ids[:1], max_new_tokens=4, do_sample=False)      # prefill + 3 decode steps
    assert (got - want).abs().max().item() < 1e-4
    assert torch.equal(gen_got, gen_want)


def test_layer_idx_is_passed_when_the_function_takes_it_and_skip_layers_is_honoured():
    model = _tiny("llama", layers=3)
    seen = []
    apply_patch_with_prefill(model, partial(dense_prefill_with_layer, seen=seen), skip_layers=[1])
    assert not hasattr(model.model.layers[1].self_attn, "original_forward")
    with torch.no_grad():
        model(torch.randint(0, 128, (1, 16)))
    assert seen == [0, 2]


def test_unsupported_model_and_missing_prefill_fn():
    assert get_supported_model_types() == ["LlamaForCausalLM", "Qwen2ForCausalLM"]
    assert not is_model_supported(torch.nn.Linear(2, 2))
    with pytest.raises(ValueError, match="not supported"):
        apply_patch_with_prefill(torch.nn.Linear(2, 2), dense_prefill)
    model = _tiny("llama")
    apply_patch_with_prefill(model, None)
    with pytest.raises(RuntimeError, match="prefill_fn required"):
        model(torch.randint(0, 128, (1, 8)))


def test_factory_returns_partial_over_a_python_function():
    fn = get_permuted_block_sparse_attn_fwd(block_size=64, segment_size=128, threshold=0.8)
    assert isinstance(fn, partial)
    assert fn.func.__name__ == "permuted_block_sparse_attn_fwd"
    assert "layer_idx" not in fn.func.__code__.co_varnames
    assert fn.keywords["block_size"] == 64 and fn.keywords["segment_size"] == 128 and fn.keywords["threshold"] == 0.8
    assert fn.keywords["causal"] is True and fn.keywords["force_select_first_block"] is True


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["llama", "qwen2"])
def test_patched_model_on_gpu_select_all_equals_dense(kind):
    """threshold == int 1 without the forced first block is dense causal attention (reference
    pbs.py:120-121): a patched tiny model must reproduce the unpatched logits in bf16, and a sparse
    threshold must still give finite logits close to them."""
    model = _tiny(kind, torch.bfloat16).cuda()
    ids = torch.randint(0, 128, (1, 700), device="cuda")       # ragged: 700 % 64 != 0
    with torch.no_grad():
        want = model(ids).logits.float()
    apply_patch_with_prefill(model, get_permuted_block_sparse_attn_fwd(block_size=64, segment_size=128, threshold=1,
                                                                        force_select_first_block=False))
    with torch.no_grad():
        got = model(ids).logits.float()
    assert (got - want).abs().max().item() < 6e-2 and (got - want).abs().mean().item() < 6e-3
    # rebind with a sparse threshold on top of the same layers
    for layer in model.model.layers:
        layer.self_attn.forward = layer.self_attn.original_forward
    apply_patch_with_prefill(model, get_permuted_block_sparse_attn_fwd(block_size=64, segment_size=128, threshold=0.9))
    with torch.no_grad():
        sparse = model(ids).logits.float()
        out = model.generate(ids[:, :300], max_new_tokens=3, do_sample=False)
    assert torch.isfinite(sparse).all() and out.shape[1] == 303


def test_shard_config_divides_heads_and_mlp_width():
    from pbs_attn_b200.efficiency import ARCHS, shard_config
    kw = {k: v for k, v in ARCHS["llama3.1-8b"].items() if k != "kind"}
    s = shard_config(kw, 4)
    assert (s["num_attention_heads"], s["num_key_value_heads"], s["intermediate_size"]) == (8, 2, 14336 // 4)
    assert s["hidden_size"] == kw["hidden_size"] and s["head_dim"] == 128
    q = {k: v for k, v in ARCHS["qwen2.5-7b"].items() if k != "kind"}
    assert shard_config(q, 4)["head_dim"] == 128 and shard_config(q, 4)["num_key_value_heads"] == 1
    with pytest.raises(ValueError):
        shard_config(q, 8)                       # 4 KV heads do not split over 8 ranks
    assert shard_config(kw, 1) is kw


def _tp_worker(rank, world, port, q):
    import os
    import torch.distributed as dist
    from pbs_attn_b200 import efficiency
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        efficiency.ARCHS["tiny"] = dict(kind="llama", vocab_size=128, hidden_size=64, intermediate_size=128,
                                        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                                        max_position_embeddings=256)
        model = efficiency.build_model("tiny", device="cpu", world=world).float()
        efficiency.add_row_parallel_reductions(model)
        apply_patch_with_prefill(model, dense_prefill)
        ids = torch.arange(24).view(1, 24) % 128
        with torch.no_grad():
            logits = model(ids).logits
        gathered = [torch.empty_like(logits) for _ in range(world)]
        dist.all_gather(gathered, logits)
        heads = model.model.layers[0].self_attn.q_proj.out_features // 16
        q.put((rank, heads, bool(torch.equal(gathered[0], gathered[1])), bool(torch.isfinite(logits).all())))
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_slices_run_and_agree_two_ranks_gloo():
    """Two CPU ranks, each holding half of the heads and of the MLP width, with the row-parallel sums in
    place: both must produce the same (finite) logits through the patched attention forward."""
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == [(0, 2, True, True), (1, 2, True, True)]
