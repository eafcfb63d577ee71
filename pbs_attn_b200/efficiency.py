"""End-to-end prefill latency of a patched Hugging Face model: time to first token.

Follows the protocol of the reference's efficiency harness (eval/efficiency/eval_efficiency.py:
136-157, 223-245): the model's attention layers are patched with a prefill function, warmed up with
``generate(max_new_tokens=1)`` calls and then timed with CUDA events around the same call, per
context length.  There is no network here, so the model is a RANDOM-INIT decoder of a named
architecture (no checkpoint) and the prompts are uniform random token ids (the reference warms up
with exactly such ids, eval_efficiency.py:136-144, and times LongBench-v2 contexts cut to length);
latencies are comparable, selection densities are whatever random weights give and are reported.

    python -m pbs_attn_b200.efficiency --method pbs --lens 8192,32768,131072
    python -m pbs_attn_b200.efficiency --method dense --layers 8

Prints one JSON line per context length.
"""
import argparse
import json

import torch

ARCHS = {
    # the two architectures the reference evaluates (model cards' config.json values)
    "llama3.1-8b": dict(kind="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                        num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                        rope_theta=500000.0, max_position_embeddings=131072, rms_norm_eps=1e-5),
    "qwen2.5-7b": dict(kind="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                       num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
                       rope_theta=1000000.0, max_position_embeddings=131072, rms_norm_eps=1e-6),
}


def build_model(arch: str, layers=None, device="cuda", seed=0):
    """Random-init bf16 model of the named architecture, built directly on the device."""
    from transformers import LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM
    kw = dict(ARCHS[arch])
    kind = kw.pop("kind")
    if layers:
        kw["num_hidden_layers"] = layers
    cfg = (LlamaConfig if kind == "llama" else Qwen2Config)(**kw)
    torch.manual_seed(seed)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            model = (LlamaForCausalLM if kind == "llama" else Qwen2ForCausalLM)(cfg)
    finally:
        torch.set_default_dtype(prev)
    return model.eval()


def dense_prefill(query_states, key_states, value_states):
    """Dense causal attention through PyTorch's fused kernel: the unsparsified baseline arm."""
    return torch.nn.functional.scaled_dot_product_attention(query_states, key_states, value_states, is_causal=True)


def no_attention(query_states, key_states, value_states):
    """Returns the queries unchanged: the time of everything in the model except attention."""
    return query_states


def prefill_function(method: str, block_size: int, segment_size: int, threshold: float):
    from .hf_patch import get_meanpooling_prefill, get_permuted_block_sparse_attn_fwd
    if method == "pbs":
        return get_permuted_block_sparse_attn_fwd(block_size=block_size, segment_size=segment_size, threshold=threshold)
    if method == "meanpooling":
        return get_meanpooling_prefill(block_size=block_size, threshold=threshold)
    if method == "dense":
        return dense_prefill
    if method == "noattn":
        return no_attention
    raise ValueError(method)


def measure_prefill_latency(model, input_ids) -> float:
    """Seconds for one ``generate(max_new_tokens=1)`` (eval_efficiency.py:147-157)."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    with torch.no_grad():
        model.generate(input_ids=input_ids, max_new_tokens=1, do_sample=False)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / 1000.0


def last_density():
    """Selected fraction of the causal block triangle in the most recent sparse call (last layer)."""
    from . import prefill
    plans = list(prefill._PLANS.values())
    if not plans:
        return None
    m = plans[-1].block_mask
    nb = m.shape[-1]
    return float(m.sum().item()) / (m.shape[0] * m.shape[1] * nb * (nb + 1) / 2)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--arch", default="llama3.1-8b", choices=sorted(ARCHS))
    ap.add_argument("--layers", type=int, default=None, help="build only this many decoder layers")
    ap.add_argument("--method", default="pbs", choices=["pbs", "meanpooling", "dense", "noattn", "unpatched"])
    ap.add_argument("--lens", default="8192,16384,32768,65536,131072")
    ap.add_argument("--block-size", type=int, default=128)
    ap.add_argument("--segment-size", type=int, default=256)
    ap.add_argument("--threshold", type=float, default=0.9)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("the efficiency harness needs a CUDA device")
    from .hf_patch import apply_patch_with_prefill
    model = build_model(args.arch, args.layers)
    if args.method != "unpatched":
        apply_patch_with_prefill(model, prefill_function(args.method, args.block_size, args.segment_size, args.threshold))
    model.generation_config.pad_token_id = 0
    vocab = model.get_input_embeddings().weight.size(0)
    gen = torch.Generator(device="cuda").manual_seed(0)
    for length in [int(x) for x in args.lens.split(",")]:
        ids = torch.randint(0, vocab, (1, length), device="cuda", dtype=torch.long, generator=gen)
        for _ in range(args.warmup):
            measure_prefill_latency(model, ids)
        times = [measure_prefill_latency(model, ids) for _ in range(args.iters)]
        rec = {"metric": "prefill_latency_s", "arch": args.arch, "layers": model.config.num_hidden_layers,
               "method": args.method, "len": length, "mean_s": sum(times) / len(times), "min_s": min(times),
               "iters": args.iters, "warmup": args.warmup, "weights": "random-init", "prompts": "uniform random ids",
               "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
        if args.method in ("pbs", "meanpooling"):
            rec.update(block_size=args.block_size, segment_size=args.segment_size, threshold=args.threshold,
                       last_layer_density=last_density())
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
