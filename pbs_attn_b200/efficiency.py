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
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 -m pbs_attn_b200.efficiency --lens 262144

Under ``torch.distributed.run`` the model is tensor-parallel the way the reference's script runs it
(``tp_plan="auto"``, eval_efficiency.py:197-203, scripts/eval_efficiency.sh:14-22: 256K tokens on 4 GPUs, 512K on
8): every rank holds its slice of the attention heads and of the MLP width, and the outputs of ``o_proj`` and
``down_proj`` are summed over the ranks (one NCCL all-reduce each).  Random weights need no loading, so each rank
simply builds the architecture with its share of the heads; the attention kernels see exactly a rank's heads.

``--parallel dp`` is multi-sequence prefill instead: every rank holds the WHOLE model and its share of a batch
of ``--batch`` sequences (default: one per rank; ``sharding.shard_batch``), nothing is exchanged while
computing, a step ends when the slowest rank ends.  ``--attention-share`` times the same model a second
time with attention replaced by a no-op and reports which share of the prefill the attention call is.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m pbs_attn_b200.efficiency \
        --parallel dp --lens 65536 --attention-share --out results.jsonl

Prints one JSON line per context length (rank 0) and appends it to ``--out`` when given, like the reference
writes one result file per run (eval_efficiency.py:261-290).
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


def shard_config(kw: dict, world: int) -> dict:
    """The architecture one tensor-parallel rank holds: heads, KV heads and MLP width divided by ``world``;
    hidden size, vocabulary and layer count unchanged (column-parallel q/k/v/gate/up, row-parallel o/down)."""
    if world == 1:
        return kw
    kw = dict(kw)
    if kw["num_attention_heads"] % world or kw["num_key_value_heads"] % world or kw["intermediate_size"] % world:
        raise ValueError(f"{world} ranks do not divide the heads / MLP width of this architecture")
    kw.setdefault("head_dim", kw["hidden_size"] // kw["num_attention_heads"])
    kw["num_attention_heads"] //= world
    kw["num_key_value_heads"] //= world
    kw["intermediate_size"] //= world
    return kw


def add_row_parallel_reductions(model, group=None):
    """Sums the outputs of every ``o_proj`` and ``down_proj`` over the ranks, which is what makes the
    per-rank slices of ``shard_config`` one tensor-parallel model."""
    import torch.distributed as dist

    def hook(_module, _inputs, output):
        dist.all_reduce(output, group=group)
        return output

    handles = []
    for layer in model.model.layers:
        handles.append(layer.self_attn.o_proj.register_forward_hook(hook))
        handles.append(layer.mlp.down_proj.register_forward_hook(hook))
    return handles


def build_model(arch: str, layers=None, device="cuda", seed=0, world=1):
    """Random-init bf16 model of the named architecture (one rank's share of it when ``world`` > 1),
    built directly on the device."""
    from transformers import LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM
    kw = dict(ARCHS[arch])
    kind = kw.pop("kind")
    if layers:
        kw["num_hidden_layers"] = layers
    kw = shard_config(kw, world)
    cfg = (LlamaConfig if kind == "llama" else Qwen2Config)(**kw)
    if str(device).startswith("cuda"):
        # With the default attention setting the model materialises a (S, S) boolean causal mask for
        # every call (64 GiB at 262144 tokens); the flash-attention setting passes no dense mask.  The
        # patched layers never look at the mask, and single-token decode runs the library kernel.
        try:
            import flash_attn  # noqa: F401
            cfg._attn_implementation = "flash_attention_2"
        except ImportError:
            pass
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


no_attention.takes_grouped_kv = True      # no repeat_kv copies either: they belong to the attention call being replaced


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
    ap.add_argument("--slice-of", type=int, default=1, metavar="N",
                    help="on ONE GPU, run the slice one rank of an N-way tensor-parallel model holds, without the "
                         "all-reduces: the compute side of a multi-GPU point when no multi-GPU machine is at hand")
    ap.add_argument("--parallel", default="tp", choices=["tp", "dp"],
                    help="under torch.distributed.run: tensor parallel (heads and MLP width split, the reference's "
                         "tp_plan) or data parallel (whole model per rank, the batch split)")
    ap.add_argument("--batch", type=int, default=None, help="sequences per step (data parallel: default one per rank)")
    ap.add_argument("--attention-share", action="store_true",
                    help="time the model a second time with attention replaced by a no-op and report the share")
    ap.add_argument("--out", default=None, help="append the JSON lines to this file (rank 0)")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("the efficiency harness needs a CUDA device")
    import os
    import torch.distributed as dist
    from .sharding import shard_batch
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from .hf_patch import apply_patch_with_prefill, remove_patch
    if args.slice_of > 1 and world > 1:
        raise SystemExit("--slice-of is for single-process runs")
    tp = world if args.parallel == "tp" else 1
    model = build_model(args.arch, args.layers, device=f"cuda:{local_rank}", world=max(tp, args.slice_of))
    if tp > 1:
        add_row_parallel_reductions(model)
    model.generation_config.pad_token_id = 0
    vocab = model.get_input_embeddings().weight.size(0)
    dev = torch.device("cuda", local_rank)
    batch = args.batch or (world if args.parallel == "dp" else 1)
    mine = shard_batch(batch, rank, world) if args.parallel == "dp" else slice(0, batch)
    methods = [args.method] + (["noattn"] if args.attention_share and args.method != "noattn" else [])

    def timed(method, ids):
        remove_patch(model)
        if method != "unpatched":
            apply_patch_with_prefill(model, prefill_function(method, args.block_size, args.segment_size, args.threshold))
        if ids.shape[0] == 0:                                   # a rank without a sequence of this batch
            times = [0.0] * args.iters
        else:
            for _ in range(args.warmup):
                measure_prefill_latency(model, ids)
            times = [measure_prefill_latency(model, ids) for _ in range(args.iters)]
        if world > 1:                                            # a step ends when the slowest rank ends
            t = torch.tensor(times, dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times = t.tolist()
        return times

    for length in [int(x) for x in args.lens.split(",")]:
        gen = torch.Generator(device=dev).manual_seed(length)    # same ids on every rank
        ids = torch.randint(0, vocab, (batch, length), device=dev, dtype=torch.long, generator=gen)[mine]
        results = {m: timed(m, ids) for m in methods}
        density = last_density() if args.method in ("pbs", "meanpooling") else None
        if rank != 0:
            continue
        times = results[args.method]
        mean_s = sum(times) / len(times)
        rec = {"metric": "prefill_latency_s", "arch": args.arch, "layers": model.config.num_hidden_layers,
               "parallel": args.parallel if world > 1 else "none", "world": world, "tp": tp, "slice_of": args.slice_of,
               "batch": batch, "method": args.method, "len": length, "mean_s": mean_s, "min_s": min(times),
               "tokens_per_s": batch * length / mean_s,
               "iters": args.iters, "warmup": args.warmup, "weights": "random-init", "prompts": "uniform random ids",
               "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
        if args.method in ("pbs", "meanpooling"):
            rec.update(block_size=args.block_size, segment_size=args.segment_size, threshold=args.threshold,
                       last_layer_density=density)
        if "noattn" in results and args.method != "noattn":
            rest = sum(results["noattn"]) / len(results["noattn"])
            rec.update(without_attention_s=rest, attention_s=mean_s - rest, attention_share=(mean_s - rest) / mean_s)
        line = json.dumps(rec)
        print(line, flush=True)
        if args.out:
            with open(args.out, "a") as f:
                f.write(line + "\n")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
