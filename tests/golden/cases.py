"""The seeded cases behind the golden fixtures (shared by the generator and the tests)."""
from pbs_attn_b200.synth import Workload

# name -> (workload, seed, extra kwargs of the attention call, row stride of the stored output)
CASES = {
    # task configuration 1: the CPU op-level check
    "op_check_fp32": (Workload("op_check_fp32", 1, 4, 1, 64, 2048, "fp32", 64, 256, 0.9, 1e4), 0, {}, 8),
    # Llama-3.1-8B head shape, shortened sequence, with sink tokens
    "llama_bf16_s4096": (Workload("llama_bf16_s4096", 1, 8, 2, 128, 4096, "bf16", 128, 256, 0.9, 5e5, sinks=4), 1, {}, 16),
    "llama_bf16_t080": (Workload("llama_bf16_t080", 1, 4, 1, 128, 2048, "bf16", 128, 256, 0.8, 5e5, sinks=4), 2, {}, 8),
    "llama_bf16_t095": (Workload("llama_bf16_t095", 1, 4, 1, 128, 2048, "bf16", 128, 256, 0.95, 5e5, sinks=4), 3, {}, 8),
    # Qwen2.5-7B head shape (7 query heads per KV head), small blocks and segments
    "qwen_bf16_bs64_seg128": (Workload("qwen_bf16_bs64_seg128", 1, 7, 1, 128, 2048, "bf16", 64, 128, 0.9, 1e6, density=0.08), 4, {}, 8),
    "qwen_bf16_seg512": (Workload("qwen_bf16_seg512", 1, 7, 1, 128, 3072, "bf16", 128, 512, 0.9, 1e6, density=0.005), 5, {}, 8),
    # ragged lengths: S % block_size != 0 and S % segment_size != 0
    "ragged_fp32_s1000": (Workload("ragged_fp32_s1000", 1, 2, 2, 64, 1000, "fp32", 64, 256, 0.9, 1e4), 6, {}, 4),
    "ragged_bf16_s1900": (Workload("ragged_bf16_s1900", 2, 4, 2, 128, 1900, "bf16", 128, 256, 0.9, 5e5, sinks=4), 7, {}, 8),
    # batch 2, fp16
    "batch2_fp16": (Workload("batch2_fp16", 2, 2, 1, 64, 1024, "fp16", 64, 256, 0.9, 1e4), 8, {}, 4),
    # options
    "no_first_block": (Workload("no_first_block", 1, 2, 1, 64, 1024, "fp32", 64, 256, 0.7, 1e4), 9,
                       {"force_select_first_block": False}, 4),
    "dense_int_threshold": (Workload("dense_int_threshold", 1, 2, 1, 64, 1024, "fp32", 64, 256, 1, 1e4), 10,
                            {"force_select_first_block": False}, 4),
    "max_pool": (Workload("max_pool", 1, 2, 1, 64, 1024, "bf16", 64, 256, 0.9, 1e4), 11,
                 {"query_pool_mode": "max", "key_pool_mode": "max"}, 4),
    "threshold_never_reached": (Workload("threshold_never_reached", 1, 2, 1, 64, 1024, "fp32", 64, 256, 1.5, 1e4), 12, {}, 4),
    # q_len <= segment_size: the dense fallback
    "short_dense": (Workload("short_dense", 1, 4, 2, 64, 200, "bf16", 64, 256, 0.9, 1e4), 13, {}, 1),
}

# MeanPooling baseline (selection without permutation): segment_size is unused by it
MEANPOOLING_CASES = {
    "meanpool_bf16_s2048": (Workload("meanpool_bf16_s2048", 1, 4, 1, 128, 2048, "bf16", 128, 128, 0.9, 5e5, sinks=4), 21, {}, 8),
    "meanpool_bf16_bs64_s1500": (Workload("meanpool_bf16_bs64_s1500", 1, 4, 2, 128, 1500, "bf16", 64, 64, 0.8, 1e6, density=0.05), 22, {}, 4),
    "meanpool_fp32_s1000": (Workload("meanpool_fp32_s1000", 2, 2, 2, 64, 1000, "fp32", 64, 64, 0.9, 1e4), 23,
                            {"force_select_first_block": False}, 4),
    # the q block's own kv block is an ordinary candidate (force_select_current_block=False)
    "meanpool_no_current_bf16": (Workload("meanpool_no_current_bf16", 1, 4, 1, 128, 2048, "bf16", 128, 128, 0.6, 5e5, sinks=4), 24,
                                 {"force_select_current_block": False}, 8),
    # ... and nothing forced at all with a threshold no row reaches: nothing is attended, the output is zero
    "meanpool_nothing_fp32": (Workload("meanpool_nothing_fp32", 1, 2, 2, 64, 1000, "fp32", 64, 64, 1.5, 1e4), 25,
                              {"force_select_first_block": False, "force_select_current_block": False}, 4),
}


# Rotary embedding (the step before the path): name -> (dtype, B, H, Hkv, S, D, theta, broadcast cos/sin over the batch)
ROPE_CASES = {
    "rope_bf16": ("bf16", 2, 3, 1, 77, 128, 5e5, False),
    "rope_fp16": ("fp16", 1, 8, 2, 300, 64, 1e4, True),
    "rope_fp32": ("fp32", 2, 2, 2, 33, 128, 1e6, True),
}


def rope_inputs(case):
    """Seeded q, k in the layout the attention layer produces ((B, S, H*D) projections viewed as (B, H, S, D)) and
    cos / sin tables (B or 1, S, D) of the same dtype, all on the CPU."""
    import torch
    dt, B, H, Hkv, S, D, theta, bcast = case
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[dt]
    g = torch.Generator().manual_seed(1234 + S)
    q = torch.randn(B, S, H * D, generator=g).to(dtype).view(B, S, H, D).transpose(1, 2)
    k = torch.randn(B, S, Hkv * D, generator=g).to(dtype).view(B, S, Hkv, D).transpose(1, 2)
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    pos = torch.arange(S, dtype=torch.float32) + 3.0 * torch.arange(B, dtype=torch.float32)[:, None]
    ang = pos[..., None] * inv
    emb = torch.cat([ang, ang], dim=-1)
    cos, sin = emb.cos().to(dtype), emb.sin().to(dtype)
    if bcast:
        cos, sin = cos[:1], sin[:1]
    return q, k, cos, sin
