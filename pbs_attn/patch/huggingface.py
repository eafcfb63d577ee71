"""Same import path as the reference's patch module (pbs_attn/patch/huggingface.py)."""
from pbs_attn_b200.hf_patch import (  # noqa: F401
    apply_patch_with_prefill,
    apply_rotary_pos_emb,
    get_meanpooling_prefill,
    get_permuted_block_sparse_attn_fwd,
    get_supported_model_types,
    is_model_supported,
    patched_attention_forward,
    repeat_kv,
    rotate_half,
)
