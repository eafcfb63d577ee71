"""Same import path as the reference's orchestrator module (pbs_attn/src/pbs.py)."""
from pbs_attn_b200.prefill import permuted_block_sparse_attn_fwd  # noqa: F401
