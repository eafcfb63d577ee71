"""Same import path as the reference's baseline module (pbs_attn/baselines/MeanPooling.py)."""
from pbs_attn_b200.prefill import MeanPooling_prefill  # noqa: F401
