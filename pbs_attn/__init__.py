"""Drop-in module path of the reference package (pbs_attn/__init__.py:4): same import, served
by the B200 CUDA library in pbs_attn_b200."""
from pbs_attn_b200.prefill import permuted_block_sparse_attn_fwd  # noqa: F401
