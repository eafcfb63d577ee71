"""pbs_key_importance_static: the key-importance stage with its scratch inside the library image,
for hosts that may pass only inputs and outputs (a plugin boundary that owns all device memory, a
running serving loop that must not call cudaMalloc).  It has to give what pbs_key_importance gives
with caller-provided scratch.  Collected last on purpose (file name), and self-contained: it passes
alone in a fresh process and after the rest of the suite."""
import ctypes as C

import pytest
import torch

from pbs_attn_b200 import _cabi
from pbs_attn_b200.synth import Workload, make_qkv


def test_oversized_shape_is_rejected_without_touching_the_gpu():
    lib = _cabi.load()
    # 32 heads x 8192 key tiles x 128 rows x 8 bytes of softmax statistics = 256 MiB: beyond the 64 MiB array
    shape = _cabi.Shape(1, 32, 8, 524288, 128, 128, 256, _cabi.BF16)
    st = _cabi.Strides4(524288 * 128 * 32, 524288 * 128, 128, 1)
    rc = lib.pbs_key_importance_static(C.byref(shape), C.c_void_p(1 << 20), st, C.c_void_p(1 << 21), st,
                                       C.c_void_p(1 << 22), None)
    assert rc == -1
    msg = lib.pbs_last_error_string().decode()
    assert "scratch" in msg and str(_cabi.STATIC_SCRATCH_BYTES) in msg


@pytest.mark.gpu
def test_static_scratch_entry_matches_caller_scratch_entry_on_two_calls_in_a_row():
    from pbs_attn_b200.prefill import Plan, key_importance_static
    cases = [Workload("a", 1, 4, 1, 128, 4096, "bf16", 128, 256, 0.9, 5e5, sinks=4),
             Workload("b", 2, 2, 2, 64, 1000, "fp32", 64, 256, 0.9, 1e4)]      # second call: other dtype, smaller
    for n, w in enumerate(cases):
        q, k, _ = make_qkv(w, seed=40 + n, device="cuda")
        plan = Plan(w.batch, w.q_heads, w.kv_heads, w.seq_len, w.head_dim, w.block_size, w.segment_size, w.torch_dtype, q.device)
        want = plan.key_importance(q, k).clone()
        got = key_importance_static(q, k, w.block_size, w.segment_size)
        torch.cuda.synchronize()
        assert got.shape == want.shape
        # same tolerance as the importance check of the stage tests (relative 2e-5); in practice the
        # two entry points run the same kernels and agree bit for bit
        rel = ((got - want).abs() / want.abs().clamp_min(1e-30)).max().item()
        assert rel <= 2e-5, f"call {n}: max relative difference {rel:.2e}"
        assert torch.isfinite(got).all()
