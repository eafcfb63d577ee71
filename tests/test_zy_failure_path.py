"""The abort path of the tcgen05 attention kernel, exercised without faulting or hanging the GPU.

Every device-side wait of that kernel is bounded.  Here the bound is set to a few milliseconds and
one softmax warpgroup of CTA 0 is told to withhold a single barrier arrive (pbs_debug_set_attn_wait),
so exactly one wait runs out: the kernel must RETURN, report which wait gave up in status[0], the
host must turn that into an exception (on the next call, without synchronising, or on check_status),
and the next normal call in the same process must give the correct result again.
"""
import pytest
import torch

from pbs_attn_b200 import _cabi
from pbs_attn_b200.synth import Workload, make_qkv

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_correct():
    from pbs_attn_b200.prefill import permuted_block_sparse_attn_fwd, release_plans
    lib = _cabi.load()
    w = Workload("abort", 1, 4, 1, 128, 2048, "bf16", 128, 256, 0.9, 5e5, sinks=4)
    q, k, v = make_qkv(w, seed=77, device="cuda")
    release_plans()

    def call(inter=None):
        return permuted_block_sparse_attn_fwd(q, k, v, w.block_size, w.segment_size, w.threshold, True,
                                              attn_impl="tcgen05", intermediates=inter)

    inter = {}
    good = call(inter)
    torch.cuda.synchronize()
    plan = inter["plan"]
    plan.check_status()

    try:
        assert lib.pbs_debug_set_attn_wait(3_000_000, 1) == 0        # 3 ms bound, one arrive withheld
        call()
        torch.cuda.synchronize()                                     # the kernel returned by itself
    finally:
        assert lib.pbs_debug_set_attn_wait(0, 0) == 0
    words = plan.status.cpu().tolist()
    print("status words after the withheld arrive:", words)
    assert words[0] != 0, "the kernel did not report the wait that ran out"
    # the status words of that call have reached the host: the next call raises instead of running
    with pytest.raises(_cabi.PbsError, match="bounded wait"):
        call()
    # and check_status() says the same for the last launched call
    with pytest.raises(_cabi.PbsError):
        plan.check_status()

    # same process, same GPU, normal settings: correct again
    again = call()
    torch.cuda.synchronize()
    plan.check_status()
    assert torch.equal(again, good)
