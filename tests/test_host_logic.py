"""CPU-only checks of the host side of the prefill path, with the CUDA library and the CUDA runtime
replaced by fakes: every library call must run with the plan's device current (tensors on cuda:1
while cuda:0 is current would otherwise be launched on the wrong device), and device-side error
flags of a whole-path call are raised on a LATER call without synchronising."""
import pytest
import torch

from pbs_attn_b200 import _cabi, prefill


class FakeGuard:
    active = []

    def __init__(self, dev):
        self.dev = torch.device(dev)

    def __enter__(self):
        FakeGuard.active.append(self.dev)

    def __exit__(self, *a):
        FakeGuard.active.pop()


class FakeLib:
    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        if not name.startswith("pbs_"):
            raise AttributeError(name)

        def fn(*args):
            self.calls.append((name, list(FakeGuard.active)))
            return 0
        return fn


class FakeEvent:
    def __init__(self):
        self.done = False
        self.synced = False

    def record(self, stream=None):
        pass

    def query(self):
        return self.done

    def synchronize(self):
        self.synced = True
        self.done = True


def fake_plan(monkeypatch, device="cuda:1"):
    """A Plan whose buffers are CPU tensors and whose library / CUDA runtime are fakes."""
    FakeGuard.active = []
    monkeypatch.setattr(prefill.torch.cuda, "device", FakeGuard)
    monkeypatch.setattr(prefill.torch.cuda, "Event", FakeEvent)
    class FakeStream:
        cuda_stream = 0

    monkeypatch.setattr(prefill.torch.cuda, "current_stream", lambda dev=None: FakeStream())
    plan = object.__new__(prefill.Plan)
    plan.lib = FakeLib()
    plan.device = torch.device(device)
    plan.dtype = torch.bfloat16
    plan.shape = _cabi.Shape(1, 4, 1, 1024, 128, 128, 256, _cabi.BF16)
    plan.n_complete, plan.nb, plan._logits_numel, plan.logits = 1024, 8, 4 * 128 * 1024, None
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt)
    plan.partials, plan.rowstats, plan.importance = z(16), z(16), z(4 * 1024)
    plan.key_indices, plan.first_block = z(1, 4, 1024, dt=torch.int32), z(4, dt=torch.int32)
    plan.perm_k = plan.perm_v = z(1, 4, 1024, 128, dt=torch.bfloat16)
    plan.pooled_q = plan.pooled_k = z(1, 4, 8, 128, dt=torch.bfloat16)
    plan.block_mask = z(1, 4, 8, 8, dt=torch.uint8)
    plan.tile_list, plan.tile_count, plan.status = z(64, dt=torch.int32), z(16, dt=torch.int32), z(8, dt=torch.int32)
    plan.scratch = _cabi.Scratch()
    plan._status_ring = torch.zeros(prefill._STATUS_SLOTS, 8, dtype=torch.int32)
    plan._status_pending, plan._status_next, plan._thr_dev = [], 0, None
    monkeypatch.setattr(prefill.Plan, "_stream", lambda self: None)
    return plan


def test_every_library_call_runs_with_the_plans_device_current(monkeypatch):
    plan = fake_plan(monkeypatch, "cuda:1")
    q = torch.zeros(1, 4, 1024, 128, dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    opt = plan.options(0.9)
    plan.key_importance(q, q)
    plan.segment_permute(q, q)
    plan.pool_queries(q)
    plan.select_blocks(opt)
    plan.build_tile_lists()
    plan.attn_fwd(q, out)
    plan.run(q, q, q, out, opt)
    names = [n for n, _ in plan.lib.calls]
    assert names == ["pbs_key_importance", "pbs_segment_permute", "pbs_pool_queries", "pbs_select_blocks",
                     "pbs_build_tile_lists", "pbs_attn_fwd", "pbs_prefill_fwd"]
    for name, active in plan.lib.calls:
        assert active == [torch.device("cuda:1")], f"{name} was called without the plan's device current"
    assert FakeGuard.active == []


def test_static_scratch_entry_runs_on_the_tensors_device(monkeypatch):
    fake_plan(monkeypatch)
    lib = FakeLib()
    monkeypatch.setattr(prefill._cabi, "load", lambda: lib)

    class Q:                        # the attributes key_importance_static reads from its tensors
        shape, dtype, device = (1, 4, 1024, 128), torch.bfloat16, torch.device("cuda:3")

        def data_ptr(self):
            return 1 << 20

        def stride(self):
            return (4 * 1024 * 128, 1024 * 128, 128, 1)

    zeros = torch.zeros
    monkeypatch.setattr(prefill.torch, "empty", lambda *a, **k: zeros(*a, dtype=k.get("dtype")))
    prefill.key_importance_static(Q(), Q(), 128, 256)
    assert lib.calls == [("pbs_key_importance_static", [torch.device("cuda:3")])]


def test_device_side_error_is_raised_on_a_later_call_without_synchronising(monkeypatch):
    plan = fake_plan(monkeypatch)
    q = torch.zeros(1, 4, 1024, 128, dtype=torch.bfloat16)
    out, opt = torch.zeros_like(q), plan.options(0.9)
    plan.run(q, q, q, out, opt)                      # call 1: its status copy is still in flight
    plan.run(q, q, q, out, opt)                      # call 2: nothing has landed, nothing is inspected or awaited
    assert len(plan._status_pending) == 2 and not any(ev.synced for ev, _ in plan._status_pending)
    ev1, slot1 = plan._status_pending[0]
    plan._status_ring[slot1, 0] = 7                  # call 1's kernel gave up in wait 7 ...
    ev1.done = True                                  # ... and its status words have reached the host
    with pytest.raises(_cabi.PbsError, match="code 7"):
        plan.run(q, q, q, out, opt)
    assert plan._status_pending == []
    plan.run(q, q, q, out, opt)                      # the plan stays usable


def test_status_ring_bounds_the_host_run_ahead(monkeypatch):
    plan = fake_plan(monkeypatch)
    q = torch.zeros(1, 4, 1024, 128, dtype=torch.bfloat16)
    out, opt = torch.zeros_like(q), plan.options(0.9)
    for _ in range(prefill._STATUS_SLOTS + 3):
        plan.run(q, q, q, out, opt)
    # never more copies in flight than slots: the oldest one is awaited before its slot is reused
    assert len(plan._status_pending) <= prefill._STATUS_SLOTS
    slots = [s for _, s in plan._status_pending]
    assert len(set(slots)) == len(slots)
