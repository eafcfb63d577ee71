"""CPU-only checks of the C-ABI library: it loads without a GPU driver, exports every symbol the
header declares, and rejects bad shapes with the documented codes (no kernel is launched)."""
import ctypes as C
import os
import re

import pytest

from pbs_attn_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_cabi.lib_path()):
        from pbs_attn_b200.build import build
        build()
    return _cabi.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "pbs_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pbs_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/pbs_b200.h but not exported"
    assert set(names) == set(_cabi.EXPORTS)


def test_version(lib):
    assert lib.pbs_version() >= 100


def _shape(**kw):
    d = dict(batch=1, q_heads=4, kv_heads=1, seq_len=2048, head_dim=64, block_size=64, segment_size=256, dtype=_cabi.FP32)
    d.update(kw)
    return _cabi.Shape(**d)


def test_scratch_sizes(lib):
    z = _cabi.ScratchSizes()
    assert lib.pbs_scratch_sizes(C.byref(_shape()), C.byref(z)) == 0
    assert z.key_indices == 4 * 2048
    assert z.perm_kv == 4 * 2048 * 64
    assert z.block_mask == 4 * 32 * 32
    assert z.logits == 4 * 64 * 2048          # size of the optional inspection output
    assert z.partials == 4 * 32 * 64 and z.rowstats == 4 * 64
    assert z.tile_list == 4 * 8 * 16 and z.tile_count == 4 * 8


@pytest.mark.parametrize("kw,code", [
    (dict(kv_heads=3), -1),
    (dict(head_dim=100), -1),
    (dict(block_size=24), -1),
    (dict(segment_size=96), -1),
    (dict(seq_len=0), -1),
    (dict(dtype=7), -3),
    (dict(seq_len=64 * 5000), -1),
])
def test_bad_shapes_are_rejected(lib, kw, code):
    z = _cabi.ScratchSizes()
    assert lib.pbs_scratch_sizes(C.byref(_shape(**kw)), C.byref(z)) == code
    assert len(lib.pbs_last_error_string()) > 0


def test_null_and_layout_arguments_are_rejected_before_any_launch(lib):
    sh = _shape()
    st = _cabi.Strides4(2048 * 4 * 64, 64, 4 * 64, 1)
    # null tensor
    assert lib.pbs_pool_queries(C.byref(sh), None, st, C.c_void_p(16), 0, None) == -3
    # non-unit inner stride
    bad = _cabi.Strides4(2048 * 4 * 64, 64, 4 * 64, 2)
    assert lib.pbs_pool_queries(C.byref(sh), C.c_void_p(1 << 20), bad, C.c_void_p(1 << 21), 0, None) == -2
    # misaligned base
    assert lib.pbs_pool_queries(C.byref(sh), C.c_void_p((1 << 20) + 4), st, C.c_void_p(1 << 21), 0, None) == -2
    # invalid pool mode
    assert lib.pbs_pool_queries(C.byref(sh), C.c_void_p(1 << 20), st, C.c_void_p(1 << 21), 5, None) == -3
    assert b"pool mode" in lib.pbs_last_error_string()


def test_cpu_tensors_are_refused():
    import torch
    from pbs_attn_b200.prefill import permuted_block_sparse_attn_fwd
    q = torch.zeros(1, 2, 512, 64)
    with pytest.raises(RuntimeError, match="CUDA"):
        permuted_block_sparse_attn_fwd(q, q, q, 64, 256, 0.9, True)


def _scratch(**null):
    """A scratch struct of plausible (never dereferenced) addresses, with the named fields NULL."""
    names = [n for n, _ in _cabi.Scratch._fields_]
    vals = {n: (i + 1) << 24 for i, n in enumerate(names)}
    vals["logits"] = None
    for n in null:
        vals[n] = None
    return _cabi.Scratch(*[vals[n] for n in names])


def _options(**kw):
    d = dict(threshold_per_head=None, threshold=0.9, select_all=0, force_select_first_block=1, query_pool_mode=0,
             key_pool_mode=0, attn_impl=0, no_permutation=0, diagonal_candidates=0, no_own_segment=0,
             out_replicas=None)
    d.update(kw)
    return _cabi.Options(*[d[n] for n, _ in _cabi.Options._fields_])


@pytest.mark.parametrize("what,code", [
    ("null_tile_list", -3), ("null_partials", -3), ("tcgen05_on_fp32", -5), ("misaligned_out", -2),
    ("bad_pool_mode", -3), ("bad_attn_impl", -3), ("zero_stride_q_with_tcgen05", -5),
])
def test_whole_path_call_validates_everything_before_the_first_enqueue(lib, what, code):
    """A rejected pbs_prefill_fwd must not leave earlier stages on the stream.  Without a GPU driver the
    first enqueue (the status memset) would fail with PBS_ERR_CUDA (-4), so getting the validation
    code instead shows that the check came first; the launch counter must not move either."""
    sh = _shape(dtype=_cabi.BF16, head_dim=128, block_size=128, q_heads=4, kv_heads=1)
    st = _cabi.Strides4(2048 * 4 * 128, 2048 * 128, 128, 1)
    q = k = v = C.c_void_p(1 << 30)
    out, ost, sc, opt, qst = C.c_void_p(1 << 31), st, _scratch(), _options(), st
    if what == "null_tile_list":
        sc = _scratch(tile_list=True)
    elif what == "null_partials":
        sc = _scratch(partials=True)
    elif what == "tcgen05_on_fp32":
        sh, opt = _shape(), _options(attn_impl=2)
        st = qst = ost = _cabi.Strides4(2048 * 4 * 64, 2048 * 64, 64, 1)
    elif what == "misaligned_out":
        out = C.c_void_p((1 << 31) + 2)
    elif what == "bad_pool_mode":
        opt = _options(key_pool_mode=3)
    elif what == "bad_attn_impl":
        opt = _options(attn_impl=9)
    elif what == "zero_stride_q_with_tcgen05":
        qst, opt = _cabi.Strides4(2048 * 128, 0, 128, 1), _options(attn_impl=2)
    before = lib.pbs_launch_count()
    rc = lib.pbs_prefill_fwd(C.byref(sh), q, qst, k, st, v, st, out, ost, C.byref(opt), C.byref(sc), None)
    assert rc == code, lib.pbs_last_error_string()
    assert lib.pbs_launch_count() == before


def test_key_importance_checks_scratch_alignment(lib):
    sh = _shape()
    st = _cabi.Strides4(2048 * 4 * 64, 2048 * 64, 64, 1)
    ok = C.c_void_p(1 << 24)
    rc = lib.pbs_key_importance(C.byref(sh), ok, st, ok, st, None, C.c_void_p((1 << 25) + 4), ok, ok, None)
    assert rc == -2 and b"alignment" in lib.pbs_last_error_string()
    rc = lib.pbs_key_importance(C.byref(sh), ok, st, ok, st, C.c_void_p((1 << 26) + 8), ok, ok, ok, None)
    assert rc == -2


def test_wait_limit_knob_rejects_negative_values(lib):
    assert lib.pbs_debug_set_attn_wait(-1, 0) == -3
    assert lib.pbs_debug_set_attn_wait(0, 0) == 0
