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
    assert z.logits == 4 * 64 * 2048
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
