"""ctypes binding of libpbs_b200.so (declared in include/pbs_b200.h).

The library is built in-tree by ``python -m pbs_attn_b200.build`` and is the only
compute backend: there is no CPU or PyTorch fallback, a missing library raises.
"""
from __future__ import annotations

import ctypes as C
import os

# PBS_B200_LIB points at an alternative build of the same library (e.g. an instrumented one)
_LIB_PATH = os.environ.get("PBS_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libpbs_b200.so")

BF16, FP16, FP32 = 0, 1, 2
POOL = {"mean": 0, "max": 1}
ATTN_IMPL = {"auto": 0, "simt": 1, "tcgen05": 2}
STATIC_SCRATCH_BYTES = 64 << 20


class Shape(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("batch", "q_heads", "kv_heads", "seq_len", "head_dim", "block_size", "segment_size", "dtype")]


class ScratchSizes(C.Structure):
    _fields_ = [(n, C.c_int64) for n in
                ("logits", "partials", "rowstats", "importance", "key_indices", "perm_kv", "pooled",
                 "first_block", "block_mask", "tile_list", "tile_count", "status")]


class Scratch(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("logits", "partials", "rowstats", "importance", "key_indices", "perm_k", "perm_v",
                 "pooled_q", "pooled_k", "first_block", "block_mask", "tile_list", "tile_count", "status")]


MAX_OUT_REPLICAS = 15


class OutReplicas(C.Structure):
    _fields_ = [("count", C.c_int32), ("reserved", C.c_int32), ("out", C.c_void_p * MAX_OUT_REPLICAS)]


class Options(C.Structure):
    _fields_ = [("threshold_per_head", C.c_void_p), ("threshold", C.c_float), ("select_all", C.c_int32),
                ("force_select_first_block", C.c_int32), ("query_pool_mode", C.c_int32),
                ("key_pool_mode", C.c_int32), ("attn_impl", C.c_int32), ("no_permutation", C.c_int32),
                ("diagonal_candidates", C.c_int32), ("no_own_segment", C.c_int32),
                ("out_replicas", C.POINTER(OutReplicas))]


Strides4 = C.c_int64 * 4
_P = C.c_void_p
_SH = C.POINTER(Shape)
_ST = C.POINTER(C.c_int64)

# name -> argument types; every function returns int except the two noted below
SIGNATURES = {
    "pbs_debug_set_attn_wait": [C.c_int64, C.c_int32],
    "pbs_scratch_sizes": [_SH, C.POINTER(ScratchSizes)],
    "pbs_key_importance": [_SH, _P, _ST, _P, _ST, _P, _P, _P, _P, _P],
    "pbs_apply_rope": [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _ST, _P, _P, _ST, _P],
    "pbs_key_importance_static": [_SH, _P, _ST, _P, _ST, _P, _P],
    "pbs_segment_permute": [_SH, _P, _P, _ST, _P, _ST, _P, _P, _P, _P, C.c_int32, _P, _P],
    "pbs_pool_queries": [_SH, _P, _ST, _P, C.c_int32, _P],
    "pbs_select_blocks": [_SH, _P, _P, _P, C.POINTER(Options), _P, _P, _P],
    "pbs_build_tile_lists": [_SH, _P, _P, _P, _P],
    "pbs_attn_fwd": [_SH, _P, _ST, _P, _P, _P, _P, _P, _P, _P, _ST, C.c_int32, _P, C.POINTER(OutReplicas), _P],
    "pbs_debug_set_select_impl": [C.c_int32],
    "pbs_enable_peer_access": [C.c_int32],
    "pbs_ipc_export": [_P, C.POINTER(C.c_ubyte * 64), C.POINTER(C.c_int64)],
    "pbs_ipc_import": [C.POINTER(C.c_ubyte * 64), C.POINTER(C.c_void_p)],
    "pbs_ipc_release": [_P],
    "pbs_prefill_fwd": [_SH, _P, _ST, _P, _ST, _P, _ST, _P, _ST, C.POINTER(Options), C.POINTER(Scratch), _P],
}
EXPORTS = ["pbs_last_error_string", "pbs_version", "pbs_launch_count"] + list(SIGNATURES)

_lib = None


def lib_path() -> str:
    return _LIB_PATH


def load():
    """Loads the library once; raises RuntimeError if it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m pbs_attn_b200.build` "
            "(there is no fallback path)")
    lib = C.CDLL(_LIB_PATH)
    lib.pbs_last_error_string.restype = C.c_char_p
    lib.pbs_last_error_string.argtypes = []
    lib.pbs_version.restype = C.c_int
    lib.pbs_version.argtypes = []
    lib.pbs_launch_count.restype = C.c_int64
    lib.pbs_launch_count.argtypes = []
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = args
    _lib = lib
    return lib


class PbsError(RuntimeError):
    pass


def check(rc: int, what: str):
    if rc != 0:
        raise PbsError(f"{what} failed ({rc}): {load().pbs_last_error_string().decode()}")
