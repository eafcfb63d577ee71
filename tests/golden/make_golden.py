"""Generates tests/golden/*.npz by running the UNMODIFIED reference on seeded inputs.

Run once, on a machine that has the reference checked out (it is imported from the
directory named by the REFERENCE_ROOT environment variable and is not needed afterwards):

    REFERENCE_ROOT=<reference checkout> python tests/golden/make_golden.py [--meanpooling-only] [--rope-only] [--only=case,case]

Per case two runs are stored: ``*_ref`` from the reference as it is (its sorts
are non-stable: the order of tied items is implementation defined) and
``*_stable`` from the same code with ``torch.sort`` / ``torch.argsort`` forced to
``stable=True`` by a shim, which is the canonical tie-break the CUDA path and
the oracle implement.  Inputs are regenerated from the seed by
``pbs_attn_b200.synth.make_qkv``; their SHA-256 is stored so that a drift of the
random generator is detected instead of silently changing the comparison.
"""
import contextlib
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REFERENCE_ROOT = os.environ.get("REFERENCE_ROOT")
if not REFERENCE_ROOT:
    raise SystemExit("set REFERENCE_ROOT to the directory of the reference checkout")


def _import_reference():
    """Import the reference's pbs_attn package, shadowing any same-named package of this repo."""
    for name in [m for m in sys.modules if m == "pbs_attn" or m.startswith("pbs_attn.")]:
        del sys.modules[name]
    sys.path.insert(0, REFERENCE_ROOT)
    try:
        import pbs_attn.src.pbs as ref_pbs
        assert os.path.abspath(ref_pbs.__file__).startswith(os.path.abspath(REFERENCE_ROOT)), ref_pbs.__file__
    finally:
        sys.path.remove(REFERENCE_ROOT)
    return ref_pbs


@contextlib.contextmanager
def stable_sorts():
    sort, argsort = torch.sort, torch.argsort

    def s(x, *a, **k):
        k["stable"] = True
        return sort(x, *a, **k)

    def a_(x, *a, **k):
        k["stable"] = True
        return argsort(x, *a, **k)

    torch.sort, torch.argsort = s, a_
    try:
        yield
    finally:
        torch.sort, torch.argsort = sort, argsort


def sha_inputs(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def raw(t: torch.Tensor) -> np.ndarray:
    """bit pattern of a tensor as a numpy array (bf16/fp16 -> uint16, fp32 -> float32)."""
    t = t.contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def run_reference(ref_pbs, q, k, v, w, kwargs):
    """One reference call plus its intermediates, obtained by calling its own stage functions."""
    n_rep = w.q_heads // w.kv_heads
    kr, vr = k.repeat_interleave(n_rep, dim=1), v.repeat_interleave(n_rep, dim=1)
    out = ref_pbs.permuted_block_sparse_attn_fwd(q, kr, vr, w.block_size, w.segment_size, w.threshold,
                                                 True, use_triton=False, **kwargs)
    if w.seq_len <= w.segment_size:
        return out, None, None, None
    perm_k, idx = ref_pbs.apply_permutation(q, kr, w.block_size, w.segment_size)
    qi = torch.arange(w.seq_len).view(1, 1, -1).expand(w.batch, w.q_heads, -1)
    scores, mask, seg_mask = ref_pbs.permuted_block_selection(
        q, perm_k, qi, idx, w.block_size, w.segment_size, threshold=w.threshold, causal=True, **kwargs)
    mask = mask | seg_mask[None, None]
    return out, idx, mask, scores


class _BlockSparseAttnStub:
    """Stands in for the external ``block_sparse_attn`` library the MeanPooling baseline imports
    (it is not part of the reference project).  ``block_sparse_attn_func`` keeps the block mask the
    reference computed and evaluates the library's documented contract in fp32: softmax over the
    keys of the selected blocks, element-causal, result rounded to the input dtype."""

    def __init__(self):
        self.block_mask = None

    def block_sparse_attn_func(self, q, k, v, cu_q, cu_k, head_mask_type, streaming_info, block_mask,
                               max_q, max_k, p_dropout=0.0, deterministic=True, is_causal=True):
        assert is_causal and p_dropout == 0.0 and streaming_info is None
        self.block_mask = block_mask.clone()
        S, H, D = q.shape
        bs = (S + block_mask.shape[-1] - 1) // block_mask.shape[-1]
        bs = 1 << (bs - 1).bit_length()                       # block sizes in the cases are powers of two
        elem = block_mask[0].repeat_interleave(bs, dim=-2).repeat_interleave(bs, dim=-1)[:, :S, :S]
        elem = elem & torch.tril(torch.ones(S, S, dtype=torch.bool))
        logits = torch.einsum("qhd,khd->hqk", q.float(), k.float()) / (D ** 0.5)
        p = torch.softmax(logits.masked_fill(~elem, float("-inf")), dim=-1)
        p = torch.nan_to_num(p, nan=0.0)                     # rows without a visible key attend nothing: zeros
        return torch.einsum("hqk,khd->qhd", p, v.float()).to(q.dtype)


def make_meanpooling(make_qkv, cases):
    """MeanPooling fixtures: the reference's own MeanPooling_prefill (pbs_attn/baselines/MeanPooling.py)
    run unmodified with the stub above in place of the external attention library."""
    import types
    stub = _BlockSparseAttnStub()
    mod = types.ModuleType("block_sparse_attn")
    mod.block_sparse_attn_func = stub.block_sparse_attn_func
    sys.modules["block_sparse_attn"] = mod
    sys.path.insert(0, REFERENCE_ROOT)
    try:
        import pbs_attn.baselines.MeanPooling as ref_mp
        import pbs_attn.src.utils as ref_utils
        assert os.path.abspath(ref_mp.__file__).startswith(os.path.abspath(REFERENCE_ROOT)), ref_mp.__file__
    finally:
        sys.path.remove(REFERENCE_ROOT)
    only = [a.split("=", 1)[1].split(",") for a in sys.argv if a.startswith("--only=")]
    for name, (w, seed, kwargs, stride) in cases.items():
        if only and name not in only[0]:
            continue
        q, k, v = make_qkv(w, seed)
        n_rep = w.q_heads // w.kv_heads
        kr, vr = k.repeat_interleave(n_rep, dim=1), v.repeat_interleave(n_rep, dim=1)
        rec = {"inputs_sha256": np.array(sha_inputs(q, k, v)), "row_stride": np.array(stride)}
        for tag, ctx in (("ref", contextlib.nullcontext()), ("stable", stable_sorts())):
            outs, masks = [], []
            with ctx:
                for b in range(w.batch):                      # the baseline asserts batch size 1
                    outs.append(ref_mp.MeanPooling_prefill(q[b:b + 1], kr[b:b + 1], vr[b:b + 1], block_size=w.block_size,
                                                           threshold=w.threshold, **kwargs))
                    masks.append(stub.block_mask)
            out, mask = torch.cat(outs), torch.cat(masks)
            rec[f"out_{tag}"] = raw(out[:, :, ::stride, :])
            rec[f"mask_{tag}"] = np.packbits(mask.numpy(), axis=-1)
        # the pooled scores, from the reference's own scoring function on the same padded inputs
        pad = (-w.seq_len) % w.block_size
        qp = torch.nn.functional.pad(q, (0, 0, 0, pad)); kp = torch.nn.functional.pad(kr, (0, 0, 0, pad))
        nb = (w.seq_len + pad) // w.block_size
        rec["scores"] = ref_utils.block_pooled_attn(qp, kp, w.block_size, torch.tril(torch.ones(nb, nb, dtype=torch.bool))).numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **rec)
        print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB, ref==stable mask: "
              f"{np.array_equal(rec['mask_ref'], rec['mask_stable'])}")


def make_rope():
    """Rotary-embedding fixture: the reference's own apply_rotary_pos_emb (pbs_attn/patch/huggingface.py:19-25)
    on seeded inputs in the layout its attention layer produces, for the three dtypes."""
    sys.path.insert(0, REFERENCE_ROOT)
    try:
        for name in [m for m in sys.modules if m == "pbs_attn" or m.startswith("pbs_attn.")]:
            del sys.modules[name]
        import pbs_attn.patch.huggingface as ref_hf
        assert os.path.abspath(ref_hf.__file__).startswith(os.path.abspath(REFERENCE_ROOT)), ref_hf.__file__
    finally:
        sys.path.remove(REFERENCE_ROOT)
    sys.path.insert(0, HERE)
    from cases import ROPE_CASES, rope_inputs
    rec = {}
    for name, case in ROPE_CASES.items():
        q, k, cos, sin = rope_inputs(case)
        qe, ke = ref_hf.apply_rotary_pos_emb(q, k, cos, sin)
        rec[f"{name}_q"], rec[f"{name}_k"] = raw(qe), raw(ke)
        rec[f"{name}_sha"] = np.array(sha_inputs(q, k, cos, sin))
    path = os.path.join(HERE, "rope.npz")
    np.savez_compressed(path, **rec)
    print(f"rope: {os.path.getsize(path) / 1024:.0f} KiB, {len(ROPE_CASES)} cases")


def main():
    sys.path.insert(0, ROOT)
    if "--rope-only" in sys.argv:
        make_rope()
        return
    from pbs_attn_b200.synth import make_qkv
    sys.path.insert(0, HERE)
    from cases import CASES, MEANPOOLING_CASES
    ref_pbs = _import_reference()
    torch.set_num_threads(os.cpu_count() or 1)
    if "--meanpooling-only" in sys.argv:
        make_meanpooling(make_qkv, MEANPOOLING_CASES)
        return
    make_meanpooling(make_qkv, MEANPOOLING_CASES)
    make_rope()
    for name, (w, seed, kwargs, stride) in CASES.items():
        q, k, v = make_qkv(w, seed)
        rec = {"inputs_sha256": np.array(sha_inputs(q, k, v)), "row_stride": np.array(stride)}
        for tag, ctx in (("ref", contextlib.nullcontext()), ("stable", stable_sorts())):
            with ctx:
                out, idx, mask, scores = run_reference(ref_pbs, q, k, v, w, kwargs)
            rec[f"out_{tag}"] = raw(out[:, :, ::stride, :])
            if idx is not None:
                rec[f"idx_{tag}"] = idx.to(torch.int32).numpy()
                rec[f"mask_{tag}"] = np.packbits(mask.numpy(), axis=-1)
                if tag == "stable":
                    rec["scores"] = torch.nan_to_num(scores, nan=-1.0).numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **rec)
        same = "idx_ref" not in rec or (np.array_equal(rec["idx_ref"], rec["idx_stable"]),
                                         np.array_equal(rec["mask_ref"], rec["mask_stable"]))
        print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB, ref==stable (idx, mask): {same}")


if __name__ == "__main__":
    main()
