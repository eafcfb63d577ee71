"""Helpers shared by the parity tests: fixture loading and mismatch classification."""
import hashlib
import os

import numpy as np
import torch

from cases import CASES, MEANPOOLING_CASES
from pbs_attn_b200.synth import make_qkv

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Output tolerances of the task statement for bf16/fp16; fp32 calls are held tighter.
TOL = {torch.bfloat16: (2e-2, 2e-3), torch.float16: (2e-2, 2e-3), torch.float32: (2e-4, 2e-5)}


def load_case(name):
    w, seed, kwargs, stride = (CASES.get(name) or MEANPOOLING_CASES[name])
    q, k, v = make_qkv(w, seed)
    g = dict(np.load(os.path.join(GOLDEN_DIR, name + ".npz")))
    h = hashlib.sha256()
    for t in (q, k, v):
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    assert h.hexdigest() == str(g["inputs_sha256"]), "seeded inputs drifted from the ones the fixture was made from"
    return w, kwargs, stride, (q, k, v), g


def golden_out(g, tag, dtype):
    a = g[f"out_{tag}"]
    if dtype == torch.float32:
        return torch.from_numpy(a)
    return torch.from_numpy(a.view(np.int16)).view(dtype)


def golden_mask(g, tag, nb):
    return torch.from_numpy(np.unpackbits(g[f"mask_{tag}"], axis=-1)[..., :nb].astype(bool))


def assert_close_out(got, want, dtype, what=""):
    d = (got.float() - want.float()).abs()
    max_tol, mean_tol = TOL[dtype]
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite output"
    assert d.max().item() <= max_tol, f"{what}: max-abs {d.max().item():.3e} > {max_tol}"
    assert d.mean().item() <= mean_tol, f"{what}: mean-abs {d.mean().item():.3e} > {mean_tol}"


def classify_permutation(idx_got, idx_want, importance, segment_size, rel=2e-5):
    """Compare two per-segment permutations.

    Returns (n_diff, n_unexplained).  A differing slot is *explained* when the two
    keys placed there have importance within ``rel`` of each other (a tie or a
    near-tie that the order of fp32 additions decides); anything else is not.
    Also asserts each segment of ``idx_got`` is a permutation of that segment.
    """
    idx_got = idx_got.long()
    idx_want = idx_want.long()
    B, H, S = idx_want.shape
    L = importance.shape[-1]
    srt = torch.sort(idx_got[..., :L].reshape(B, H, -1, segment_size), dim=-1).values
    base = torch.arange(L).view(1, 1, -1, segment_size)
    assert torch.equal(srt, base.expand_as(srt)), "a segment is not a permutation of its own positions"
    assert torch.equal(idx_got[..., L:], idx_want[..., L:]), "tail positions moved"
    diff = idx_got != idx_want
    n_diff = int(diff.sum())
    if n_diff == 0:
        return 0, 0
    a = torch.gather(importance, 2, idx_got[..., :L])
    b = torch.gather(importance, 2, idx_want[..., :L])
    near = (a - b).abs() <= rel * torch.maximum(a.abs(), b.abs())
    unexplained = diff[..., :L] & ~near
    return n_diff, int(unexplained.sum())


def classify_mask(mask_got, mask_want, scores, threshold, blocks_per_segment, atol=2e-6, rel=1e-5):
    """Compare two final block masks row by row.

    Returns (rows_diff, rows_unexplained).  A differing row is *explained* when
      - tie: got and want select the same number of blocks and the symmetric
        difference consists of blocks whose score equals (within ``rel``) the
        score at the cut, or
      - boundary: the counts differ by one and the running sum at the cut is
        within ``atol`` of the threshold (the last bit of an fp32 sum decides).
    ``scores`` are the oracle's pooled softmax scores (NaN rows = no candidates).
    """
    B, H, nb, _ = mask_want.shape
    rows = (mask_got != mask_want).any(-1)
    n_rows = int(rows.sum())
    if n_rows == 0:
        return 0, 0
    bad = 0
    sc = torch.nan_to_num(scores, nan=0.0)
    thr = torch.as_tensor(threshold, dtype=torch.float32).reshape(-1)
    for b, h, qb in torch.nonzero(rows).tolist():
        t = float(thr[h] if thr.numel() > 1 else thr[0])
        g, w, s = mask_got[b, h, qb], mask_want[b, h, qb], sc[b, h, qb]
        sym = g ^ w
        vals, _ = torch.sort(s, descending=True)
        cum = torch.cumsum(vals.double(), 0)
        n_w = int((w & (s > 0)).sum())
        cut = vals[max(n_w - 1, 0)]
        tie = int(g.sum()) == int(w.sum()) and bool(((s[sym] - cut).abs() <= rel * cut.abs()).all())
        near = [abs(float(cum[i]) - t) <= atol for i in (max(n_w - 2, 0), max(n_w - 1, 0)) ]
        boundary = abs(int(g.sum()) - int(w.sum())) == 1 and any(near) and int(sym.sum()) == 1
        if not (tie or boundary):
            bad += 1
    return n_rows, bad


def classify_permutation_chain(idx_got, idx_want, imp_got, imp_want, segment_size, rel=2e-5):
    """Exact accounting of permutation differences for 16-bit inputs.

    ``imp_got`` is the importance the CUDA path sorted (its own fp32 output), ``imp_want`` the
    oracle's.  Two links are checked:
      1. ``idx_got`` is EXACTLY the stable descending per-segment sort of ``imp_got`` (the sort
         itself has no tolerance);
      2. where ``idx_got`` and ``idx_want`` differ, the keys whose importance differs between the
         two runs beyond ``rel`` (the keys hit by a one-step flip of a scoring logit: the GEMM
         summation order is not part of the reference's contract) are set aside per segment; the
         remaining keys must appear in the same relative order in both permutations, except
         neighbours whose oracle importance is within ``rel`` (fp32 near-ties).  A segment where
         that fails is *unexplained*.
    Returns a dict of counts.
    """
    idx_got, idx_want = idx_got.long(), idx_want.long()
    B, H, S = idx_want.shape
    L = imp_want.shape[-1]
    nseg = L // segment_size
    own = torch.argsort(imp_got.view(B, H, nseg, segment_size), dim=-1, descending=True, stable=True)
    own = (own + torch.arange(0, L, segment_size).view(1, 1, nseg, 1)).reshape(B, H, L)
    sort_exact = bool(torch.equal(own, idx_got[..., :L])) and bool(torch.equal(idx_got[..., L:], idx_want[..., L:]))
    diff = idx_got[..., :L] != idx_want[..., :L]
    n_diff = int(diff.sum())
    seg_diff = diff.view(B, H, nseg, segment_size).any(-1)
    moved = (imp_got - imp_want).abs() > rel * torch.maximum(imp_got.abs(), imp_want.abs())
    n_unexplained = 0
    n_affected = 0
    for b, h, s in torch.nonzero(seg_diff).tolist():
        lo = s * segment_size
        g = idx_got[b, h, lo:lo + segment_size]
        w = idx_want[b, h, lo:lo + segment_size]
        hit = moved[b, h]
        n_affected += int(hit[lo:lo + segment_size].sum())
        g2, w2 = g[~hit[g]], w[~hit[w]]
        bad = g2 != w2
        if bool(bad.any()):
            a, c = imp_want[b, h][g2[bad]], imp_want[b, h][w2[bad]]
            if not bool(((a - c).abs() <= rel * torch.maximum(a.abs(), c.abs())).all()):
                n_unexplained += 1
    return {"idx_sort_exact": sort_exact, "idx_diff_slots": n_diff, "idx_slots": int(idx_want.numel()),
            "idx_diff_segments": int(seg_diff.sum()), "idx_keys_with_moved_importance": n_affected,
            "idx_unexplained_segments": n_unexplained}


def attended_key_signature(idx, mask, block_size):
    """(B, H, nb) int64: an order-independent signature of the SET of keys each q block attends (sum
    over its selected kv blocks of a per-block hash of the original positions the block holds).
    Equal signatures of two runs mean the two q blocks attend the same keys even when permutation
    or mask differ in ways that cancel (e.g. two keys swapped between two selected blocks)."""
    B, H, S = idx.shape
    nb = mask.shape[-1]
    pad = nb * block_size - S
    x = idx.long()
    if pad:
        x = torch.cat([x, torch.full((B, H, pad), -1, dtype=torch.long)], dim=-1)
    hsh = ((x + 7) * 2654435761 % 2147483647) * (x >= 0)
    per_block = hsh.view(B, H, nb, block_size).sum(-1)                    # (B, H, nb)
    return (mask.long() * per_block[:, :, None, :]).sum(-1)


def parity_report(request, **fields):
    """One machine-readable line per parity case: printed, attached to the junit record, and appended
    to the file named by PBS_PARITY_REPORT when that is set."""
    import json
    rec = {"test": request.node.name}
    rec.update(fields)
    line = json.dumps(rec, sort_keys=True)
    print("PARITY " + line)
    for k, v in fields.items():
        request.node.user_properties.append((k, v))
    path = os.environ.get("PBS_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(line + "\n")
