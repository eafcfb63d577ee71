"""The in-place rotary-embedding kernel against the tensor operations it replaces
(pbs_attn/patch/huggingface.py:14-26 of the reference): bit-exact for every dtype."""
import pytest
import torch

from pbs_attn.patch.huggingface import apply_rotary_pos_emb

pytestmark = pytest.mark.gpu


def _tables(B, S, D, dtype, theta=10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D))
    pos = torch.arange(S, device="cuda", dtype=torch.float32) + 3.0 * torch.arange(B, device="cuda", dtype=torch.float32)[:, None]
    ang = pos[..., None] * inv                                     # (B, S, D/2)
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,H,Hkv,S,D,bcast", [(2, 3, 1, 77, 128, False), (1, 8, 2, 1000, 64, True), (2, 2, 2, 33, 128, True)])
def test_rope_kernel_is_bit_exact(dtype, B, H, Hkv, S, D, bcast):
    from pbs_attn_b200.prefill import apply_rope_
    torch.manual_seed(0)
    # the layout the attention layer produces: (B, S, H*D) projections viewed as (B, H, S, D)
    q = torch.randn(B, S, H * D, device="cuda").to(dtype).view(B, S, H, D).transpose(1, 2)
    k = torch.randn(B, S, Hkv * D, device="cuda").to(dtype).view(B, S, Hkv, D).transpose(1, 2)
    cos, sin = _tables(B, S, D, dtype)
    if bcast:
        cos, sin = cos[:1], sin[:1]
    want_q, want_k = apply_rotary_pos_emb(q, k, cos, sin)
    got_q, got_k = apply_rope_(q.clone(memory_format=torch.preserve_format), cos, sin), apply_rope_(k.clone(memory_format=torch.preserve_format), cos, sin)
    assert got_q.stride() == q.stride()
    assert torch.equal(got_q, want_q) and torch.equal(got_k, want_k)


@pytest.mark.parametrize("name", ["rope_bf16", "rope_fp16", "rope_fp32"])
def test_rope_kernel_equals_the_reference_fixture(name):
    """Against outputs of the reference's own apply_rotary_pos_emb (tests/golden/rope.npz, made by
    tests/golden/make_golden.py from the unmodified reference): bit-exact."""
    import hashlib
    import os
    import numpy as np
    from cases import ROPE_CASES, rope_inputs
    from pbs_attn_b200.prefill import apply_rope_
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rope.npz"))
    q, k, cos, sin = rope_inputs(ROPE_CASES[name])
    h = hashlib.sha256()
    for t in (q, k, cos, sin):
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    assert h.hexdigest() == str(g[f"{name}_sha"]), "seeded inputs drifted from the ones the fixture was made from"
    for x, want in ((q, g[f"{name}_q"]), (k, g[f"{name}_k"])):
        got = apply_rope_(x.cuda().clone(memory_format=torch.preserve_format), cos.cuda(), sin.cuda()).cpu().contiguous()
        raw = got.view(torch.int16).numpy().view(np.uint16) if got.dtype != torch.float32 else got.numpy()
        assert np.array_equal(raw, want)


def test_rope_rejects_bad_tables():
    from pbs_attn_b200.prefill import apply_rope_
    x = torch.zeros(1, 2, 16, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        apply_rope_(x, torch.zeros(1, 16, 32, device="cuda", dtype=torch.bfloat16), torch.zeros(1, 16, 32, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        apply_rope_(x, torch.zeros(1, 16, 64, device="cuda"), torch.zeros(1, 16, 64, device="cuda"))
