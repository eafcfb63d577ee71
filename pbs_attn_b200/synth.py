"""Seeded synthetic prefill inputs: Q/K/V with planted heavy-hitter keys and RoPE.

They stand in for the LongBench-v2 contexts the reference's efficiency script
feeds its model (eval/efficiency/eval_efficiency.py:174-175,223-231); no dataset
or checkpoint is read.  Q, K, V are N(0,1); a shared unit direction ``u`` is added
to every query, ``+3u`` to a random fraction ``density`` of the key positions and
``+5u`` to ``sinks`` leading positions; rotary embedding in the rotate-half form
(pbs_attn/patch/huggingface.py:14-26) is applied to Q and K; then everything is
cast to ``dtype``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    head_dim: int
    seq_len: int
    dtype: str            # "bf16" | "fp16" | "fp32"
    block_size: int
    segment_size: int
    threshold: float
    rope_theta: float
    density: float = 0.02
    sinks: int = 0

    @property
    def torch_dtype(self) -> torch.dtype:
        return {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[self.dtype]

    def with_(self, **kw) -> "Workload":
        return replace(self, **kw)


# The benchmark configurations of the task description (attention-op level).
OP_CHECK = Workload("op_check_s2048", 1, 4, 1, 64, 2048, "fp32", 64, 256, 0.9, 1e4)
LLAMA8B_32K = Workload("llama8b_heads_s32768", 1, 32, 8, 128, 32768, "bf16", 128, 256, 0.9, 5e5, sinks=4)
LLAMA8B_128K = Workload("llama8b_heads_s131072", 1, 32, 8, 128, 131072, "bf16", 128, 256, 0.9, 5e5, sinks=4)
QWEN7B_32K = Workload("qwen7b_heads_s32768", 1, 28, 4, 128, 32768, "bf16", 128, 256, 0.9, 1e6)

WORKLOADS = {w.name: w for w in (OP_CHECK, LLAMA8B_32K, LLAMA8B_128K, QWEN7B_32K)}


def rope_tables(seq_len: int, head_dim: int, theta: float, device, generator=None):
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.arange(seq_len, dtype=torch.float32, device=device)[:, None] * inv_freq[None, :]
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def apply_rope_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x (B, H, S, D) fp32, rotated head by head to bound the temporaries."""
    for h in range(x.shape[1]):
        xh = x[:, h]
        x[:, h] = xh * cos + _rotate_half(xh) * sin
    return x


def make_qkv(w: Workload, seed: int = 0, device="cpu", kv_heads: int | None = None, q_heads: int | None = None):
    """Returns q (B,Hq,S,D), k, v (B,Hkv,S,D) in ``w.dtype`` on ``device``.

    All random draws come from one ``torch.Generator`` on ``device`` seeded with
    ``seed``; CPU draws are what the committed golden fixtures were made from.
    ``q_heads`` / ``kv_heads`` override the head counts (a head-sharded rank
    generates only its own heads; pass distinct seeds per shard).
    """
    Hq = q_heads or w.q_heads
    Hkv = kv_heads or w.kv_heads
    B, S, D = w.batch, w.seq_len, w.head_dim
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(B, Hq, S, D, generator=g, device=device)
    k = torch.randn(B, Hkv, S, D, generator=g, device=device)
    v = torch.randn(B, Hkv, S, D, generator=g, device=device)
    u = torch.randn(D, generator=g, device=device)
    u = u / u.norm()
    n_hot = int(round(w.density * S))
    pos = torch.randperm(S, generator=g, device=device)[:n_hot]
    k[:, :, pos] += 3.0 * u
    q += u
    if w.sinks:
        k[:, :, : w.sinks] += 5.0 * u
    cos, sin = rope_tables(S, D, w.rope_theta, device)
    apply_rope_(q, cos, sin)
    apply_rope_(k, cos, sin)
    dt = w.torch_dtype
    return q.to(dt), k.to(dt), v.to(dt)


def make_qkv_heads(w: Workload, seed: int, kv_start: int, kv_count: int, q_start: int | None = None,
                   q_count: int | None = None, device="cpu"):
    """The same kind of inputs as ``make_qkv``, drawn PER KV-HEAD GROUP so that a rank of a
    head-sharded run generates exactly the heads it owns and every partition of the heads (1, 2, 4
    or 8 ranks; query heads split inside a group) works on the same global problem.

    Group j (KV head j with its query heads) comes from a generator seeded with (seed, j); the
    shared direction ``u`` and the planted key positions come from a generator seeded with ``seed``.
    Returns q (B, q_count, S, D) for the query heads [q_start, q_start + q_count) (default: all query
    heads of the KV heads asked for) and k, v (B, kv_count, S, D).
    """
    B, S, D = w.batch, w.seq_len, w.head_dim
    group = w.q_heads // w.kv_heads
    if q_start is None:
        q_start, q_count = kv_start * group, kv_count * group
    g0 = torch.Generator(device=device).manual_seed(seed)
    u = torch.randn(D, generator=g0, device=device)
    u = u / u.norm()
    pos = torch.randperm(S, generator=g0, device=device)[: int(round(w.density * S))]
    cos, sin = rope_tables(S, D, w.rope_theta, device)
    dt = w.torch_dtype
    qs, ks, vs = [], [], []
    for j in range(kv_start, kv_start + kv_count):
        g = torch.Generator(device=device).manual_seed(seed * 1000003 + 7919 * (j + 1))
        q = torch.randn(B, group, S, D, generator=g, device=device)
        k = torch.randn(B, 1, S, D, generator=g, device=device)
        v = torch.randn(B, 1, S, D, generator=g, device=device)
        k[:, :, pos] += 3.0 * u
        q += u
        if w.sinks:
            k[:, :, : w.sinks] += 5.0 * u
        apply_rope_(q, cos, sin)
        apply_rope_(k, cos, sin)
        lo = max(q_start, j * group) - j * group
        hi = min(q_start + q_count, (j + 1) * group) - j * group
        if hi > lo:
            qs.append(q[:, lo:hi].to(dt))
        ks.append(k.to(dt))
        vs.append(v.to(dt))
    return torch.cat(qs, dim=1), torch.cat(ks, dim=1), torch.cat(vs, dim=1)
