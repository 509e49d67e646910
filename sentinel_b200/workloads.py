"""The five attention workloads the benchmark and the parity tests are quoted on, with their seeded inputs.

Inputs are fully synthetic (no dataset is involved on this path).  One CPU ``torch.Generator`` seeded with
``20261125 + index`` draws Q, K, V, dO in that order as fp32 ``[B, H, S, D]`` (token-major); the bf16
workloads are then rounded to bf16.  Rotary position embedding, where a workload asks for it, follows the
reference's convention: interleaved pairs ``(2i, 2i+1)``, angle ``pos * base**(-2i/D)``, positions
restarting at 0 for every sequence (sentinel/NeuralNet/Layers/RotaryEmbedding.cpp:19-27, :38-59).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    index: int
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    seq: int
    head_dim: int
    dtype: str            # "f32" | "bf16"
    qk_std: float
    v_std: float
    do_std: float
    rope_base: float | None = None
    seq_shards: int = 1   # > 1: sequence-sharded ring workload

    @property
    def scale(self) -> float:
        return self.head_dim ** -0.5   # sentinel/NeuralNet/Layers/CausalSelfAttention.cpp:224

    @property
    def flops(self) -> float:
        """Causal-adjusted forward+backward work: 7 GEMMs of 2*S^2*D per head, halved by the mask."""
        return 7.0 * self.batch * self.q_heads * float(self.seq) ** 2 * self.head_dim

    @property
    def algorithmic_bytes(self) -> float:
        """Read Q,K,V,O,dO,LSE and write O,LSE,dQ,dK,dV once each (2-byte elements, fp32 LSE)."""
        nq = self.batch * self.q_heads * self.seq * self.head_dim
        nkv = self.batch * self.kv_heads * self.seq * self.head_dim
        esz = 4 if self.dtype == "f32" else 2
        return esz * (6 * nq + 6 * nkv) + 12.0 * self.batch * self.q_heads * self.seq

    @property
    def kv_groups(self) -> int:
        """Independent units (batch element x KV head) a multi-GPU run shards without communication."""
        return self.batch * self.kv_heads


WORKLOADS = {
    "toy_f32": Workload(0, "toy_f32", 4, 4, 4, 64, 16, "f32", 1.0, 1.0, 1.0),
    "gpt2_small": Workload(1, "gpt2_small", 8, 12, 12, 1024, 64, "bf16", 0.5, 0.5, 1e-2),
    "llama1b_gqa": Workload(2, "llama1b_gqa", 4, 32, 8, 4096, 64, "bf16", 0.5, 1.0, 1e-2, rope_base=1e4),
    "gqa7b_d128": Workload(3, "gqa7b_d128", 2, 28, 4, 8192, 128, "bf16", 0.5, 1.0, 1e-2, rope_base=1e6),
    "longctx_ring": Workload(4, "longctx_ring", 1, 32, 8, 131072, 128, "bf16", 0.5, 0.5, 1e-2, seq_shards=8),
}


def apply_rope_(x: torch.Tensor, base: float) -> torch.Tensor:
    """In-place interleaved-pair rotation of ``x`` [B, H, S, D] (fp32)."""
    B, H, S, D = x.shape
    pair = torch.arange(D // 2, dtype=torch.float32)
    inv = torch.pow(torch.tensor(float(base), dtype=torch.float32), -2.0 * pair / D)
    ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)
    even, odd = x[..., 0::2].clone(), x[..., 1::2].clone()
    x[..., 0::2] = even * cos - odd * sin
    x[..., 1::2] = even * sin + odd * cos
    return x


def make_inputs(w: Workload, *, batch: int | None = None, q_heads: int | None = None, kv_heads: int | None = None,
                seq: int | None = None, seed_offset: int = 0):
    """Seeded (Q, K, V, dO) for workload ``w`` as CPU tensors in the workload's dtype.

    The keyword overrides let a test or a shard draw a smaller instance with the same distributions."""
    B = batch or w.batch
    Hq = q_heads or w.q_heads
    Hkv = kv_heads or w.kv_heads
    S = seq or w.seq
    D = w.head_dim
    g = torch.Generator(device="cpu").manual_seed(20261125 + w.index + 1000 * seed_offset)
    q = torch.randn(B, Hq, S, D, generator=g, dtype=torch.float32) * w.qk_std
    k = torch.randn(B, Hkv, S, D, generator=g, dtype=torch.float32) * w.qk_std
    v = torch.randn(B, Hkv, S, D, generator=g, dtype=torch.float32) * w.v_std
    do = torch.randn(B, Hq, S, D, generator=g, dtype=torch.float32) * w.do_std
    if w.rope_base is not None:
        apply_rope_(q, w.rope_base)
        apply_rope_(k, w.rope_base)
    if w.dtype == "bf16":
        q, k, v, do = (t.to(torch.bfloat16) for t in (q, k, v, do))
    return q, k, v, do


def shard_units(batch: int, kv_heads: int, rank: int, world: int):
    """The (batch element, KV head) units rank ``rank`` of ``world`` owns: a contiguous, balanced slice of the
    ``batch * kv_heads`` independent units.  A KV group is never split (that would need a dK/dV reduction)."""
    units = [(b, hk) for b in range(batch) for hk in range(kv_heads)]
    per, extra = divmod(len(units), world)
    start = rank * per + min(rank, extra)
    return units[start:start + per + (1 if rank < extra else 0)]
