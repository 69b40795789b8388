"""Seeded synthetic inputs for the benchmark configurations, and their FLOP / byte counts.

The reference benchmarks with downloaded GPT-2 weights and one English prompt
(src/py/model_inference.py:403-410, 428); neither is available offline, so every workload here is
synthetic: values i.i.d. N(0, 1) from a fixed seed, shapes as the configuration states.  The
generator call order is fixed (q, then k, then v, on the CPU generator) so that the parity tests
and the CPU baseline see identical values.  The benchmark's timed tensors are drawn on the device
(bench.device_inputs: same shapes, distribution and seed, a CUDA generator) -- at 400 MB and more
per configuration a host-side draw plus upload would dominate the run; nothing is compared
element by element across the two.
"""
from __future__ import annotations

import dataclasses

import torch

HEAD_DIM = 64


@dataclasses.dataclass(frozen=True)
class AttnWorkload:
    name: str
    B: int
    H: int
    N: int
    seed: int
    causal: bool = True
    stress_k_rows: bool = False   # multiply a random 1% of K rows by 4 (long-context stress case)

    @property
    def d(self) -> int:
        return HEAD_DIM

    def flops(self) -> float:
        """Causal-adjusted FLOPs: 2*B*H*N^2*d when causal (half of the dense 4*B*H*N^2*d)."""
        dense = 4.0 * self.B * self.H * self.N * self.N * self.d
        return dense / 2 if self.causal else dense

    def bytes(self, with_lse: bool = False) -> float:
        """Algorithmic HBM bytes: Q, K, V read once and O written once in bf16 (+ LSE fp32)."""
        n = 4.0 * self.B * self.H * self.N * self.d * 2
        return n + (4.0 * self.B * self.H * self.N if with_lse else 0.0)

    def make_cpu(self, heads: slice | None = None):
        """fp32 CPU tensors q, k, v of shape [B, H, N, d] (or the flattened-head slice
        [n, 1, N, d] when `heads` selects a range of the B*H heads)."""
        g = torch.Generator().manual_seed(self.seed)
        shape = (self.B, self.H, self.N, self.d)
        q = torch.randn(shape, generator=g)
        k = torch.randn(shape, generator=g)
        v = torch.randn(shape, generator=g)
        if self.stress_k_rows:
            n_rows = max(1, self.N // 100)
            idx = torch.randperm(self.N, generator=g)[:n_rows]
            k[:, :, idx, :] *= 4.0
        if heads is not None:
            q, k, v = (t.reshape(self.B * self.H, 1, self.N, self.d)[heads] for t in (q, k, v))
        return q, k, v


def config1() -> AttnWorkload:
    """GPT-2 small shape, single causal forward: B=4, H=12, N=1024, seed 0."""
    return AttnWorkload("gpt2-small-attn", 4, 12, 1024, seed=0)


def config3(N: int, causal: bool = True) -> AttnWorkload:
    """GPT-2 medium attention-only sweep: B=16, H=16, N in {512, 1024, 2048, 4096}, seed 2."""
    return AttnWorkload(f"gpt2-medium-attn-N{N}", 16, 16, N, seed=2, causal=causal)


def config4_attention(batch: int = 32) -> AttnWorkload:
    """The attention problem of one GPT-2 XL layer at prefill: B=32 per GPU, H=25, N=1024."""
    return AttnWorkload("gpt2-xl-layer-attn", batch, 25, 1024, seed=3)


def config5(N: int) -> AttnWorkload:
    """Long-context stress: B=4, H=25, N in {8192, 16384, 32768}, 1% of K rows scaled x4, seed 4."""
    return AttnWorkload(f"long-context-N{N}", 4, 25, N, seed=4, stress_k_rows=True)


def shard_heads(total: int, world: int, rank: int) -> slice:
    """Contiguous slice of `total` independent (batch, head) problems owned by `rank`; the first
    `total % world` ranks get one extra.  No head is split and none is shared, so the path needs
    no collective."""
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))
