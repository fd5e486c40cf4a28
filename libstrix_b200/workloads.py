"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (used by bench.py, the smoke check and the tests).

Everything is generated on the CPU from a torch.Generator so the CPU oracle and
the GPU path see identical bits; callers move tensors to the device.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class DecodeBatch:
    """Paged int8 KV cache plus one bf16 query per sequence."""

    q: torch.Tensor            # bf16 [B, Hq, D]
    key_cache: torch.Tensor    # int8 [blocks, bs, Hkv, D]
    value_cache: torch.Tensor  # int8 [blocks, bs, Hkv, D]
    k_scale: torch.Tensor      # fp32 [blocks, bs, Hkv]
    v_scale: torch.Tensor      # fp32 [blocks, bs, Hkv]
    seq_lens: torch.Tensor     # int32 [B]
    block_table: torch.Tensor  # int32 [B, max_blocks]
    scale: float

    def to(self, device) -> "DecodeBatch":
        return DecodeBatch(*[
            v.to(device) if isinstance(v, torch.Tensor) else v for v in self.__dict__.values()
        ])

    @property
    def kv_bytes(self) -> int:
        """Algorithmic bytes one decode step must read: every live key's K and V
        rows and their two fp32 scales, for every KV head."""
        hkv, d = self.key_cache.size(2), self.q.size(-1)
        return int(self.seq_lens.sum().item()) * hkv * (2 * d + 8)


def decode_batch(
    batch: int = 64,
    hq: int = 32,
    hkv: int = 4,
    head_dim: int = 128,
    block_size: int = 16,
    ctx_lo: int = 1024,
    ctx_hi: int = 65536,
    seed: int = 0,
    ctx_lens: list[int] | None = None,
    spare_blocks: int = 3,
    device: str | torch.device = "cpu",
) -> DecodeBatch:
    """Decode attention batch: context lengths ~ U[ctx_lo, ctx_hi] per sequence
    (or `ctx_lens`), block tables a random permutation of the physical blocks,
    K/V int8 = clip(round(N(0,1) * 32), +-127), per-token-per-head fp32 scales
    ~ U(0.01, 0.05), q bf16 ~ N(0,1), softmax scale head_dim ** -0.5.

    `device` is where the tensors are generated (and left); the same seed gives
    different bits on different devices, so parity checks copy what they need
    to the CPU rather than regenerating it."""
    gen = torch.Generator(device=device).manual_seed(seed)
    lgen = torch.Generator().manual_seed(seed)
    if ctx_lens is None:
        lens = torch.randint(ctx_lo, ctx_hi + 1, (batch,), generator=lgen, dtype=torch.int64)
    else:
        lens = torch.tensor(ctx_lens, dtype=torch.int64)
        batch = lens.numel()
    nblk = (lens + block_size - 1) // block_size
    total = int(nblk.sum()) + spare_blocks
    shape = (total, block_size, hkv, head_dim)

    def int8_normal():
        out = torch.empty(shape, dtype=torch.int8, device=device)
        flat = out.view(-1)
        step = 1 << 26  # bounded temporaries for multi-GB caches
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            x = torch.randn(n, generator=gen, device=device).mul_(32).round_().clamp_(-127, 127)
            flat[i:i + n] = x.to(torch.int8)
        return out

    key_cache, value_cache = int8_normal(), int8_normal()
    k_scale = torch.rand(shape[:3], generator=gen, device=device) * 0.04 + 0.01
    v_scale = torch.rand(shape[:3], generator=gen, device=device) * 0.04 + 0.01
    perm = torch.randperm(total, generator=lgen).to(torch.int32)
    table = torch.zeros(batch, max(int(nblk.max()), 1), dtype=torch.int32)
    used = 0
    for i, nb in enumerate(nblk.tolist()):
        table[i, :nb] = perm[used:used + nb]
        used += nb
    q = torch.randn(batch, hq, head_dim, generator=gen, device=device).bfloat16()
    return DecodeBatch(q, key_cache, value_cache, k_scale, v_scale,
                       lens.to(torch.int32).to(device), table.to(device), head_dim ** -0.5)
