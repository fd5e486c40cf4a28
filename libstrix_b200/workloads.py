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


@dataclass
class MoeFp8Layer:
    """One MoE layer in the FP8 W8A8 block-scaled form (benchmark config 1)."""

    x: torch.Tensor          # bf16 [T, H]
    logits: torch.Tensor     # fp32 [T, E]
    w13: torch.Tensor        # e4m3 [E, 2I, H]   rows [gate; up]
    w13_scale: torch.Tensor  # fp32 [E, 2I/128, H/128]
    w2: torch.Tensor         # e4m3 [E, H, I]
    w2_scale: torch.Tensor   # fp32 [E, H/128, I/128]
    top_k: int

    def to(self, device) -> "MoeFp8Layer":
        return MoeFp8Layer(*[
            v.to(device) if isinstance(v, torch.Tensor) else v for v in self.__dict__.values()
        ])

    @property
    def flops(self) -> int:
        t, h = self.x.shape
        n13 = self.w13.size(1)
        return 2 * t * self.top_k * (n13 * h + h * (n13 // 2))

    @property
    def weight_bytes(self) -> int:
        return self.w13.numel() + self.w2.numel() + 4 * (self.w13_scale.numel() + self.w2_scale.numel())


def quantize_fp8_block(w: torch.Tensor):
    """fp32 [E, N, K] -> (e4m3, fp32 scales [E, N/128, K/128]) with s = amax / 448 per block."""
    e, n, k = w.shape
    blocks = w.view(e, n // 128, 128, k // 128, 128)
    s = blocks.abs().amax(dim=(2, 4)).clamp_min(1e-12) / 448.0
    q = (blocks / s[:, :, None, :, None]).reshape(e, n, k).to(torch.float8_e4m3fn)
    return q, s.contiguous()


def moe_fp8_layer(tokens=256, hidden=2048, experts=128, top_k=8, inter=768, seed=0,
                  device="cpu", zipf_bias: float | None = None) -> MoeFp8Layer:
    """Activations bf16 ~ N(0,1); router logits fp32 ~ N(0,1) (plus a Zipf(1.1)
    per-expert log-bias when `zipf_bias` is given); weights ~ N(0, 0.02)
    quantised to e4m3 with fp32 128x128 block scales."""
    gen = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(tokens, hidden, generator=gen, device=device).bfloat16()
    logits = torch.randn(tokens, experts, generator=gen, device=device)
    if zipf_bias is not None:
        ranks = torch.arange(1, experts + 1, device=device, dtype=torch.float32)
        bias = torch.log(ranks.pow(-zipf_bias) / ranks.pow(-zipf_bias).sum())
        perm = torch.randperm(experts, generator=torch.Generator().manual_seed(seed)).to(device)
        logits = logits + bias[perm]

    def weights(n, k):
        q = torch.empty(experts, n, k, dtype=torch.float8_e4m3fn, device=device)
        s = torch.empty(experts, n // 128, k // 128, dtype=torch.float32, device=device)
        for e0 in range(0, experts, 16):  # bounded fp32 temporaries
            w = torch.randn(min(16, experts - e0), n, k, generator=gen, device=device) * 0.02
            q[e0:e0 + 16], s[e0:e0 + 16] = quantize_fp8_block(w)
        return q, s

    w13, s13 = weights(2 * inter, hidden)
    w2, s2 = weights(hidden, inter)
    return MoeFp8Layer(x, logits, w13, s13, w2, s2, top_k)


# ------------------------------------------------------------------ MXFP4 (config 5)
def quantize_mxfp4(w: torch.Tensor):
    """fp32 [..., K] (K % 32 == 0) -> (uint8 [..., K/2], uint8 e8m0 scales [..., K/32]).

    Per 32 elements the scale is the power of two 2^ceil(log2(amax / 6)) (byte =
    exponent + 127; an all-zero group takes byte 0, the zero block), the elements
    are x / scale rounded to nearest-even onto the e2m1 grid {0, .5, 1, 1.5, 2, 3,
    4, 6} with a sign bit, and byte j holds element 2j in its low nibble - the
    layout csrc/gemm/mxfp4_wmma_gemm.hip:14-23,38-57 of the reference decodes."""
    k = w.size(-1)
    g = w.float().reshape(*w.shape[:-1], k // 32, 32)
    amax = g.abs().amax(-1)
    m, ex = torch.frexp(amax / 6.0)                 # amax / 6 = m * 2^ex, m in [0.5, 1)
    e = torch.where(m > 0.5, ex, ex - 1)            # ceil(log2(.))
    byte = torch.where(amax > 0, (e + 127).clamp(1, 254), torch.zeros_like(e))
    scale = torch.ldexp(torch.ones_like(amax), byte - 127)
    x = (g / scale[..., None]).abs()
    # thresholds are the midpoints of the grid; a tie goes to the even mantissa
    code = ((x > 0.25).to(torch.uint8) + (x >= 0.75) + (x > 1.25) + (x >= 1.75) + (x > 2.5)
            + (x >= 3.5) + (x > 5.0)).to(torch.uint8)
    code = code | ((g < 0).to(torch.uint8) << 3)
    code = torch.where((byte == 0)[..., None], torch.zeros_like(code), code).reshape(*w.shape[:-1], k)
    packed = code[..., 0::2] | (code[..., 1::2] << 4)
    return packed.contiguous(), byte.to(torch.uint8).contiguous()


def zipf_bias(experts: int, alpha: float = 1.1, seed: int = 7, device="cpu") -> torch.Tensor:
    """log of Zipf(alpha) weights over the experts, randomly permuted: the
    per-expert router bias that skews the load of config 5."""
    ranks = torch.arange(1, experts + 1, dtype=torch.float32)
    wts = ranks.pow(-alpha)
    bias = torch.log(wts / wts.sum())
    perm = torch.randperm(experts, generator=torch.Generator().manual_seed(seed))
    return bias[perm].to(device)


@dataclass
class MoeMxfp4Layer:
    """One MXFP4 MoE layer (benchmark config 5), or a rank's expert shard of it."""

    x: torch.Tensor          # bf16 [T, H]
    logits: torch.Tensor     # fp32 [T, E_global]
    w13: torch.Tensor        # uint8 [E, 2I, H/2]   rows [gate; up], e2m1 nibbles
    w13_scale: torch.Tensor  # uint8 [E, 2I, H/32]  e8m0
    w2: torch.Tensor         # uint8 [E, H, I/2]
    w2_scale: torch.Tensor   # uint8 [E, H, I/32]
    top_k: int

    def to(self, device) -> "MoeMxfp4Layer":
        return MoeMxfp4Layer(*[
            v.to(device) if isinstance(v, torch.Tensor) else v for v in self.__dict__.values()
        ])

    @property
    def flops(self) -> int:
        t, h = self.x.shape
        n13 = self.w13_scale.size(1)
        return 2 * t * self.top_k * (n13 * h + h * (n13 // 2))


def moe_mxfp4_layer(tokens=8192, hidden=2880, experts=128, top_k=4, inter=2880, seed=0,
                    device="cpu", expert_lo=0, expert_hi=None, token_lo=0, token_hi=None,
                    zipf_alpha: float | None = 1.1, expert_list=None) -> MoeMxfp4Layer:
    """Config 5: x bf16 ~ N(0,1); router logits N(0,1) plus a Zipf(1.1) per-expert
    bias; weights N(0, 0.02) quantised to MXFP4 (quantize_mxfp4). Every expert
    and every token block has its own generator seed, so a rank can build only
    its experts [expert_lo, expert_hi) and tokens [token_lo, token_hi) and still
    hold exactly the slices of the one global layer (token blocks of 256).
    `expert_list` names the global experts to build instead of a range (a rank of a
    round-robin placement holds rank, rank + N, ...)."""
    expert_hi = experts if expert_hi is None else expert_hi
    token_hi = tokens if token_hi is None else token_hi
    assert token_lo % 256 == 0 and (token_hi % 256 == 0 or token_hi == tokens)
    xs, ls = [], []
    bias = zipf_bias(experts, zipf_alpha, device=device) if zipf_alpha is not None else 0.0
    for t0 in range(token_lo, token_hi, 256):
        g = torch.Generator(device=device).manual_seed(seed * 1_000_003 + 17 + t0)
        n = min(256, tokens - t0)
        xs.append(torch.randn(n, hidden, generator=g, device=device).bfloat16())
        ls.append(torch.randn(n, experts, generator=g, device=device) + bias)
    which = list(range(expert_lo, expert_hi)) if expert_list is None else list(expert_list)
    e_n = len(which)
    w13 = torch.empty(e_n, 2 * inter, hidden // 2, dtype=torch.uint8, device=device)
    s13 = torch.empty(e_n, 2 * inter, hidden // 32, dtype=torch.uint8, device=device)
    w2 = torch.empty(e_n, hidden, inter // 2, dtype=torch.uint8, device=device)
    s2 = torch.empty(e_n, hidden, inter // 32, dtype=torch.uint8, device=device)
    for i, e in enumerate(which):
        g = torch.Generator(device=device).manual_seed(seed * 1_000_003 + 1_000 + e)
        w13[i], s13[i] = quantize_mxfp4(torch.randn(2 * inter, hidden, generator=g, device=device) * 0.02)
        w2[i], s2[i] = quantize_mxfp4(torch.randn(hidden, inter, generator=g, device=device) * 0.02)
    return MoeMxfp4Layer(torch.cat(xs), torch.cat(ls), w13, s13, w2, s2, top_k)
