"""libstrix_b200: sm_100a (B200) kernels behind libstrix's op surface.

Usable as a drop-in for the reference's `strix` package on its quantized
inference path (`import libstrix_b200 as strix`): the same `select / explain /
geometries / kernels / ops / selections / Range` table API
(python/strix/registry.py of the reference), the same wrappers (`attn_decode`,
python/strix/__init__.py:343-381) and the same `torch.ops.strix.*` schemas.

Importing loads libstrix_b200.so (the C-ABI of include/strix_b200.h) and fails
if it has not been built; nothing here computes on the CPU.
"""

from __future__ import annotations

import torch

from . import _lib
from .registry import Range, explain, geometries, kernels, ops, select, selections

_lib.load()
from . import torch_ops  # noqa: E402  (registers torch.ops.strix.*)
from . import moe  # noqa: E402

StrixError = _lib.StrixError


def is_supported_device() -> bool:
    """True on a CUDA device of compute capability 10.x (B200). The reference
    gates on HIP + gfx1151 instead (python/strix/__init__.py:510-513)."""
    if not torch.cuda.is_available() or torch.version.cuda is None:
        return False
    return torch.cuda.get_device_capability(0)[0] == 10


def attn_decode(
    out: torch.Tensor,
    q: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    seq_lens: torch.Tensor,
    block_table: torch.Tensor,
    scale: float,
    num_splits: int = 1,
    window_left: int = -1,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    sinks: torch.Tensor | None = None,
) -> torch.Tensor:
    """Paged attention for one query token per sequence (decode), split-KV.

    q, out: [N, Hq, D] bf16; caches: [blocks, block_size, Hkv, D] views; the
    query is position seq_lens[n] - 1. The caches are int8 with k_scale /
    v_scale ([blocks, block_size, Hkv] fp32) as dequant scales, one per (key,
    head). sinks: optional fp32 [Hq] attention-sink logits. num_splits in
    1..64 divides each sequence's keys as the reference does; num_splits = 0
    uses fixed 1024-key segments, which balances ragged batches. No host sync.
    """
    torch.ops.strix.attn_decode_bf16(
        out, q, key_cache, value_cache, seq_lens.to(torch.int32),
        block_table.to(torch.int32), scale, num_splits, window_left, k_scale, v_scale, sinks,
    )
    return out


def attn_prefill(
    out: torch.Tensor,
    q: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    seq_lens: torch.Tensor,
    block_table: torch.Tensor,
    scale: float,
    num_splits: int = 1,
    window_left: int = -1,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    sinks: torch.Tensor | None = None,
) -> torch.Tensor:
    """Causal paged attention for prefill (no host sync); same arguments as the
    reference's strix.attn_prefill (python/strix/__init__.py:214-268).

    q, out: [T, Hq, D] bf16, D = 64, 128, 256 or 512; caches [blocks, block_size, Hkv, D]
    views, bf16 or int8 with k_scale / v_scale fp32 [blocks, block_size, Hkv];
    the queries of sequence n are the last q_len of its seq_lens[n] positions.
    window_left >= 0: the query at position p sees keys p - window_left .. p.
    sinks: optional fp32 [Hq]; num_splits must be 1 then. num_splits is a hint
    the kernel does not need."""
    cu = cu_seqlens_q.to(torch.int32)
    torch.ops.strix.attn_prefill_bf16(
        out, q, key_cache, value_cache, k_scale, v_scale, cu, seq_lens.to(torch.int32),
        block_table.to(torch.int32), cu, 0, scale, num_splits, window_left, sinks,
    )
    return out


def kv_write_int8(key, value, key_cache, value_cache, k_scale, v_scale, slot_mapping,
                  rule: str = "reference") -> None:
    """Quantises new K/V rows ([tokens, Hkv, D] bf16/fp16) per (token, head) into
    the int8 paged cache ([blocks, block_size, Hkv, >= D] views) and writes their
    fp32 scales ([blocks, block_size, Hkv] views); slot_mapping int64 [tokens]
    gives each token's slot, negative = skip. The reference leaves this step to
    vLLM; rule "reference" is quantize() of its tests/test_attn_prefill.py:202-206,
    "vllm" the rule of vLLM 0.22's int8_per_token_head writer."""
    torch.ops.strix.kv_write_i8(key, value, key_cache, value_cache, k_scale, v_scale,
                                slot_mapping.to(torch.int64), rule)


def packed_int8_kv_views(kv_cache: torch.Tensor):
    """(key_cache, value_cache, k_scale, v_scale) views of vLLM 0.22's packed
    int8_per_token_head cache [blocks, 2, block_size, Hkv, D + 4] (int8; the last
    four bytes of every head row hold its fp32 scale): byte views [blocks,
    block_size, Hkv, D] and strided fp32 views [blocks, block_size, Hkv]. The
    reference's plugin carves the same views (python/strix_vllm/attn.py:185-203)."""
    assert kv_cache.dtype == torch.int8 and kv_cache.dim() == 5 and kv_cache.size(1) == 2
    blocks, _, bs, hkv, padded = kv_cache.shape
    d = padded - 4
    key_cache, value_cache = kv_cache[:, 0, :, :, :d], kv_cache[:, 1, :, :, :d]
    f32 = torch.empty(0, dtype=torch.float32, device=kv_cache.device).set_(kv_cache.untyped_storage())
    st = kv_cache.stride()
    base = kv_cache.storage_offset()
    assert all(x % 4 == 0 for x in (st[0], st[1], st[2], st[3], base, d)), "cache not 4-byte aligned"

    def scales(half):
        return torch.as_strided(f32, (blocks, bs, hkv), (st[0] // 4, st[2] // 4, st[3] // 4),
                                (base + half * st[1] + d) // 4)

    return key_cache, value_cache, scales(0), scales(1)


__all__ = [
    "attn_prefill",
    "Range",
    "StrixError",
    "attn_decode",
    "explain",
    "geometries",
    "is_supported_device",
    "kernels",
    "kv_write_int8",
    "moe",
    "ops",
    "packed_int8_kv_views",
    "select",
    "selections",
]
