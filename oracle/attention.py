"""Oracle for paged attention (decode and prefill), CPU torch, fp32.

Restates tests/test_attn_prefill.py of the reference: `build` (:9-27),
`reference` (:30-59) and `quantize` (:202-206). The reference hard-codes
device="cuda" in those helpers; here everything runs on the CPU.
"""

from __future__ import annotations

import torch


def build_paged_kv(q_lens, ctx_lens, hq, hkv, block_size, seed=0, hd=256, spare_blocks=3):
    """Random paged KV, K/V interleaved per slot ([blocks, Hkv, bs, 2*hd] storage
    viewed as two [blocks, bs, Hkv, hd] caches), shuffled block tables.

    Follows build() at tests/test_attn_prefill.py:9-27. Returns
    (q, key_cache, value_cache, cu_seqlens_q, seq_lens, block_table).
    """
    gen = torch.Generator().manual_seed(seed)
    seq_lens = [q + c for q, c in zip(q_lens, ctx_lens)]
    nblk = [(s + block_size - 1) // block_size for s in seq_lens]
    total = sum(nblk) + spare_blocks
    kv = torch.randn(total, hkv, block_size, 2 * hd, generator=gen).bfloat16()
    key_cache, value_cache = kv.transpose(1, 2).split(hd, dim=-1)
    perm = torch.randperm(total, generator=gen)
    table = torch.zeros(len(q_lens), max(max(nblk), 1), dtype=torch.int32)
    used = 0
    for i, nb in enumerate(nblk):
        table[i, :nb] = perm[used:used + nb]
        used += nb
    q = torch.randn(sum(q_lens), hq, hd, generator=gen).bfloat16()
    cu = torch.tensor([0, *torch.tensor(q_lens).cumsum(0).tolist()], dtype=torch.int32)
    return q, key_cache, value_cache, cu, torch.tensor(seq_lens, dtype=torch.int32), table


def quantize_kv(cache: torch.Tensor):
    """[blocks, bs, Hkv, D] bf16 -> int8 bytes + fp32 scale [blocks, bs, Hkv].

    scale = max(absmax, 1e-8) / 127, q = clamp(round(x / scale), +-127):
    quantize() at tests/test_attn_prefill.py:202-206.
    """
    s = cache.abs().amax(-1).float().clamp_min(1e-8) / 127.0
    q = (cache.float() / s[..., None]).round().clamp(-127, 127).to(torch.int8)
    return q, s.contiguous()


def quantize_kv_vllm(cache: torch.Tensor):
    """The rule of vLLM 0.22's int8_per_token_head cache writer
    (vllm/v1/attention/ops/triton_reshape_and_cache_flash.py, the third-party
    dependency that writes the cache in a deployment): scale = max(absmax / 127,
    1e-6), q = x * (1 / scale) clamped to [-128, 127] and converted to int8 by
    truncation. Parity unpinned: that Triton kernel cannot run without a GPU,
    so this restates its source."""
    s = (cache.abs().amax(-1).float() / 127.0).clamp_min(1e-6)
    q = (cache.float() * (1.0 / s)[..., None]).clamp(-128, 127).trunc().to(torch.int8)
    return q, s.contiguous()


def attention_reference(q, key_cache, value_cache, cu, seq_lens, table, scale,
                        window_left=-1, sinks=None):
    """Dense causal softmax attention over the gathered pages, fp32.

    Follows reference() at tests/test_attn_prefill.py:30-59: the queries of
    sequence n are the last q_len of its seq_lens[n] positions; query at
    position p sees keys <= p (and >= p - window_left when window_left >= 0);
    a sink is one extra unscaled logit per head that is dropped after the
    softmax. key_cache / value_cache may be any float dtype (dequantise int8
    caches before the call, as the reference's int8 tests do).
    """
    hq, hkv = q.size(1), key_cache.size(2)
    bs = key_cache.size(1)
    out = torch.empty_like(q, dtype=torch.float32)
    for n in range(cu.numel() - 1):
        a, b, kv_len = int(cu[n]), int(cu[n + 1]), int(seq_lens[n])
        pos = torch.arange(kv_len)
        blocks = table[n, pos // bs].long()
        k = key_cache[blocks, pos % bs].float().repeat_interleave(hq // hkv, 1)
        v = value_cache[blocks, pos % bs].float().repeat_interleave(hq // hkv, 1)
        s = torch.einsum("thd,khd->htk", q[a:b].float(), k) * scale
        qpos = kv_len - (b - a) + torch.arange(b - a)
        s.masked_fill_(pos[None, None, :] > qpos[None, :, None], float("-inf"))
        if window_left >= 0:
            s.masked_fill_(qpos[None, :, None] - pos[None, None, :] > window_left, float("-inf"))
        if sinks is not None:
            sink = sinks.float()[:, None, None].expand(-1, b - a, 1)
            p = torch.cat([s, sink], -1).softmax(-1)[..., :-1]
        else:
            p = s.softmax(-1)
        out[a:b] = torch.einsum("htk,khd->thd", p, v)
    return out


def decode_reference(q, key_q, val_q, k_scale, v_scale, seq_lens, table, scale,
                     window_left=-1, sinks=None):
    """Decode (one query per sequence) over an int8 cache: dequantise, then the
    dense reference - test_decode_int8_matches_reference,
    tests/test_attn_prefill.py:167-195."""
    n = q.size(0)
    cu = torch.arange(n + 1, dtype=torch.int32)
    return attention_reference(
        q, key_q.float() * k_scale[..., None], val_q.float() * v_scale[..., None],
        cu, seq_lens, table, scale, window_left, sinks)
