"""The int8 KV-cache writer (strix_kv_write_i8) against the oracle's
quantize_kv - the reference's quantize(), tests/test_attn_prefill.py:202-206 -
bit for bit, in both cache layouts, and the written cache read back by the
attention kernels."""

import pytest
import torch

from oracle import attention as A

DEV = "cuda"


def _inputs(tokens, hkv, d, blocks, bs, seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    key = (torch.randn(tokens, hkv, d, generator=g) * 1.7).to(dtype)
    value = torch.randn(tokens, hkv, d, generator=g).to(dtype)
    key[0, 0] = 0                                        # an all-zero row: scale 1e-8 / 127
    if tokens > 2:
        key[2, hkv - 1, 3] = 300.0                       # an outlier sets the scale of its row
    slots = torch.randperm(blocks * bs, generator=g)[:tokens].to(torch.int64)
    if tokens > 3:
        slots[3] = -1                                    # a padding token writes nothing
    return key, value, slots


def _expect(key, value, slots, blocks, bs, rule):
    quant = A.quantize_kv if rule == "reference" else A.quantize_kv_vllm
    hkv, d = key.shape[1:]
    kq, ks = quant(key)
    vq, vs = quant(value)
    kc = torch.full((blocks, bs, hkv, d), 77, dtype=torch.int8)
    vc, ksc, vsc = kc.clone(), torch.full((blocks, bs, hkv), -1.0), torch.full((blocks, bs, hkv), -1.0)
    live = slots >= 0
    b, o = slots[live] // bs, slots[live] % bs
    kc[b, o], vc[b, o], ksc[b, o], vsc[b, o] = kq[live], vq[live], ks[live], vs[live]
    return kc, vc, ksc, vsc


@pytest.mark.gpu
@pytest.mark.parametrize("rule", ["reference", "vllm"])
@pytest.mark.parametrize("tokens,hkv,d,dtype", [(1, 1, 64, torch.bfloat16), (37, 4, 128, torch.bfloat16),
                                                (19, 2, 256, torch.float16), (5, 8, 512, torch.bfloat16),
                                                (300, 8, 128, torch.bfloat16)])
def test_separate_scale_layout_is_bit_exact(strix, tokens, hkv, d, dtype, rule):
    blocks, bs = 40, 16
    key, value, slots = _inputs(tokens, hkv, d, blocks, bs, seed=tokens, dtype=dtype)
    kc = torch.full((blocks, bs, hkv, d), 77, dtype=torch.int8, device=DEV)
    vc = kc.clone()
    ks = torch.full((blocks, bs, hkv), -1.0, device=DEV)
    vs = ks.clone()
    strix.kv_write_int8(key.to(DEV), value.to(DEV), kc, vc, ks, vs, slots.to(DEV), rule)
    ekc, evc, eks, evs = _expect(key, value, slots, blocks, bs, rule)
    assert torch.equal(ks.cpu(), eks) and torch.equal(vs.cpu(), evs)
    assert torch.equal(kc.cpu(), ekc) and torch.equal(vc.cpu(), evc)


@pytest.mark.gpu
def test_packed_layout_with_inline_scales(strix):
    """vLLM 0.22's cache: [blocks, 2, block_size, Hkv, D + 4], scale after the bytes."""
    blocks, bs, hkv, d, tokens = 12, 16, 4, 128, 50
    key, value, slots = _inputs(tokens, hkv, d, blocks, bs, seed=9)
    cache = torch.full((blocks, 2, bs, hkv, d + 4), 77, dtype=torch.int8, device=DEV)
    kc, vc, ks, vs = strix.packed_int8_kv_views(cache)
    ks.fill_(-1.0), vs.fill_(-1.0)
    strix.kv_write_int8(key.to(DEV), value.to(DEV), kc, vc, ks, vs, slots.to(DEV))
    ekc, evc, eks, evs = _expect(key, value, slots, blocks, bs, "reference")
    assert torch.equal(kc.cpu(), ekc) and torch.equal(vc.cpu(), evc)
    assert torch.equal(ks.cpu(), eks) and torch.equal(vs.cpu(), evs)
    # the scale bytes sit right after each head's D bytes
    raw = cache.cpu()[:, 0, :, :, d:].contiguous().view(torch.float32).squeeze(-1)
    assert torch.equal(raw, eks)


@pytest.mark.gpu
def test_written_cache_feeds_decode_attention(strix):
    """bf16 K/V -> kv_write_int8 -> attn_decode equals the oracle over the oracle's cache."""
    hq, hkv, d, bs = 32, 4, 128, 16
    ctx = [700, 33, 1500]
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([1] * len(ctx), ctx, hq, hkv, bs, seed=4, hd=d)
    kq, ks = A.quantize_kv(kc)
    vq, vs = A.quantize_kv(vc)
    ref = A.decode_reference(q, kq, vq, ks, vs, seq_lens, table, d ** -0.5)
    # present every cache row as a "new token" at its own slot
    blocks = kc.size(0)
    slots = torch.arange(blocks * bs, dtype=torch.int64, device=DEV)
    gk = torch.zeros(blocks, bs, hkv, d, dtype=torch.int8, device=DEV)
    gv = torch.zeros_like(gk)
    gks = torch.zeros(blocks, bs, hkv, device=DEV)
    gvs = torch.zeros_like(gks)
    strix.kv_write_int8(kc.reshape(-1, hkv, d).contiguous().to(DEV),
                        vc.reshape(-1, hkv, d).contiguous().to(DEV), gk, gv, gks, gvs, slots)
    assert torch.equal(gk.cpu(), kq) and torch.equal(gvs.cpu(), vs)
    out = torch.empty_like(q, device=DEV)
    strix.attn_decode(out, q.to(DEV), gk, gv, seq_lens.to(DEV), table.to(DEV), d ** -0.5, 0, -1,
                      gks, gvs)
    err = (out.float().cpu() - ref).abs()
    rms = ref.pow(2).mean().sqrt().item()
    assert bool((err <= 2e-2 * rms + ref.abs() * 2.0 ** -8).all())


@pytest.mark.gpu
def test_rejects_bad_arguments(strix):
    k = torch.zeros(2, 1, 12, dtype=torch.bfloat16, device=DEV)
    c = torch.zeros(1, 16, 1, 12, dtype=torch.int8, device=DEV)
    s = torch.zeros(1, 16, 1, device=DEV)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        strix.kv_write_int8(k, k, c, c, s, s, torch.zeros(2, dtype=torch.int64, device=DEV))


def test_vllm_rule_oracle_properties():
    """CPU: the vLLM-rule twin clamps to [-128, 127], truncates, and floors the scale."""
    x = torch.tensor([[[0.0] * 8, [1.0, -1.0, 0.999, -0.999, 0.5, 0.004, -0.004, 0.0]]]).bfloat16()
    q, s = A.quantize_kv_vllm(x)
    assert float(s[0, 0]) == pytest.approx(1e-6) and int(q[0, 0].abs().max()) == 0
    assert q[0, 1, 0] in (126, 127) and q[0, 1, 1] in (-127, -126) and int(q[0, 1, 5]) == 0
    qr, sr = A.quantize_kv(x)
    assert int(qr[0, 1, 0]) == 127 and int(qr[0, 1, 5]) == 1   # the reference rule rounds
