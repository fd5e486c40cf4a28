"""Parity of the sm_100a decode-attention kernel (through the C-ABI) with the CPU
oracle. Mirrors the decode cases of the reference's tests/test_attn_prefill.py
(test_decode_int8_matches_reference :167-195, test_h128_g8_decode_sinks :283-312)
and adds the benchmark geometry (batch of ragged contexts, GQA 8, head 128)."""

from pathlib import Path

import pytest
import torch

from libstrix_b200.workloads import decode_batch
from oracle import attention as A

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"
DEV = "cuda"


def check(out, ref, tol=2e-2):
    """Reference tolerance (rtol = atol = 2e-2) plus the stricter bound for
    int8-KV outputs: |err| <= 2e-2 x RMS(ref), widened per element by the bf16
    output quantum (half an ulp, at most 2^-8 |ref|) that no kernel can avoid."""
    out = out.float().cpu()
    assert torch.isfinite(out).all()
    torch.testing.assert_close(out, ref, rtol=tol, atol=tol)
    rms = ref.pow(2).mean().sqrt().item()
    bound = tol * max(rms, 1e-3) + ref.abs() * 2.0 ** -8
    assert bool(((out - ref).abs() <= bound).all()), \
        f"max err {(out - ref).abs().max().item():.3g} vs {tol} x rms {rms:.3g}"


def run_case(strix, hq, hkv, hd, ctx_lens, block_size, num_splits, window_left, use_sinks,
             seed=0):
    q_lens = [1] * len(ctx_lens)
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv(q_lens, ctx_lens, hq, hkv, block_size,
                                                      seed=seed, hd=hd)
    kq, ks = A.quantize_kv(kc)
    vq, vs = A.quantize_kv(vc)
    sinks = (torch.randn(hq, generator=torch.Generator().manual_seed(seed + 1)) * 2).float() \
        if use_sinks else None
    scale = hd ** -0.5
    ref = A.decode_reference(q, kq, vq, ks, vs, seq_lens, table, scale, window_left, sinks)
    out = torch.full_like(q, float("nan"), device=DEV)
    strix.attn_decode(out, q.to(DEV), kq.to(DEV), vq.to(DEV), seq_lens.to(DEV), table.to(DEV),
                      scale, num_splits, window_left, ks.to(DEV), vs.to(DEV),
                      sinks=None if sinks is None else sinks.to(DEV))
    check(out, ref)


@pytest.mark.parametrize("ctx_lens", [[0], [70, 200, 3], [500, 31, 1000, 64]])
@pytest.mark.parametrize("num_splits", [1, 4, 0])
@pytest.mark.parametrize("window_left", [-1, 40])
@pytest.mark.parametrize("use_sinks", [False, True])
def test_h128_g8_decode(strix, ctx_lens, num_splits, window_left, use_sinks):
    run_case(strix, 32, 4, 128, ctx_lens, 16, num_splits, window_left, use_sinks)


@pytest.mark.parametrize("hq,hkv,hd", [(16, 2, 256), (32, 16, 256), (24, 4, 256), (8, 1, 128),
                                       (8, 4, 128), (4, 4, 128)])
@pytest.mark.parametrize("num_splits", [1, 4, 13])
@pytest.mark.parametrize("block_size", [16, 272])
def test_other_geometries(strix, hq, hkv, hd, num_splits, block_size):
    run_case(strix, hq, hkv, hd, [500, 31, 1000, 64], block_size, num_splits, 31 if hkv == 16 else -1,
             False)


@pytest.mark.parametrize("hq,hkv,hd", [(16, 2, 512), (32, 2, 128), (8, 2, 64), (24, 2, 256)])
@pytest.mark.parametrize("window_left,use_sinks", [(-1, False), (40, True)])
def test_int8_cache_through_the_grouped_form(strix, hq, hkv, hd, window_left, use_sinks):
    """Head 512 GQA 8 over an int8 cache (python/strix/registry.py:478-492 of the
    reference), head 64, and GQA ratios above 8: served by the prefill kernel in its
    decode form (the query heads of a KV head as rows of one sequence)."""
    run_case(strix, hq, hkv, hd, [70, 200, 3, 0, 1000], 16, 1, window_left, use_sinks)


def test_golden_fixture_cases(strix):
    """The reference's own outputs for its own inputs (tests/golden/attn_decode.pt)."""
    for c in torch.load(GOLDEN / "attn_decode.pt"):
        out = torch.full_like(c["q"], float("nan"), device=DEV)
        for splits in (1, 3, 0):
            strix.attn_decode(out, c["q"].to(DEV), c["key_cache"].to(DEV),
                              c["value_cache"].to(DEV), c["seq_lens"].to(DEV),
                              c["block_table"].to(DEV), c["scale"], splits, c["window_left"],
                              c["k_scale"].to(DEV), c["v_scale"].to(DEV),
                              sinks=None if c["sinks"] is None else c["sinks"].to(DEV))
            check(out, c["out"])


def test_strided_layouts(strix):
    """Interleaved K/V storage (the reference's fork layout), a packed layout
    whose head stride (D + 4 bytes) breaks 16-byte alignment, strided scales,
    and a strided q/out - all must give the contiguous answer."""
    hq, hkv, hd, bs = 32, 4, 128, 16
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([1, 1, 1], [300, 17, 90], hq, hkv, bs, hd=hd)
    kq, ks = A.quantize_kv(kc)
    vq, vs = A.quantize_kv(vc)
    scale = hd ** -0.5
    ref = A.decode_reference(q, kq, vq, ks, vs, seq_lens, table, scale)
    nb = kq.size(0)
    # (a) K and V interleaved per slot: [blocks, bs, Hkv, 2 * hd] storage
    inter = torch.empty(nb, bs, hkv, 2 * hd, dtype=torch.int8, device=DEV)
    inter[..., :hd] = kq.to(DEV)
    inter[..., hd:] = vq.to(DEV)
    # (b) packed: bytes followed by the fp32 scale, head stride hd + 4
    packed_k = torch.zeros(nb, bs, hkv, hd + 4, dtype=torch.int8, device=DEV)
    packed_v = torch.zeros_like(packed_k)
    packed_k[..., :hd] = kq.to(DEV)
    packed_v[..., :hd] = vq.to(DEV)
    packed_k[..., hd:].view(torch.float32)[..., 0] = ks.to(DEV)
    packed_v[..., hd:].view(torch.float32)[..., 0] = vs.to(DEV)
    ks_view = packed_k[..., hd:].view(torch.float32)[..., 0]
    vs_view = packed_v[..., hd:].view(torch.float32)[..., 0]
    assert ks_view.stride(2) == (hd + 4) // 4
    qbig = torch.zeros(3, hq, 2 * hd, dtype=torch.bfloat16, device=DEV)
    qbig[..., :hd] = q.to(DEV)
    obig = torch.full_like(qbig, float("nan"))
    for splits in (1, 0):
        out = torch.full_like(q, float("nan"), device=DEV)
        strix.attn_decode(out, q.to(DEV), inter[..., :hd], inter[..., hd:], seq_lens.to(DEV),
                          table.to(DEV), scale, splits, -1, ks.to(DEV), vs.to(DEV))
        check(out, ref)
        strix.attn_decode(obig[..., :hd], qbig[..., :hd], packed_k[..., :hd], packed_v[..., :hd],
                          seq_lens.to(DEV), table.to(DEV), scale, splits, -1, ks_view, vs_view)
        check(obig[..., :hd], ref)


def test_stale_slots_past_the_sequence_do_not_leak(strix):
    """Bytes and scales of slots past seq_len (same page) are garbage: NaN
    scales and extreme bytes there must not reach the output."""
    hq, hkv, hd, bs = 32, 4, 128, 16
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([1, 1], [36, 5], hq, hkv, bs, hd=hd)
    kq, ks = A.quantize_kv(kc)
    vq, vs = A.quantize_kv(vc)
    ref = A.decode_reference(q, kq, vq, ks, vs, seq_lens, table, hd ** -0.5)
    for n, ln in enumerate(seq_lens.tolist()):
        blk, off = int(table[n, (ln - 1) // bs]), (ln - 1) % bs + 1
        ks[blk, off:] = float("nan")
        vs[blk, off:] = float("nan")
        kq[blk, off:] = 127
        vq[blk, off:] = -128
    for splits in (1, 2, 0):
        out = torch.full_like(q, float("nan"), device=DEV)
        strix.attn_decode(out, q.to(DEV), kq.to(DEV), vq.to(DEV), seq_lens.to(DEV), table.to(DEV),
                          hd ** -0.5, splits, -1, ks.to(DEV), vs.to(DEV))
        check(out, ref)


def test_all_int8_codes_and_extreme_scores(strix):
    """Every int8 code appears in K and V (exact widening), and one key dominates
    the softmax by a wide margin (max tracking)."""
    hq, hkv, hd, bs = 32, 4, 128, 16
    b = decode_batch(ctx_lens=[256, 40], hq=hq, hkv=hkv, head_dim=hd, block_size=bs, seed=3)
    codes = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8)
    b.key_cache.view(-1)[: 256 * 8] = codes.repeat(8)
    b.value_cache.view(-1)[: 256 * 8] = codes.flip(0).repeat(8)
    blk = int(b.block_table[0, 3])
    b.k_scale[blk, 5] = 2.0   # a key with a far larger logit
    ref = A.decode_reference(b.q, b.key_cache, b.value_cache, b.k_scale, b.v_scale, b.seq_lens,
                             b.block_table, b.scale)
    g = b.to(DEV)
    for splits in (1, 0):
        out = torch.full_like(g.q, float("nan"))
        strix.attn_decode(out, g.q, g.key_cache, g.value_cache, g.seq_lens, g.block_table, g.scale,
                          splits, -1, g.k_scale, g.v_scale)
        check(out, ref)


def test_ragged_batch_benchmark_geometry(strix):
    """The benchmark's geometry at a size the oracle finishes in seconds: 12
    sequences with contexts from 1 to 9,000 keys, automatic segmentation vs
    reference-style splits, guard rows around the output untouched."""
    lens = [1, 15, 16, 17, 1023, 1024, 1025, 2048, 4100, 9000, 333, 7777]
    b = decode_batch(ctx_lens=lens, seed=1)
    ref = A.decode_reference(b.q, b.key_cache, b.value_cache, b.k_scale, b.v_scale, b.seq_lens,
                             b.block_table, b.scale)
    g = b.to(DEV)
    guarded = torch.full((len(lens) + 2, 32, 128), 7.0, dtype=torch.bfloat16, device=DEV)
    outs = []
    for splits in (0, 1, 8, 64):
        out = guarded[1:-1]
        out.fill_(float("nan"))
        strix.attn_decode(out, g.q, g.key_cache, g.value_cache, g.seq_lens, g.block_table, g.scale,
                          splits, -1, g.k_scale, g.v_scale)
        check(out, ref)
        assert bool((guarded[0] == 7).all()) and bool((guarded[-1] == 7).all())
        outs.append(out.float().cpu())
    # split-count invariance (size-independent property): all partitions agree
    for o in outs[1:]:
        torch.testing.assert_close(o, outs[0], rtol=1e-2, atol=1e-2)


def test_full_size_properties(strix):
    """At the benchmark's full size (64 sequences, contexts U[1024, 65536],
    ~2.2 GB of KV) the oracle is run on a sample of sequences only; the whole
    batch is checked through size-independent properties: (1) two different
    key partitions agree; (2) shuffling the physical blocks (with the table)
    leaves the output unchanged bit for bit."""
    g = decode_batch(seed=0, device=DEV)
    out_auto = torch.full_like(g.q, float("nan"))
    out_split = torch.full_like(g.q, float("nan"))
    strix.attn_decode(out_auto, g.q, g.key_cache, g.value_cache, g.seq_lens, g.block_table,
                      g.scale, 0, -1, g.k_scale, g.v_scale)
    strix.attn_decode(out_split, g.q, g.key_cache, g.value_cache, g.seq_lens, g.block_table,
                      g.scale, 16, -1, g.k_scale, g.v_scale)
    assert torch.isfinite(out_auto.float()).all()
    torch.testing.assert_close(out_auto.float(), out_split.float(), rtol=1e-2, atol=1e-2)
    # oracle on the shortest, the longest and two more sequences
    lens = g.seq_lens.cpu()
    pick = sorted({int(lens.argmin()), int(lens.argmax()), 7, 42})
    for n in pick:
        nb = (int(lens[n]) + 15) // 16
        blocks = g.block_table[n, :nb].long()
        sub_tbl = torch.arange(nb, dtype=torch.int32)[None]
        ref = A.decode_reference(
            g.q[n:n + 1].cpu(), g.key_cache[blocks].cpu(), g.value_cache[blocks].cpu(),
            g.k_scale[blocks].cpu(), g.v_scale[blocks].cpu(), lens[n:n + 1], sub_tbl, g.scale)
        check(out_auto[n:n + 1], ref)
    # block shuffle: permute physical blocks of the first 6 sequences in place
    nbs = [(int(x) + 15) // 16 for x in lens[:6]]
    ids = torch.cat([g.block_table[i, :nb] for i, nb in enumerate(nbs)]).long()
    perm = ids[torch.randperm(ids.numel(), device=DEV)]
    for t in (g.key_cache, g.value_cache, g.k_scale, g.v_scale):
        t[perm] = t[ids]
    table2 = g.block_table.clone()
    ofs = 0
    for i, nb in enumerate(nbs):
        table2[i, :nb] = perm[ofs:ofs + nb].int()
        ofs += nb
    out2 = torch.full_like(g.q, float("nan"))
    strix.attn_decode(out2, g.q, g.key_cache, g.value_cache, g.seq_lens, table2, g.scale, 0, -1,
                      g.k_scale, g.v_scale)
    assert torch.equal(out2[:6], out_auto[:6])


@pytest.mark.parametrize("hq,hkv,hd", [(32, 4, 128), (16, 2, 128), (8, 8, 64), (6, 1, 128),
                                       (16, 2, 256), (8, 4, 256), (6, 1, 256), (16, 2, 512), (4, 4, 512),
                                       (32, 2, 128), (24, 2, 64)])
@pytest.mark.parametrize("num_splits", [0, 1, 5])
def test_bf16_kv_cache(strix, hq, hkv, hd, num_splits):
    """The reference's native form: a bf16 cache, split-KV, window and sinks, ragged
    lengths, stale NaN rows past the sequences - against the dense oracle."""
    lens = [1, 17, 300, 1500, 16, 33]
    bs = 16
    g = torch.Generator().manual_seed(hq * 100 + hd + num_splits)
    nblk = [(n + bs - 1) // bs for n in lens]
    total = sum(nblk) + 2
    kc = torch.randn(total, bs, hkv, hd, generator=g).bfloat16()
    vc = torch.randn(total, bs, hkv, hd, generator=g).bfloat16()
    perm = torch.randperm(total, generator=g)
    table = torch.zeros(len(lens), max(nblk), dtype=torch.int32)
    at = 0
    for i, nb in enumerate(nblk):
        table[i, :nb] = perm[at:at + nb].int()
        at += nb
    seq_lens = torch.tensor(lens, dtype=torch.int32)
    q = torch.randn(len(lens), hq, hd, generator=g).bfloat16()
    scale = hd ** -0.5
    for window, use_sinks in ((-1, False), (200, True)):
        if use_sinks and num_splits not in (0, 1):
            continue
        sinks = torch.randn(hq, generator=g) if use_sinks else None
        cu = torch.arange(len(lens) + 1, dtype=torch.int32)
        ref = A.attention_reference(q, kc.float(), vc.float(), cu, seq_lens, table, scale, window, sinks)
        # slots past each sequence hold NaN: they must not reach the output
        kd, vd = kc.clone(), vc.clone()
        for i, n in enumerate(lens):
            if n % bs:
                blk = int(table[i, (n - 1) // bs])
                kd[blk, n % bs:] = float("nan")
                vd[blk, n % bs:] = float("nan")
        out = torch.full_like(q, float("nan")).to(DEV)
        strix.attn_decode(out, q.to(DEV), kd.to(DEV), vd.to(DEV), seq_lens.to(DEV), table.to(DEV), scale,
                          num_splits, window, None, None, None if sinks is None else sinks.to(DEV))
        torch.cuda.synchronize()
        check(out, ref)


def test_op_errors(strix):
    b = decode_batch(ctx_lens=[40]).to(DEV)
    out = torch.empty_like(b.q)
    args = (b.key_cache, b.value_cache, b.seq_lens, b.block_table, b.scale)
    with pytest.raises(RuntimeError, match="int8 KV needs k_scale and v_scale"):
        torch.ops.strix.attn_decode_bf16(out, b.q, *args, 1)
    with pytest.raises(RuntimeError, match=r"num_splits in \[1, 64\]"):
        torch.ops.strix.attn_decode_bf16(out, b.q, *args, 65, -1, b.k_scale, b.v_scale)
    with pytest.raises(RuntimeError, match="int32 metadata"):
        torch.ops.strix.attn_decode_bf16(out, b.q, b.key_cache, b.value_cache, b.seq_lens.long(),
                                         b.block_table, b.scale, 1, -1, b.k_scale, b.v_scale)
    with pytest.raises(RuntimeError, match="out must match q"):
        torch.ops.strix.attn_decode_bf16(out[:, :16], b.q, *args, 1, -1, b.k_scale, b.v_scale)
    with pytest.raises(RuntimeError, match="sinks must be contiguous fp32"):
        torch.ops.strix.attn_decode_bf16(out, b.q, *args, 1, -1, b.k_scale, b.v_scale,
                                         torch.zeros(3, device=DEV))
    with pytest.raises(RuntimeError, match="not built"):
        strix.attn_decode(torch.empty(1, 8, 64, dtype=torch.bfloat16, device=DEV),
                          torch.empty(1, 8, 64, dtype=torch.bfloat16, device=DEV),
                          b.key_cache[..., :64], b.value_cache[..., :64], b.seq_lens, b.block_table,
                          0.1, 1, -1, b.k_scale, b.v_scale)


def test_empty_batch_and_zero_length(strix):
    b = decode_batch(ctx_lens=[40, 0, 9]).to(DEV)
    out = torch.full_like(b.q, float("nan"))
    strix.attn_decode(out, b.q, b.key_cache, b.value_cache, b.seq_lens, b.block_table, b.scale, 1,
                      -1, b.k_scale, b.v_scale)
    assert bool((out[1] == 0).all()) and torch.isfinite(out.float()).all()
    strix.attn_decode(out, b.q, b.key_cache, b.value_cache, b.seq_lens, b.block_table, b.scale, 0,
                      -1, b.k_scale, b.v_scale)
    assert bool((out[1] == 0).all()) and torch.isfinite(out.float()).all()
    empty = b.q[:0]
    strix.attn_decode(torch.empty_like(empty), empty, b.key_cache, b.value_cache, b.seq_lens[:0],
                      b.block_table[:0], b.scale, 4, -1, b.k_scale, b.v_scale)
