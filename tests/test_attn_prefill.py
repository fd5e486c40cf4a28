"""Prefill attention against the CPU oracle; cases follow the reference's
tests/test_attn_prefill.py (ragged q lens, prefix context, block sizes 16 and a
hybrid-style large block, int8 KV against the dequantised reference, window,
sinks), at the head sizes built here (64 and 128), plus the config-4 geometry
(40 q / 8 kv heads) at a size the CPU oracle finishes, and size-independent
properties at 8192 tokens."""

import pytest
import torch

import libstrix_b200 as strix
from oracle import attention as A

pytestmark = pytest.mark.gpu
DEV = "cuda"


LONG = ("test_long_sequence", "test_config4", "test_decode_with_bf16", "test_unbuilt", "test_sinks_refuse")


@pytest.fixture(params=["auto", "mma"], autouse=True)
def prefill_impl(request, monkeypatch):
    """Every case runs on the tcgen05 kernel ("auto": it covers head 64 / 128 with
    16-byte aligned rows) and, the short ones, on the mma.sync kernel that serves
    the remaining layouts."""
    from libstrix_b200 import torch_ops

    if request.param == "mma" and request.node.name.startswith(LONG):
        pytest.skip("long cases run once, on the default kernel")
    monkeypatch.setattr(torch_ops, "PREFILL_IMPL", request.param)
    return request.param


def umma_status():
    import ctypes

    from libstrix_b200 import _lib

    flag = ctypes.c_int32(-1)
    assert _lib.load().strix_umma_status(ctypes.byref(flag)) == 0
    return flag.value


def run(q, kc, vc, cu, seq_lens, table, scale, num_splits=1, window_left=-1, ks=None, vs=None,
        sinks=None):
    out = torch.full_like(q, float("nan"), device=DEV)
    d = lambda t: None if t is None else t.to(DEV)  # noqa: E731
    strix.attn_prefill(out, d(q), d(kc), d(vc), d(cu), d(seq_lens), d(table), scale, num_splits,
                       window_left, d(ks), d(vs), d(sinks))
    res = out.float().cpu()
    assert umma_status() == 0, "a bounded wait of a tcgen05 kernel gave up"
    return res


def check(out, ref):
    """rtol = atol = 2e-2 as the reference's tests, and the tighter bound
    |err| <= 2e-2 x RMS(ref) + the bf16 output quantum."""
    assert torch.isfinite(out).all()
    torch.testing.assert_close(out, ref, rtol=2e-2, atol=2e-2)
    rms = ref.pow(2).mean().sqrt().item()
    err = (out - ref).abs()
    assert bool((err <= 2e-2 * rms + ref.abs() * 2.0 ** -8).all()), \
        f"max err {err.max().item():.3g} vs rms {rms:.3g}"


def dequant_refs(q, kq, ks, vq, vs, cu, seq_lens, table, scale, window_left=-1, sinks=None):
    """(reference on the exact dequantised cache, reference on the cache rounded
    to bf16 - the statement of tests/test_attn_prefill.py:224-226). The kernel
    keeps the int8 values exact and applies the fp32 scales to score and P, so
    the tight bound is taken against the first."""
    kx, vx = kq.float() * ks[..., None], vq.float() * vs[..., None]
    exact = A.attention_reference(q, kx, vx, cu, seq_lens, table, scale, window_left, sinks)
    rounded = A.attention_reference(q, kx.bfloat16(), vx.bfloat16(), cu, seq_lens, table, scale,
                                    window_left, sinks)
    return exact, rounded


CASES = [([64], [0]), ([1], [0]), ([37], [0]), ([100, 5, 17], [0, 40, 300]), ([200], [77])]


@pytest.mark.parametrize("hq,hkv,hd", [(32, 4, 128), (40, 8, 128), (32, 8, 64), (24, 4, 128)])
@pytest.mark.parametrize("q_lens,ctx_lens", CASES)
@pytest.mark.parametrize("block_size", [16, 544])
def test_bf16_kv_matches_reference(hq, hkv, hd, q_lens, ctx_lens, block_size):
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv(q_lens, ctx_lens, hq, hkv, block_size, hd=hd)
    scale = hd ** -0.5
    check(run(q, kc, vc, cu, seq_lens, table, scale),
          A.attention_reference(q, kc, vc, cu, seq_lens, table, scale))


@pytest.mark.parametrize("hq,hkv,hd", [(32, 4, 128), (40, 8, 128), (32, 8, 64)])
@pytest.mark.parametrize("q_lens,ctx_lens", CASES)
@pytest.mark.parametrize("num_splits", [1, 4])
def test_int8_kv_matches_dequantized_reference(hq, hkv, hd, q_lens, ctx_lens, num_splits):
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv(q_lens, ctx_lens, hq, hkv, 16, hd=hd)
    kq, ks = A.quantize_kv(kc)
    vq, vs = A.quantize_kv(vc)
    scale = hd ** -0.5
    out = run(q, kq, vq, cu, seq_lens, table, scale, num_splits, -1, ks, vs)
    exact, rounded = dequant_refs(q, kq, ks, vq, vs, cu, seq_lens, table, scale)
    check(out, exact)
    torch.testing.assert_close(out, rounded, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("hq,hkv,hd", [(12, 2, 256), (16, 2, 256), (4, 2, 256), (16, 2, 512), (3, 1, 512)])
@pytest.mark.parametrize("q_lens,ctx_lens", [([64], [0]), ([100, 5, 17], [0, 40, 300]), ([1, 1], [70, 200]),
                                             ([130], [77])])
@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("window_left,use_sinks", [(-1, False), (40, True)])
def test_head_256_and_512(hq, hkv, hd, q_lens, ctx_lens, int8, window_left, use_sinks):
    """Head 256 at GQA 6 / 8 / 2 and head 512 at GQA 8 (the reference's rows at
    python/strix/registry.py:368-441): the mma.sync kernel with the query tile in
    shared memory, at head 512 with the head's dims split over pairs of warps."""
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv(q_lens, ctx_lens, hq, hkv, 16, hd=hd)
    scale = hd ** -0.5
    sinks = torch.linspace(-1.0, 2.0, hq) if use_sinks else None
    if int8:
        kq, ks = A.quantize_kv(kc)
        vq, vs = A.quantize_kv(vc)
        out = run(q, kq, vq, cu, seq_lens, table, scale, 1, window_left, ks, vs, sinks)
        exact, _ = dequant_refs(q, kq, ks, vq, vs, cu, seq_lens, table, scale, window_left, sinks)
        check(out, exact)
    else:
        check(run(q, kc, vc, cu, seq_lens, table, scale, 1, window_left, None, None, sinks),
              A.attention_reference(q, kc, vc, cu, seq_lens, table, scale, window_left, sinks))


@pytest.mark.parametrize("q_lens,ctx_lens",
                         [([64], [0]), ([37], [0]), ([100, 5, 17], [0, 40, 300]), ([200], [700]),
                          ([1, 1, 1], [70, 200, 3])])
@pytest.mark.parametrize("window_left", [-1, 40, 512])
@pytest.mark.parametrize("use_sinks", [False, True])
@pytest.mark.parametrize("int8", [False, True])
def test_h128_g8_sinks_window(q_lens, ctx_lens, window_left, use_sinks, int8):
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv(q_lens, ctx_lens, 32, 4, 16, hd=128)
    scale = 128 ** -0.5
    sinks = (torch.randn(32, generator=torch.Generator().manual_seed(1)) * 2).float() \
        if use_sinks else None
    if int8:
        kq, ks = A.quantize_kv(kc)
        vq, vs = A.quantize_kv(vc)
        out = run(q, kq, vq, cu, seq_lens, table, scale, 1, window_left, ks, vs, sinks)
        exact, rounded = dequant_refs(q, kq, ks, vq, vs, cu, seq_lens, table, scale, window_left, sinks)
        check(out, exact)
        torch.testing.assert_close(out, rounded, rtol=2e-2, atol=2e-2)
        return
    out = run(q, kc, vc, cu, seq_lens, table, scale, 1, window_left, sinks=sinks)
    check(out, A.attention_reference(q, kc, vc, cu, seq_lens, table, scale, window_left, sinks))


def test_inline_scale_cache_layout():
    """vLLM's int8 cache keeps the fp32 scale after each head's bytes (head stride
    D + 4): byte view + strided scale view, rows only 4-byte aligned."""
    hq, hkv, hd, bs = 16, 4, 128, 16
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([70, 3], [0, 90], hq, hkv, bs, hd=hd)
    kq, ks = A.quantize_kv(kc)
    vq, vs = A.quantize_kv(vc)

    def inline(qv):
        """bytes of every head followed by 4 spare bytes: [blocks, bs, Hkv, D + 4]"""
        raw = torch.zeros(*qv.shape[:3], hd + 4, dtype=torch.int8)
        raw[..., :hd] = qv
        return raw.to(DEV)[..., :hd]

    kb, vb = inline(kq), inline(vq)
    scale = hd ** -0.5
    out = torch.full_like(q, float("nan"), device=DEV)
    strix.attn_prefill(out, q.to(DEV), kb, vb, cu.to(DEV), seq_lens.to(DEV), table.to(DEV), scale, 1,
                       -1, ks.to(DEV), vs.to(DEV))
    check(out.float().cpu(), dequant_refs(q, kq, ks, vq, vs, cu, seq_lens, table, scale)[0])


def test_sinks_refuse_split_kv():
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([4], [600], 32, 4, 16, hd=128)
    sinks = torch.zeros(32)
    with pytest.raises(RuntimeError, match="sinks need num_splits == 1"):
        run(q, kc, vc, cu, seq_lens, table, 0.1, 4, sinks=sinks)


def test_unbuilt_head_dim_is_rejected():
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([4], [0], 8, 2, 16, hd=96)
    with pytest.raises(RuntimeError, match="head_dim 64, 128, 256 or 512"):
        run(q, kc, vc, cu, seq_lens, table, 0.1)
    assert strix.select("attn_prefill", head_dim=96, gqa=4, dtype="bf16", kv_dtype="int8",
                        split_kv=False, window=False, causal=True, sinks=False) is None


def test_config4_geometry_2048_tokens():
    """40 q / 8 kv heads, head 128, block 16, one sequence of 2048 tokens, int8 KV
    written from bf16 N(0,1) values."""
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([2048], [0], 40, 8, 16, hd=128)
    kq, ks = A.quantize_kv(kc)
    vq, vs = A.quantize_kv(vc)
    scale = 128 ** -0.5
    out = run(q, kq, vq, cu, seq_lens, table, scale, 1, -1, ks, vs)
    check(out, dequant_refs(q, kq, ks, vq, vs, cu, seq_lens, table, scale)[0])


def test_long_sequence_properties():
    """8192 tokens: (1) the first query sees one key, so its output is that key's
    V row; (2) chunked prefill - the last 512 queries alone, with the rest as
    context - reproduces the tail of the full pass; (3) with constant V every
    output equals that constant (softmax weights sum to one)."""
    t, hq, hkv, hd = 8192, 8, 2, 128
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([t], [0], hq, hkv, 16, hd=hd)
    kq, ks = A.quantize_kv(kc)
    vq, vs = A.quantize_kv(vc)
    scale = hd ** -0.5
    full = run(q, kq, vq, cu, seq_lens, table, scale, 1, -1, ks, vs)
    blk0 = int(table[0, 0])
    v0 = (vq[blk0, 0].float() * vs[blk0, 0][:, None]).repeat_interleave(hq // hkv, 0)
    torch.testing.assert_close(full[0], v0.bfloat16().float(), rtol=1e-2, atol=1e-2)
    cu2 = torch.tensor([0, 512], dtype=torch.int32)
    tail = run(q[-512:], kq, vq, cu2, seq_lens, table, scale, 1, -1, ks, vs)
    torch.testing.assert_close(tail, full[-512:], rtol=0, atol=0)
    vconst = torch.full_like(vq, 64)
    ones = torch.full_like(vs, 1 / 64)
    flat = run(q, kq, vconst, cu, seq_lens, table, scale, 1, -1, ks, ones)
    torch.testing.assert_close(flat, torch.ones_like(flat), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("hq,hkv,hd", [(32, 4, 128), (32, 8, 64)])
@pytest.mark.parametrize("ctx_lens", [[0], [70, 200, 3], [500, 31, 1000, 64]])
@pytest.mark.parametrize("window_left", [-1, 31])
def test_decode_with_bf16_cache(hq, hkv, hd, ctx_lens, window_left):
    """strix.attn_decode on a bf16 cache (tests/test_attn_prefill.py:146-163)."""
    q_lens = [1] * len(ctx_lens)
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv(q_lens, ctx_lens, hq, hkv, 16, hd=hd)
    scale = hd ** -0.5
    out = torch.full_like(q, float("nan"), device=DEV)
    strix.attn_decode(out, q.to(DEV), kc.to(DEV), vc.to(DEV), seq_lens.to(DEV), table.to(DEV), scale,
                      1, window_left)
    check(out.float().cpu(), A.attention_reference(q, kc, vc, cu, seq_lens, table, scale, window_left))


def test_tcgen05_kernel_is_the_default_for_config4():
    """head 128 with contiguous rows is covered by the tensor-core kernel."""
    from libstrix_b200 import _lib

    assert _lib.load().strix_attn_prefill_umma_covers(128, 40 * 128, 128, 40 * 128, 128, 1) == 1
    assert _lib.load().strix_attn_prefill_umma_covers(256, 8 * 256, 256, 8 * 256, 256, 1) == 0
    assert _lib.load().strix_attn_prefill_umma_covers(128, 40 * 128 + 2, 128, 40 * 128, 128, 1) == 0


@pytest.mark.parametrize("q_lens,ctx_lens", [([300, 1, 257], [0, 511, 130]), ([129], [1000]),
                                             ([256, 256], [0, 256]), ([513], [0])])
@pytest.mark.parametrize("int8", [False, True])
def test_tile_boundaries(q_lens, ctx_lens, int8):
    """Query counts and contexts around the 128 / 256 tile sizes of the tensor-core
    kernel (second Q tile empty or ragged, keys ending inside a tile)."""
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv(q_lens, ctx_lens, 16, 4, 16, hd=128)
    scale = 128 ** -0.5
    if int8:
        kq, ks = A.quantize_kv(kc)
        vq, vs = A.quantize_kv(vc)
        out = run(q, kq, vq, cu, seq_lens, table, scale, 1, -1, ks, vs)
        check(out, dequant_refs(q, kq, ks, vq, vs, cu, seq_lens, table, scale)[0])
    else:
        check(run(q, kc, vc, cu, seq_lens, table, scale),
              A.attention_reference(q, kc, vc, cu, seq_lens, table, scale))


def test_lazy_rescale_with_growing_scores():
    """Scores that keep growing along the keys force the accumulator rescale of the
    tensor-core kernel (the row maximum moves by far more than 2^8 between tiles)."""
    t, hq, hkv, hd = 700, 4, 2, 128
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([t], [0], hq, hkv, 16, hd=hd)
    ramp = torch.linspace(0.05, 3.0, t)                  # key j is ~ ramp[j] x a common direction
    direction = torch.randn(hd, generator=torch.Generator().manual_seed(3))
    pos = torch.arange(t)
    blocks = table[0, pos // 16].long()
    kc[blocks, pos % 16] = (ramp[:, None, None] * direction[None, None, :] * 4).bfloat16().expand(t, hkv, hd)
    q[:] = (direction * 2).bfloat16()
    scale = hd ** -0.5
    check(run(q, kc, vc, cu, seq_lens, table, scale),
          A.attention_reference(q, kc, vc, cu, seq_lens, table, scale))


def test_config4_geometry_65536_tokens_on_a_tile_sample():
    """Config 4 at full length: one sequence of 65,536 tokens, 40 q / 8 kv heads,
    head 128, int8 KV. The oracle evaluates every 128th 64-query tile plus the
    first and the last (a tile = the last 64 queries of a context that ends
    with it, the chunked-prefill reading of tests/test_attn_prefill.py:31-59)."""
    t, hq, hkv, hd = 65536, 40, 8, 128
    q, kc, vc, cu, seq_lens, table = A.build_paged_kv([t], [0], hq, hkv, 16, hd=hd)
    kq, ks = A.quantize_kv(kc)
    vq, vs = A.quantize_kv(vc)
    del kc, vc
    scale = hd ** -0.5
    out = run(q, kq, vq, cu, seq_lens, table, scale, 1, -1, ks, vs)
    kx, vx = kq.float() * ks[..., None], vq.float() * vs[..., None]
    tiles = sorted(set(range(0, t // 64, 128)) | {t // 64 - 1})
    for tile in tiles:
        a, b = tile * 64, tile * 64 + 64
        ref = A.attention_reference(q[a:b], kx, vx, torch.tensor([0, 64], dtype=torch.int32),
                                    torch.tensor([b], dtype=torch.int32), table, scale)
        check(out[a:b], ref)
