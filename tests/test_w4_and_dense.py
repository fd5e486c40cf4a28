"""4-bit expert formats (MXFP4, int4) and the dense 4-/8-bit GEMMs and decoders
against the CPU oracle. Cases follow the reference's tests/test_mxfp4.py,
tests/test_moe_wna16.py, tests/test_w8a16.py and tests/test_fp8.py (same shapes
where the CPU oracle stays fast, fewer experts)."""

import pytest
import torch

import libstrix_b200 as strix  # noqa: F401  (registers torch.ops.strix)
from oracle import gemm as G
from oracle import moe as M

pytestmark = pytest.mark.gpu
DEV = "cuda"
ops = torch.ops.strix


def close_to_peak(out, ref, atol):
    out, ref = out.float().cpu(), ref.float()
    assert torch.isfinite(out).all()
    peak = ref.abs().amax().clamp_min(1e-30)
    torch.testing.assert_close(out / peak, ref / peak, rtol=0, atol=atol)


def rms_check(out, ref, tol):
    out, ref = out.float().cpu(), ref.float()
    assert torch.isfinite(out).all()
    rms = ref.pow(2).mean().sqrt().item()
    err = (out - ref).abs()
    assert bool((err <= tol * max(rms, 1e-6) + ref.abs() * 2.0 ** -8).all()), \
        f"max err {err.max().item():.3g}, rms {rms:.3g}"


# ------------------------------------------------------------------ MXFP4 dense

def mx_case(n, k, seed=0, lo=118, hi=134):
    g = torch.Generator().manual_seed(seed)
    w = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    s = torch.randint(lo, hi, (n, k // 32), generator=g, dtype=torch.uint8)
    return w, s


@pytest.mark.parametrize("n,k", [(256, 1024), (2048, 2688), (96, 5376)])
def test_mxfp4_dequant_is_byte_exact(n, k):
    w, s = mx_case(n, k)
    s[0, :3] = 0
    out = ops.mxfp4_dequant(w.to(DEV), s.to(DEV))
    assert out.dtype == torch.bfloat16 and out.shape == (n, k)
    torch.testing.assert_close(out.float().cpu(), G.mxfp4_dequant(w, s), rtol=0, atol=0)


def test_mxfp4_gemm_is_the_dequantiser_on_one_hot_rows():
    n, k = 256, 128
    w, s = mx_case(n, k, lo=120, hi=135)
    x = torch.eye(k, dtype=torch.bfloat16)
    out = ops.mxfp4_wmma_gemm(w.to(DEV), x.to(DEV), s.to(DEV), None)
    torch.testing.assert_close(out.t().float().cpu(), G.mxfp4_dequant(w, s), rtol=0, atol=0)


def test_mxfp4_zero_block_scale_is_zero():
    n, k = 64, 128
    w, _ = mx_case(n, k)
    s = torch.zeros(n, k // 32, dtype=torch.uint8)
    s[:, 1] = 127
    x0 = torch.zeros(8, k, dtype=torch.bfloat16)
    x0[:, :32] = 1.0
    x1 = torch.zeros(8, k, dtype=torch.bfloat16)
    x1[:, 32:] = 1.0
    assert torch.count_nonzero(ops.mxfp4_wmma_gemm(w.to(DEV), x0.to(DEV), s.to(DEV), None)) == 0
    assert torch.count_nonzero(ops.mxfp4_wmma_gemm(w.to(DEV), x1.to(DEV), s.to(DEV), None)) > 0


@pytest.mark.parametrize("n,k", [(256, 1024), (2048, 2688), (5376, 2688)])
@pytest.mark.parametrize("m", [1, 5, 32, 513])
def test_mxfp4_gemm_matches_dequant(n, k, m):
    w, s = mx_case(n, k)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(1)).bfloat16()
    out = ops.mxfp4_wmma_gemm(w.to(DEV), x.to(DEV), s.to(DEV), None)
    close_to_peak(out, x.float() @ G.mxfp4_dequant(w, s).t(), 1e-2)


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8])
def test_mxfp4_gemv(m):
    n, k = 1024, 2688
    w, s = mx_case(n, k)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(1)).bfloat16()
    out = ops.mxfp4_gemv(x.to(DEV), w.to(DEV), s.to(DEV))
    close_to_peak(out, x.float() @ G.mxfp4_dequant(w, s).t(), 1e-2)


@pytest.mark.parametrize("bias_dim", [1, 2])
def test_mxfp4_bias(bias_dim):
    n, k, m = 512, 1024, 33
    w, s = mx_case(n, k)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(m, k, generator=g).bfloat16()
    bias = torch.randn((n,) if bias_dim == 1 else (m, n), generator=g).bfloat16()
    out = ops.mxfp4_wmma_gemm(w.to(DEV), x.to(DEV), s.to(DEV), bias.to(DEV))
    close_to_peak(out, x.float() @ G.mxfp4_dequant(w, s).t() + bias.float(), 1e-2)


def test_mxfp4_rejects_unbuilt_shapes():
    x = torch.zeros(4, 96, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 48, dtype=torch.uint8, device=DEV)
    s = torch.zeros(8, 3, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="K must be a multiple of 128"):
        ops.mxfp4_wmma_gemm(w, x, s, None)
    x = torch.zeros(4, 128, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 64, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="scale must be uint8"):
        ops.mxfp4_wmma_gemm(w, x, w.to(torch.bfloat16), None)


# ------------------------------------------------------------- grouped 4-bit experts

E, TOP_K = 16, 4


def routing(tokens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randperm(E, generator=g)[:TOP_K] for _ in range(tokens)]).int()


def run_grouped(op, extra, a, w_dev, s_dev, b_deq, ids, gemm, activation, block_m):
    tokens = ids.size(0)
    n = b_deq.size(1)
    if gemm == "w13":
        a_topk, weights, out_cols = TOP_K, None, n // 2
    else:
        a_topk, out_cols = 1, n
        weights = torch.rand(tokens, TOP_K, generator=torch.Generator().manual_seed(5))
    sorted_ids, expert_ids, num_post = M.align(ids, block_m, E)
    c = torch.full((tokens * TOP_K, out_cols), float("nan"), dtype=torch.bfloat16, device=DEV)
    op(c, a.to(DEV), w_dev, s_dev, sorted_ids.to(DEV), expert_ids.to(DEV), num_post.to(DEV),
       None if weights is None else weights.flatten().to(DEV), a_topk, block_m, 64, gemm == "w13",
       activation, *extra)
    ref = M.grouped_reference(a, b_deq, ids, a_topk, weights)
    if gemm == "w13":
        ref = M.gate_mul(ref, activation)
    return c, ref


# gemma-4-26B-like (group 32, K tail of 64 on the down GEMM) and a group-128 model
W4_MODELS = {"gemma": (32, (1408, 2816), (2816, 704)), "qfn": (128, (1280, 2560), (2560, 640))}


@pytest.mark.parametrize("scale_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens", [1, 5, 70])
@pytest.mark.parametrize("block_m", [16, 64])
@pytest.mark.parametrize("gemm,activation", [("w13", "silu"), ("w13", "gelu_tanh"), ("w2", "silu")])
@pytest.mark.parametrize("model", ["gemma", "qfn"])
def test_moe_gemm_w4a16(model, tokens, block_m, gemm, activation, scale_dtype):
    group, w13, w2 = W4_MODELS[model]
    n, k = w13 if gemm == "w13" else w2
    g = torch.Generator().manual_seed(0)
    w_u8 = G.int4_pack(torch.randint(0, 16, (E, n, k), generator=g, dtype=torch.uint8))
    scales = (torch.rand(E, n, k // group, generator=g) * 0.02 + 0.001).to(scale_dtype)
    b = G.int4_dequant(w_u8, scales, group, exact=group % 64 == 0)
    a = torch.randn(tokens if gemm == "w13" else tokens * TOP_K, k, generator=g).bfloat16()
    c, ref = run_grouped(ops.moe_gemm_w4a16, (group,), a, w_u8.to(DEV), scales.to(DEV), b,
                         routing(tokens), gemm, activation, block_m)
    torch.testing.assert_close(c.float().cpu(), ref, rtol=2e-2, atol=2e-2)


# gpt-oss-120B-like: hidden 2880 = 22.5 x 128 (the last K block is half empty)
@pytest.mark.parametrize("tokens", [1, 7, 70])
@pytest.mark.parametrize("block_m", [16, 32, 64])
@pytest.mark.parametrize("gemm,activation", [("w13", "silu"), ("w2", "silu")])
def test_moe_gemm_mxfp4(tokens, block_m, gemm, activation):
    n, k = (5760, 2880) if gemm == "w13" else (2880, 2880)
    g = torch.Generator().manual_seed(0)
    w = torch.randint(0, 256, (E, n, k // 2), generator=g, dtype=torch.uint8)
    s = torch.randint(118, 126, (E, n, k // 32), generator=g, dtype=torch.uint8)
    s[0, :4, :2] = 0
    b = G.mxfp4_dequant(w, s)
    a = torch.randn(tokens if gemm == "w13" else tokens * TOP_K, k, generator=g).bfloat16()
    c, ref = run_grouped(ops.moe_gemm_mxfp4, (), a, w.to(DEV), s.to(DEV), b, routing(tokens), gemm,
                         activation, block_m)
    rms_check(c, ref, 2e-2)


@pytest.mark.parametrize("group", [32, 64, 128])
def test_w4a16_dense_and_dequant(group):
    """The dense int4 ops read vLLM's ExLlama word order (tests/test_w8a16.py:100-135
    of the reference): the decode is judged against the values before packing."""
    n, k = 512, 1024
    g = torch.Generator().manual_seed(group)
    q4 = torch.randint(0, 16, (n, k), generator=g, dtype=torch.uint8)
    w_x = G.int4_pack_exllama(q4)
    seq = G.int4_pack(q4)                                   # the same values, sequential order
    scales = (torch.rand(n, k // group, generator=g) * 0.02 + 0.001).bfloat16()
    x = torch.randn(40, k, generator=g).bfloat16()
    dq = ops.w4a16_dequant(w_x.to(DEV), scales.to(DEV), group)
    assert torch.equal(dq.cpu(), G.int4_dequant(seq, scales, group))
    out = ops.w4a16_wmma_gemm(x.to(DEV), w_x.view(torch.int8).to(DEV), scales.to(DEV), None, group)
    close_to_peak(out, x.float() @ G.int4_dequant(seq, scales, group, exact=True).t(), 1e-2)


def test_exllama_packing_is_a_nibble_permutation():
    q4 = torch.arange(16, dtype=torch.uint8).repeat(2).view(1, 32)
    w = G.int4_pack_exllama(q4).view(-1)
    word = int.from_bytes(bytes(w[:4].tolist()), "little")
    assert [(word >> (4 * i)) & 15 for i in range(8)] == [0, 2, 4, 6, 1, 3, 5, 7]


@pytest.mark.parametrize("n,k", [(16384, 5120), (256, 1024)])
@pytest.mark.parametrize("m", [6, 64, 300])
@pytest.mark.parametrize("group_size", [0, 128])
def test_w4a8_wmma_gemm(n, k, m, group_size):
    """tests/test_w8a16.py:74-98 of the reference: int4 (ExLlama order) x activations
    quantised to int8 per 128 group inside the op."""
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, k, generator=g).bfloat16()
    q4 = torch.randint(0, 16, (n, k), generator=g, dtype=torch.uint8)
    s = (torch.rand(n, k // group_size if group_size else 1, generator=g) * 0.05 + 0.01).bfloat16()
    full = s.float().repeat_interleave(group_size, 1) if group_size else s.float()
    w = (q4.float() - 8.0) * full
    sf = s.float().reshape(n) if group_size == 0 else s.float().t().contiguous()
    out = ops.w4a8_wmma_gemm(G.int4_pack_exllama(q4).to(DEV), x.to(DEV), sf.to(DEV))
    qa, sa = G.act_quant_group_i8(x)
    close_to_peak(out, (qa.float() * sa.repeat_interleave(128, 1)) @ w.t(), 1e-2)
    close_to_peak(out, x.float() @ w.t(), 6e-2)             # the reference's statement
    with pytest.raises(RuntimeError, match=r"\[K/32, N\]"):
        ops.w4a8_wmma_gemm(G.int4_pack_exllama(q4).to(DEV), x.to(DEV),
                           torch.ones(k // 64, n, device=DEV))


@pytest.mark.parametrize("n,k", [(16384, 5120), (256, 1024)])
@pytest.mark.parametrize("m", [6, 300])
def test_w4a8_wmma_gemm_scales_per_32(n, k, m):
    """group_size 32 of tests/test_w8a16.py:74-98: scales [K/32, N]. Served without
    quantising the activations, so it meets the reference's bound against the
    unquantised product with room to spare."""
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, k, generator=g).bfloat16()
    q4 = torch.randint(0, 16, (n, k), generator=g, dtype=torch.uint8)
    s = (torch.rand(n, k // 32, generator=g) * 0.05 + 0.01).bfloat16()
    w = (q4.float() - 8.0) * s.float().repeat_interleave(32, 1)
    out = ops.w4a8_wmma_gemm(G.int4_pack_exllama(q4).to(DEV), x.to(DEV), s.float().t().contiguous().to(DEV))
    close_to_peak(out, x.float() @ w.t(), 1e-2)


# ------------------------------------------------------------------ dense 8-bit

@pytest.mark.parametrize("n,k", [(16384, 5120), (5120, 17408), (256, 1024)])
@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("group_size", [0, 32, 64, 128])
def test_w8a16_skinny(n, k, m, group_size):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(m, k, generator=g).bfloat16()
    w_u8 = torch.randint(0, 256, (n, k), generator=g, dtype=torch.uint8)
    s = (torch.rand(n, k // group_size if group_size else 1, generator=g) * 0.01).bfloat16()
    if group_size == 0:
        s = s.reshape(n)
    out = ops.w8a16_skinny_gemm(w_u8.to(DEV), x.to(DEV), s.to(DEV), None, 40, group_size)
    close_to_peak(out, G.w8a16_reference(x, w_u8, s, group_size), 3e-2)


def test_w8a16_skinny_rejects_more_than_8_rows():
    x = torch.randn(9, 256, device=DEV, dtype=torch.bfloat16)
    w_u8 = torch.randint(0, 256, (128, 256), device=DEV, dtype=torch.uint8)
    s = torch.full((128,), 0.01, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="1-8 rows"):
        ops.w8a16_skinny_gemm(w_u8, x, s, None, 40, 0)


def fp8_case(n, k, scheme, seed=0):
    g = torch.Generator().manual_seed(seed)
    wf = torch.randn(n, k, generator=g) * 0.02
    if scheme == "block":
        nb, kb = (n + 127) // 128, k // 128
        pad = torch.zeros(nb * 128, k)
        pad[:n] = wf
        amax = pad.view(nb, 128, kb, 128).abs().amax((1, 3)).clamp_min(1e-12)
        scales = amax / 448.0
        full = scales.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)
    else:
        scales = wf.abs().amax(1).clamp_min(1e-12) / 448.0
        full = scales[:, None]
    return (wf / full).to(torch.float8_e4m3fn), scales.float()


@pytest.mark.parametrize("scheme", ["block", "channel"])
@pytest.mark.parametrize("n,k", [(2048, 2048), (1024 + 64, 1024)])
def test_fp8_dequant_and_gemms(scheme, n, k):
    w, scales = fp8_case(n, k, scheme)
    ref_w = G.fp8_dequant(w, scales)
    dq = ops.fp8_dequant(w.to(DEV), scales.to(DEV))
    assert torch.equal(dq.cpu(), ref_w.to(torch.bfloat16))
    g = torch.Generator().manual_seed(3)
    for m in (1, 8, 70):
        x = torch.randn(m, k, generator=g).bfloat16()
        ref = x.float() @ ref_w.to(torch.bfloat16).float().t()
        if m <= 8:
            out = ops.fp8_skinny_gemm(w.to(DEV), x.to(DEV), scales.to(DEV), None, 40)
            close_to_peak(out, ref, 1e-2)
        out = ops.fp8_wmma_gemm(w.to(DEV), x.to(DEV), scales.to(DEV))
        close_to_peak(out, ref, 1e-2)
        out = ops.fp8_wmma_gemm_raw(w.to(DEV), x.half().to(DEV), scales.to(DEV))
        close_to_peak(out, x.half().float() @ ref_w.t(), 1e-2)


# ------------------------------------------------------------ int8 activations

@pytest.mark.parametrize("scale_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens", [1, 37, 130])
@pytest.mark.parametrize("block_m", [16, 64, 128])
@pytest.mark.parametrize("gemm,activation", [("w13", "silu"), ("w13", "gelu_tanh"), ("w2", "silu")])
def test_moe_gemm_w4a8(tokens, block_m, gemm, activation, scale_dtype):
    """The oracle consumes the dequantised int8 activations and the exact weights
    (tests/test_moe_w4a8.py:78-85)."""
    n, k = (1280, 2560) if gemm == "w13" else (2560, 640)
    g = torch.Generator().manual_seed(0)
    q4 = torch.randint(0, 16, (E, n, k), generator=g, dtype=torch.uint8)
    w_u8 = G.int4_pack(q4)
    scales = (torch.rand(E, n, k // 128, generator=g) * 0.02 + 0.001).to(scale_dtype)
    b = (q4.float() - 8) * scales.float().repeat_interleave(128, dim=-1)
    a = torch.randn(tokens if gemm == "w13" else tokens * TOP_K, k, generator=g).bfloat16()
    qa, sa = M.act_quant_i8(a)
    a_deq = qa.float() * sa.repeat_interleave(128, dim=-1)
    ids = routing(tokens)
    if gemm == "w13":
        a_topk, weights, out_cols = TOP_K, None, n // 2
    else:
        a_topk, weights, out_cols = 1, torch.rand(tokens, TOP_K, generator=g), n
    sorted_ids, expert_ids, num_post = M.align(ids, block_m, E)
    c = torch.full((tokens * TOP_K, out_cols), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.moe_gemm_w4a8(c, qa.to(DEV), sa.to(DEV), w_u8.to(DEV), scales.to(DEV), sorted_ids.to(DEV),
                      expert_ids.to(DEV), num_post.to(DEV),
                      None if weights is None else weights.flatten().to(DEV), a_topk, block_m, 64,
                      gemm == "w13", activation)
    ref = M.grouped_reference(a_deq, b, ids, a_topk, weights)
    if gemm == "w13":
        ref = M.gate_mul(ref, activation)
    torch.testing.assert_close(c.float().cpu(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("n,k", [(2048, 2048), (1024, 2048), (256, 4096)])
@pytest.mark.parametrize("m", [6, 64, 300])
@pytest.mark.parametrize("scale_form", ["channel", "group_major", "row_major"])
def test_w8a8_wmma_gemm_reference_schema(n, k, m, scale_form):
    """tests/test_w8a8_int8.py:84-104 (per-channel) and tests/test_w8a16.py:34-42
    (per-group scales, group-major)."""
    g = torch.Generator().manual_seed(0)
    w_i8 = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    w_u8 = (w_i8.to(torch.int16) + 128).to(torch.uint8)
    x = torch.randn(m, k, generator=g).bfloat16()
    if scale_form == "channel":
        s = torch.rand(n, generator=g) * 0.01 + 1e-4
        full, arg = s.reshape(n, 1), s
    else:
        s = torch.rand(n, k // 128, generator=g) * 0.01 + 1e-4
        full = s.repeat_interleave(128, 1)
        arg = s.t().contiguous() if scale_form == "group_major" else s
    out = ops.w8a8_wmma_gemm(w_u8.to(DEV), x.to(DEV), arg.to(DEV))
    # the op's own arithmetic, exactly: quantise, int sums per group, fp32 fold
    q, sg = G.act_quant_group_i8(x)
    exact = (q.float() * sg.repeat_interleave(128, 1)) @ (w_i8.float() * full).t()
    close_to_peak(out, exact, 1e-2)
    # and the reference's looser statement against unquantised activations
    close_to_peak(out, x.float() @ (w_i8.float() * full).t(), 6e-2)


# ------------------------------------------------------- bench-only *_cfg ops

@pytest.mark.parametrize("cfg", [0, 1, 2])
@pytest.mark.parametrize("m", [5, 130])
def test_cfg_ops_match_the_production_ops(cfg, m):
    """The four tile-sweep ops of the reference's schema (csrc/torch_ops.cpp:258-292):
    the same GEMM pinned to one token tile, against the oracle and against the op that
    picks the tile by row count."""
    from libstrix_b200 import torch_ops

    n, k = 1024, 1024
    g = torch.Generator().manual_seed(cfg)
    x = torch.randn(m, k, generator=g).bfloat16()
    w, s = mx_case(n, k)
    out = ops.mxfp4_wmma_gemm_cfg(w.to(DEV), x.to(DEV), s.to(DEV), None, cfg)
    close_to_peak(out, x.float() @ G.mxfp4_dequant(w, s).t(), 1e-2)
    close_to_peak(out, ops.mxfp4_wmma_gemm(w.to(DEV), x.to(DEV), s.to(DEV), None).float().cpu(), 1e-2)
    for scheme in ("block", "channel"):
        w8, sc = fp8_case(n, k, scheme)
        ref_w = G.fp8_dequant(w8, sc)
        out = ops.fp8_wmma_gemm_cfg(w8.to(DEV), x.to(DEV), sc.to(DEV), cfg)
        close_to_peak(out, x.float() @ ref_w.to(torch.bfloat16).float().t(), 1e-2)
        out = ops.fp8_wmma_gemm_raw_cfg(w8.to(DEV), x.half().to(DEV), sc.to(DEV), cfg)
        close_to_peak(out, x.half().float() @ ref_w.t(), 1e-2)
    w_i8 = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    w_u8 = (w_i8.to(torch.int16) + 128).to(torch.uint8)
    sw = torch.rand(n, generator=g) * 0.01 + 1e-4
    out = ops.w8a8_wmma_gemm_cfg(w_u8.to(DEV), x.to(DEV), sw.to(DEV), cfg)
    q, sg = G.act_quant_group_i8(x)
    close_to_peak(out, (q.float() * sg.repeat_interleave(128, 1)) @ (w_i8.float() * sw[:, None]).t(), 1e-2)
    with pytest.raises(RuntimeError, match="cfg must be in"):
        ops.w8a8_wmma_gemm_cfg(w_u8.to(DEV), x.to(DEV), sw.to(DEV), len(torch_ops.TILE_CFGS))


# ------------------------------------------------- MXFP4 on tcgen05 (sorted layout)

@pytest.mark.parametrize("tokens", [1, 40, 300])
@pytest.mark.parametrize("gemm,activation,n,k", [("w13", "silu", 5760, 2880), ("w13", "gelu_tanh", 512, 256),
                                                 ("w2", "silu", 2880, 2880), ("w2", "silu", 256, 128)])
def test_moe_gemm_mxfp4_sorted(tokens, gemm, activation, n, k):
    _mxfp4_sorted_case(tokens, gemm, activation, n, k)


@pytest.mark.parametrize("gemm,activation,n,k", [("w13", "silu", 512, 256), ("w2", "silu", 256, 128),
                                                 ("w13", "silu", 5760, 2880)])
def test_moe_gemm_mxfp4_sorted_units_of_two_m_blocks(gemm, activation, n, k):
    """1200 tokens over 16 experts: about 300 rows per expert = a pair of
    m-blocks sharing each decoded weight tile plus a single one."""
    _mxfp4_sorted_case(1200, gemm, activation, n, k)


def _mxfp4_sorted_case(tokens, gemm, activation, n, k):
    """The tensor-core kernel (m-blocks of 128 tokens, activations in sorted order)
    against the gathered oracle; the permute kernel bit for bit."""
    import libstrix_b200 as strix
    from libstrix_b200 import _lib

    g = torch.Generator().manual_seed(0)
    w = torch.randint(0, 256, (E, n, k // 2), generator=g, dtype=torch.uint8)
    s = torch.randint(118, 126, (E, n, k // 32), generator=g, dtype=torch.uint8)
    s[0, :4, :2] = 0
    b = G.mxfp4_dequant(w, s)
    ids = routing(tokens)
    slots = tokens * TOP_K
    sorted_ids, expert_ids, num_post, slot_pos = strix.moe.align_with_positions(ids.to(DEV), 128, E)
    cap = sorted_ids.numel()
    pos = sorted_ids.cpu().long()
    live = pos < slots
    n_post = int(num_post.item())
    if gemm == "w13":
        a = torch.randn(tokens, k, generator=g).bfloat16()
        a_sorted = torch.full((cap, k), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.moe_permute_bf16(a.to(DEV), a_sorted, slot_pos, sorted_ids, num_post, TOP_K)
        got = a_sorted.cpu()
        assert torch.equal(got[live].view(torch.int16), a[pos[live] // TOP_K].view(torch.int16))
        pad = (~live) & (torch.arange(cap) < n_post)
        assert not got[pad].view(torch.int16).any()
        a_topk, weights = TOP_K, None
    else:
        a = torch.randn(slots, k, generator=g).bfloat16()
        a_sorted = torch.zeros(cap, k, dtype=torch.bfloat16)
        a_sorted[live] = a[pos[live]]
        a_sorted = a_sorted.to(DEV)
        a_topk, weights = 1, torch.rand(tokens, TOP_K, generator=g)
    c_sorted = gemm == "w13"
    out_cols = n // 2 if gemm == "w13" else n
    c = torch.full((cap if c_sorted else slots, out_cols), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.moe_gemm_mxfp4_sorted(c, a_sorted, w.to(DEV), s.to(DEV), sorted_ids, expert_ids, num_post,
                              None if weights is None else weights.flatten().to(DEV), slots, 128,
                              gemm == "w13", activation, c_sorted)
    torch.cuda.synchronize()
    import ctypes
    flag = ctypes.c_int32(-1)
    assert _lib.load().strix_umma_status(ctypes.byref(flag)) == 0 and flag.value == 0
    ref = M.grouped_reference(a, b, ids, a_topk, weights)
    if gemm == "w13":
        ref = M.gate_mul(ref, activation)
    out = c.float().cpu()
    if c_sorted:
        by_slot = torch.full((slots, out_cols), float("nan"))
        by_slot[pos[live]] = out[live]
        out = by_slot
    rms_check(out, ref, 2e-2)
