"""Parity of the MoE path (router, permutation, quantisers, grouped expert GEMMs
with the fused gate, combine) with the CPU oracle, through torch.ops.strix /
the C-ABI. GEMM cases mirror the reference's tests/test_moe_gemm.py,
test_moe_fp8.py, test_moe_fp8_raw.py and test_moe_w8a16.py (same shapes per
expert, fewer experts so the CPU oracle stays fast)."""

from pathlib import Path

import pytest
import torch

import libstrix_b200 as strix
from libstrix_b200.workloads import moe_fp8_layer
from oracle import moe as M

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"
DEV = "cuda"
E, TOP_K = 32, 8


@pytest.fixture(autouse=True)
def tcgen05_kernels_met_their_waits():
    """Every bounded wait inside the tcgen05 kernels must have been met: a
    timed-out wait makes a kernel give up (wrong output, but no hang)."""
    import ctypes

    from libstrix_b200 import _lib

    yield
    flag = ctypes.c_int32(-1)
    assert _lib.load().strix_umma_status(ctypes.byref(flag)) == 0 and flag.value == 0


def rms_check(out, ref, tol):
    """|err| <= tol x RMS(ref), widened per element by the bf16 output quantum."""
    out, ref = out.float().cpu(), ref.float()
    assert torch.isfinite(out).all()
    rms = ref.pow(2).mean().sqrt().item()
    bound = tol * max(rms, 1e-6) + ref.abs() * 2.0 ** -8
    err = (out - ref).abs()
    assert bool((err <= bound).all()), f"max err {err.max().item():.3g}, rms {rms:.3g}, tol {tol}"


def routing(tokens, e=E, top_k=TOP_K, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randperm(e, generator=g)[:top_k] for _ in range(tokens)]).int()


# ------------------------------------------------------------------ router

@pytest.mark.parametrize("tokens,experts,top_k", [(1, 128, 8), (256, 128, 8), (77, 64, 4),
                                                  (33, 256, 8), (5, 8, 2), (300, 128, 4)])
def test_router_matches_oracle(tokens, experts, top_k):
    torch.manual_seed(tokens)
    logits = torch.randn(tokens, experts)
    ids_ref, w_ref = M.router(logits, top_k)
    w, ids = strix.moe.route(logits.to(DEV), top_k)
    ids, w = ids.cpu(), w.cpu()
    # bit-exact ids except where the oracle's k-th and (k+1)-th probabilities tie
    p = torch.softmax(logits, -1).sort(-1, descending=True).values
    tied = p[:, top_k - 1] == p[:, min(top_k, experts - 1)]
    assert torch.equal(ids[~tied], ids_ref[~tied])
    torch.testing.assert_close(w[~tied], w_ref[~tied], rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(w.sum(-1), torch.ones(tokens), rtol=1e-5, atol=1e-6)


def test_router_ties_take_the_lower_index():
    logits = torch.zeros(3, 128)
    w, ids = strix.moe.route(logits.to(DEV), 8)
    assert torch.equal(ids.cpu(), torch.arange(8, dtype=torch.int32).expand(3, 8))
    torch.testing.assert_close(w.cpu(), torch.full((3, 8), 0.125))


# ------------------------------------------------------------------- align

@pytest.mark.parametrize("tokens,experts,top_k", [(1, 128, 8), (5, 8, 3), (256, 128, 8),
                                                  (700, 256, 8), (4096, 128, 4), (0, 16, 2)])
@pytest.mark.parametrize("block_m", [16, 64, 128])
def test_align_is_bit_exact(tokens, experts, top_k, block_m):
    ids = routing(tokens, experts, top_k, seed=tokens + block_m) if tokens else \
        torch.zeros(0, top_k, dtype=torch.int32)
    s_ref, e_ref, n_ref = M.align(ids, block_m, experts)
    s, e, n = strix.moe.align(ids.to(DEV), block_m, experts)
    total = int(n_ref)
    assert int(n.cpu()) == total
    assert torch.equal(s.cpu()[:total], s_ref[:total])
    assert torch.equal(e.cpu()[: total // block_m], e_ref[: total // block_m])
    assert bool((s.cpu()[total:] == ids.numel()).all()) and bool((e.cpu()[total // block_m:] == -1).all())


@pytest.mark.parametrize("numel,experts,block_m", [(4097, 8, 16), (5000, 128, 128), (32768, 128, 128),
                                                   (20001, 1000, 32), (9000, 3, 1), (6000, 2000, 16)])
def test_two_level_align_equals_the_one_kernel_form(numel, experts, block_m):
    """Above 4096 slots the permutation is built by two launches over a scratch
    (one CTA per 1024 slots): every output - sorted ids, block experts, padded total,
    inverse positions, counts - equals the one-kernel form and the oracle, with ids
    that name no local expert (-1, >= experts) sprinkled in. More than 1024 experts
    fall back to the one-kernel form inside the same call."""
    from libstrix_b200 import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(numel)
    ids = torch.randint(0, experts, (numel,), generator=g, dtype=torch.int32)
    ids[torch.rand(numel, generator=g) < 0.1] = -1
    ids[torch.rand(numel, generator=g) < 0.05] = experts + 3
    cap = lib.strix_moe_align_capacity(numel, experts, block_m)
    d = ids.to(DEV)

    def run(two_level):
        out = dict(s=torch.full((cap,), -7, dtype=torch.int32, device=DEV),
                   e=torch.full((cap // block_m,), -7, dtype=torch.int32, device=DEV),
                   n=torch.full((1,), -7, dtype=torch.int32, device=DEV),
                   pos=torch.full((numel,), -7, dtype=torch.int32, device=DEV),
                   cnt=torch.full((experts,), -7, dtype=torch.int32, device=DEV))
        nbytes = lib.strix_moe_align_scratch_bytes(numel, experts)
        scratch = torch.full((nbytes // 4,), 0x7f7f7f7f, dtype=torch.int32, device=DEV)
        if two_level:
            _lib.call("strix_moe_align_scratch", d.data_ptr(), out["s"].data_ptr(), out["e"].data_ptr(),
                      out["n"].data_ptr(), out["pos"].data_ptr(), out["cnt"].data_ptr(), scratch.data_ptr(),
                      nbytes, numel, experts, block_m, cap, cap // block_m,
                      torch.cuda.current_stream().cuda_stream)
        else:
            _lib.call("strix_moe_align_counts", d.data_ptr(), out["s"].data_ptr(), out["e"].data_ptr(),
                      out["n"].data_ptr(), out["pos"].data_ptr(), out["cnt"].data_ptr(), numel, experts,
                      block_m, cap, cap // block_m, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        return {k: v.cpu() for k, v in out.items()}

    a, b = run(True), run(False)
    for k in a:
        assert torch.equal(a[k], b[k]), k
    s_ref, e_ref, n_ref = M.align(ids.view(-1, 1), block_m, experts)
    total = int(n_ref)
    assert int(a["n"]) == total and torch.equal(a["s"][:total], s_ref[:total])
    assert torch.equal(a["e"][: total // block_m], e_ref[: total // block_m])
    valid = (ids >= 0) & (ids < experts)
    assert bool((a["pos"][~valid] == -1).all())
    assert torch.equal(a["s"][a["pos"][valid].long()].long(), torch.arange(numel)[valid])
    assert torch.equal(a["cnt"].long(), torch.bincount(ids[valid].long(), minlength=experts))


def test_align_golden_and_foreign_ids():
    for c in torch.load(GOLDEN / "moe.pt")["align"]:
        s, e, n = strix.moe.align(c["topk_ids"].int().to(DEV), c["block_m"], c["experts"])
        total = int(c["num_post"])
        assert int(n.cpu()) == total and torch.equal(s.cpu()[:total], c["sorted_ids"][:total])
        assert torch.equal(e.cpu()[: total // c["block_m"]], c["expert_ids"][: total // c["block_m"]])
    # ids outside [0, experts) (another rank's experts) are not placed anywhere
    ids = torch.tensor([[0, 5], [-1, 1], [7, 9]], dtype=torch.int32)
    s, e, n = strix.moe.align(ids.to(DEV), 4, 4)
    assert int(n.cpu()) == 8 and s.cpu()[:8].tolist() == [0, 6, 6, 6, 3, 6, 6, 6]
    assert e.cpu()[:2].tolist() == [0, 1]


# -------------------------------------------------------------- quantisers

def test_act_quant_fp8_is_bit_exact():
    torch.manual_seed(0)
    x = (torch.randn(37, 640) * 3).bfloat16()
    x[5, 128:256] = 0
    x[7, :128] = 1e-30  # denormal-scale group
    q_ref, s_ref = M.act_quant_fp8(x)
    q, s = strix.moe.act_quant_fp8(x.to(DEV))
    torch.testing.assert_close(s.cpu(), s_ref, rtol=0, atol=0)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))


def test_act_quant_i8_matches_reference_rule():
    torch.manual_seed(0)
    x = (torch.randn(37, 640) * 3).bfloat16()
    x[5, 128:256] = 0
    q_ref, s_ref = M.act_quant_i8(x)
    q = torch.empty(x.shape, dtype=torch.int8, device=DEV)
    sa = torch.empty(37, 5, dtype=torch.float32, device=DEV)
    torch.ops.strix.moe_act_quant_i8(x.to(DEV), q, sa)
    torch.testing.assert_close(sa.cpu(), s_ref, rtol=1e-6, atol=0)
    diff = (q.cpu().float() - q_ref.float()).abs()   # x * (1/s) vs x / s on .5 ties
    assert diff.max() <= 1 and (diff > 0).float().mean() < 2e-3


def test_moe_sum():
    torch.manual_seed(0)
    c3 = torch.randn(50, 8, 256).bfloat16()
    out = torch.empty(50, 256, dtype=torch.bfloat16, device=DEV)
    torch.ops.strix.moe_sum(c3.to(DEV), out)
    rms_check(out, M.moe_sum(c3), 5e-3)


# -------------------------------------------------------------------- GEMMs

def run_gemm(op, a, w_dev, scales_dev, b_deq, ids, gemm, activation, block_m, *, sa=None,
             a_deq=None, out_dtype=torch.bfloat16, tol=2e-2, rel_tol=None):
    tokens = ids.size(0)
    n = b_deq.size(1)
    if gemm == "w13":
        a_topk, weights, out_cols = TOP_K, None, n // 2
    else:
        a_topk, out_cols = 1, n
        weights = torch.rand(tokens, TOP_K, generator=torch.Generator().manual_seed(1))
    sorted_ids, expert_ids, num_post = M.align(ids, block_m, b_deq.size(0))
    c = torch.full((tokens * TOP_K, out_cols), float("nan"), dtype=out_dtype, device=DEV)
    args = [c, a.to(DEV)] + ([sa.to(DEV)] if sa is not None else []) + [w_dev]
    if scales_dev is not None:
        args.append(scales_dev)
    args += [sorted_ids.to(DEV), expert_ids.to(DEV), num_post.to(DEV),
             None if weights is None else weights.flatten().to(DEV), a_topk, block_m, 64,
             gemm == "w13", activation]
    op(*args)
    ref = M.grouped_reference(a if a_deq is None else a_deq, b_deq, ids, a_topk, weights)
    if gemm == "w13":
        ref = M.gate_mul(ref, activation)
    out = c.float().cpu()
    assert torch.isfinite(out).all(), "a valid row was left unwritten"
    if rel_tol is not None:
        peak = ref.abs().max()
        torch.testing.assert_close(out / peak, ref / peak, rtol=0, atol=rel_tol)
    else:
        torch.testing.assert_close(out, ref, rtol=tol, atol=tol)
    return out, ref


def shapes(gemm):
    return (1024, 2048) if gemm == "w13" else (2048, 512)


@pytest.mark.parametrize("tokens", [1, 5, 64, 300])
@pytest.mark.parametrize("block_m", [16, 64, 128])
@pytest.mark.parametrize("gemm,activation", [("w13", "silu"), ("w13", "gelu_tanh"), ("w2", "silu")])
def test_moe_gemm_bf16(tokens, block_m, gemm, activation):
    n, k = shapes(gemm)
    g = torch.Generator().manual_seed(0)
    b = (torch.randn(E, n, k, generator=g) / k ** 0.5).bfloat16()
    a = torch.randn(tokens if gemm == "w13" else tokens * TOP_K, k, generator=g).bfloat16()
    run_gemm(torch.ops.strix.moe_gemm_bf16, a, b.to(DEV), None, b, routing(tokens), gemm,
             activation, block_m)


@pytest.mark.parametrize("scheme", ["block", "channel"])
@pytest.mark.parametrize("tokens", [1, 5, 40])
@pytest.mark.parametrize("block_m", [16, 64, 128])
@pytest.mark.parametrize("gemm,activation", [("w13", "silu"), ("w13", "gelu_tanh"), ("w2", "silu")])
def test_moe_gemm_fp8(tokens, block_m, gemm, activation, scheme):
    n, k = shapes(gemm)
    w, scales, b = M.make_fp8_weights(E, n, k, scheme)
    g = torch.Generator().manual_seed(0)
    a = torch.randn(tokens if gemm == "w13" else tokens * TOP_K, k, generator=g).bfloat16()
    run_gemm(torch.ops.strix.moe_gemm_fp8, a, w.to(DEV), scales.to(DEV), b, routing(tokens), gemm,
             activation, block_m)


@pytest.mark.parametrize("scheme", ["block", "channel"])
@pytest.mark.parametrize("tokens", [1, 40])
@pytest.mark.parametrize("block_m", [16, 32, 128])
@pytest.mark.parametrize("gemm,activation", [("w13", "silu"), ("w13", "gelu_tanh"), ("w2", "silu")])
def test_moe_gemm_fp8_raw(tokens, block_m, gemm, activation, scheme):
    """fp16 activations, exact weights: tolerance relative to the output's peak
    (2e-3 for fp16 outputs, 1e-2 for bf16), tests/test_moe_fp8_raw.py:83-91."""
    n, k = shapes(gemm)
    w, scales, b = M.make_fp8_weights(E, n, k, scheme, keep_fp32=True)
    g = torch.Generator().manual_seed(0)
    a = torch.randn(tokens if gemm == "w13" else tokens * TOP_K, k, generator=g).half()
    fp16_out = gemm == "w13"
    run_gemm(torch.ops.strix.moe_gemm_fp8_raw, a, w.to(DEV), scales.to(DEV), b, routing(tokens),
             gemm, activation, block_m, out_dtype=torch.float16 if fp16_out else torch.bfloat16,
             rel_tol=2e-3 if fp16_out else 1e-2)


def test_fp8_all_finite_codes_pass_through_exactly():
    """Every finite e4m3 code as a weight, one-hot activations: the GEMM becomes
    the dequantiser (tests/test_moe_fp8_raw.py:94-115)."""
    codes = torch.tensor([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=torch.uint8)
    n, k = 256, 128
    wb = torch.zeros(1, n, k, dtype=torch.uint8)
    wb[0, :, :] = codes[torch.arange(n * k) % codes.numel()].view(n, k)
    w = wb.view(torch.float8_e4m3fn)
    scales = torch.ones(1, n)
    a = torch.eye(k).half()          # token t selects column t of W
    ids = torch.zeros(k, 1, dtype=torch.int32)
    sorted_ids, expert_ids, num_post = M.align(ids, 64, 1)
    c = torch.full((k, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    torch.ops.strix.moe_gemm_fp8_raw(c, a.to(DEV), w.to(DEV), scales.to(DEV), sorted_ids.to(DEV),
                                     expert_ids.to(DEV), num_post.to(DEV), None, 1, 64, 64, False,
                                     "silu")
    assert torch.equal(c.float().cpu(), w[0].float().t())


@pytest.mark.parametrize("tokens", [1, 40])
@pytest.mark.parametrize("block_m", [16, 64])
@pytest.mark.parametrize("gemm,activation", [("w13", "silu"), ("w2", "silu")])
@pytest.mark.parametrize("scale_dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_moe_gemm_w8a16(tokens, block_m, gemm, activation, scale_dtype):
    n, k = shapes(gemm)
    g = torch.Generator().manual_seed(0)
    w = torch.randint(-128, 128, (E, n, k), generator=g, dtype=torch.int8)
    scales = (torch.rand(E, n, generator=g) * 0.02 + 0.001).to(scale_dtype)
    # dequantised the long way and rounded to bf16, as tests/test_moe_w8a16.py:71
    b = (w.float() * scales.float()[..., None]).to(torch.bfloat16)
    a = torch.randn(tokens if gemm == "w13" else tokens * TOP_K, k, generator=g).bfloat16()
    run_gemm(torch.ops.strix.moe_gemm_w8a16, a, w.to(DEV), scales.to(DEV), b, routing(tokens),
             gemm, activation, block_m)


@pytest.mark.parametrize("scheme", ["block", "channel"])
@pytest.mark.parametrize("tokens", [1, 5, 40, 300])
@pytest.mark.parametrize("block_m", [16, 32, 64, 128])
@pytest.mark.parametrize("gemm,activation", [("w13", "silu"), ("w13", "gelu_tanh"), ("w2", "silu")])
def test_moe_gemm_fp8_w8a8(tokens, block_m, gemm, activation, scheme):
    """The oracle consumes the kernel path's own quantised activations
    (dequantised), the convention of tests/test_moe_w4a8.py:78-80. Gathered
    form (token rows fetched by slot id inside the GEMM)."""
    n, k = shapes(gemm)
    w, scales, _ = M.make_fp8_weights(E, n, k, scheme)
    full = scales.repeat_interleave(128, 1).repeat_interleave(128, 2) if scheme == "block" \
        else scales[..., None]
    b = w.float() * full
    g = torch.Generator().manual_seed(0)
    a = torch.randn(tokens if gemm == "w13" else tokens * TOP_K, k, generator=g).bfloat16()
    qa, sa = M.act_quant_fp8(a)
    out, ref = run_gemm(torch.ops.strix.moe_gemm_fp8_w8a8, qa, w.to(DEV), scales.to(DEV), b,
                        routing(tokens), gemm, activation, block_m, sa=sa,
                        a_deq=M.dequant_act(qa, sa))
    rms_check(out, ref, 2e-2)


@pytest.mark.parametrize("scheme", ["block", "channel"])
@pytest.mark.parametrize("tokens", [1, 5, 40, 300])
@pytest.mark.parametrize("block_m", [16, 32, 64, 128])
@pytest.mark.parametrize("gemm,activation", [("w13", "silu"), ("w13", "gelu_tanh"), ("w2", "silu")])
def test_moe_gemm_fp8_sorted(tokens, block_m, gemm, activation, scheme):
    """The tcgen05 kernel over activations in sorted order: the quantiser
    permutes (w13) or keeps (w2) the rows, the GEMM writes sorted rows under the
    gate and slot rows otherwise; both against the gathered oracle."""
    n, k = shapes(gemm)
    w, scales, _ = M.make_fp8_weights(E, n, k, scheme)
    full = scales.repeat_interleave(128, 1).repeat_interleave(128, 2) if scheme == "block" \
        else scales[..., None]
    b = w.float() * full
    g = torch.Generator().manual_seed(0)
    ids = routing(tokens)
    slots = tokens * TOP_K
    sorted_ids, expert_ids, num_post = (t.to(DEV) for t in M.align(ids, block_m, E))
    cap = sorted_ids.numel()
    qs = torch.empty(cap, k, dtype=torch.float8_e4m3fn, device=DEV)
    ss = torch.empty(cap, k // 128, dtype=torch.float32, device=DEV)
    pos = sorted_ids.cpu().long()
    live = pos < slots
    if gemm == "w13":
        a = torch.randn(tokens, k, generator=g).bfloat16()
        torch.ops.strix.moe_act_quant_fp8_sorted(a.to(DEV), qs, ss, sorted_ids, num_post, TOP_K, slots)
        a_topk, weights = TOP_K, None
    else:
        # the intermediate arrives in sorted order: row p belongs to slot sorted_ids[p]
        a = torch.randn(slots, k, generator=g).bfloat16()
        a_sorted = torch.zeros(cap, k, dtype=torch.bfloat16)
        a_sorted[live] = a[pos[live]]
        torch.ops.strix.moe_act_quant_fp8_sorted(a_sorted.to(DEV), qs, ss, None, num_post, 1, slots)
        a_topk, weights = 1, torch.rand(tokens, TOP_K, generator=g)
    # the quantiser itself: bit-exact against the oracle's, row by row
    qa_ref, sa_ref = M.act_quant_fp8(a)
    src = pos[live] // a_topk if gemm == "w13" else pos[live]
    assert torch.equal(qs.cpu()[live].view(torch.uint8), qa_ref[src].view(torch.uint8))
    assert torch.equal(ss.cpu()[live], sa_ref[src])
    n_post = int(num_post.item())
    pad = (~live) & (torch.arange(cap) < n_post)
    assert not qs.cpu()[pad].view(torch.uint8).any()

    c_sorted = gemm == "w13"
    out_cols = n // 2 if gemm == "w13" else n
    c = torch.full((cap if c_sorted else slots, out_cols), float("nan"), dtype=torch.bfloat16,
                   device=DEV)
    torch.ops.strix.moe_gemm_fp8_sorted(c, qs, ss, w.to(DEV), scales.to(DEV), sorted_ids, expert_ids,
                                        num_post, None if weights is None else weights.flatten().to(DEV),
                                        slots, block_m, gemm == "w13", activation, c_sorted)
    ref = M.grouped_reference(M.dequant_act(qa_ref, sa_ref), b, ids, a_topk, weights)
    if gemm == "w13":
        ref = M.gate_mul(ref, activation)
    out = c.float().cpu()
    if c_sorted:
        assert not out[pad].any(), "padding rows of a processed m-block must come out as zeros"
        by_slot = torch.full((slots, out_cols), float("nan"))
        by_slot[pos[live]] = out[live]
        out = by_slot
    rms_check(out, ref, 2e-2)


def test_moe_gemm_fp8_sorted_rejects_uncovered_geometry():
    w = torch.zeros(2, 256, 128, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.ones(2, 256, device=DEV)
    ids = torch.zeros(24, dtype=torch.int32, device=DEV)
    q = torch.zeros(24, 128, dtype=torch.float8_e4m3fn, device=DEV)
    sa = torch.ones(24, 1, device=DEV)
    c = torch.zeros(24, 256, dtype=torch.bfloat16, device=DEV)
    one = torch.ones(1, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="geometry not covered"):
        torch.ops.strix.moe_gemm_fp8_sorted(c, q, sa, w, s, ids, one, one, None, 24, 24)


def test_moe_gemm_golden_fixtures():
    gold = torch.load(GOLDEN / "moe.pt")
    for c in gold["fp8"]:
        w = c["w"].view(torch.float8_e4m3fn)
        ids = c["topk_ids"].int()
        op = torch.ops.strix.moe_gemm_fp8 if c["kind"] == "plain" else torch.ops.strix.moe_gemm_fp8_raw
        for act in ("silu", "gelu"):
            sorted_ids, expert_ids, num_post = M.align(ids, 16, 2)
            fp16 = c["kind"] == "raw"
            out = torch.full((12, 128), float("nan"), dtype=torch.float16 if fp16 else torch.bfloat16,
                             device=DEV)
            op(out, c["a"].to(DEV), w.to(DEV), c["scales"].to(DEV), sorted_ids.to(DEV),
               expert_ids.to(DEV), num_post.to(DEV), None, 2, 16, 64, True,
               "silu" if act == "silu" else "gelu_tanh")
            torch.testing.assert_close(out.float().cpu(), c[act], rtol=2e-2, atol=2e-2)


def test_skipped_blocks_and_padding_write_nothing():
    """expert_ids < 0 skips a block (the expert-parallel hook), padded ids write
    no row, rows past num_post_padded are ignored."""
    n, k = 256, 128
    g = torch.Generator().manual_seed(0)
    b = (torch.randn(4, n, k, generator=g) / k ** 0.5).bfloat16()
    a = torch.randn(6, k, generator=g).bfloat16()
    ids = torch.tensor([[0], [1], [1], [2], [3], [3]], dtype=torch.int32)
    sorted_ids, expert_ids, num_post = M.align(ids, 16, 4)
    expert_ids[1] = -1                     # drop expert 1's block
    c = torch.full((6, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    torch.ops.strix.moe_gemm_bf16(c, a.to(DEV), b.to(DEV), sorted_ids.to(DEV), expert_ids.to(DEV),
                                  num_post.to(DEV), None, 1, 16, 64)
    ref = M.grouped_reference(a, b, ids, 1)
    out = c.float().cpu()
    assert torch.isnan(out[1:3]).all()
    torch.testing.assert_close(out[[0, 3, 4, 5]], ref[[0, 3, 4, 5]], rtol=2e-2, atol=2e-2)


def test_gemm_errors():
    b = torch.zeros(2, 256, 128, dtype=torch.bfloat16, device=DEV)
    a = torch.zeros(4, 128, dtype=torch.bfloat16, device=DEV)
    c = torch.zeros(4, 256, dtype=torch.bfloat16, device=DEV)
    s, e, n = (t.to(DEV) for t in M.align(torch.zeros(4, 1, dtype=torch.int32), 16, 2))
    with pytest.raises(RuntimeError, match="shape mismatch"):
        torch.ops.strix.moe_gemm_bf16(c[:, :100], a, b, s, e, n, None, 1, 16, 64)
    with pytest.raises(RuntimeError, match="routing tensors must be int32"):
        torch.ops.strix.moe_gemm_bf16(c, a, b, s.long(), e, n, None, 1, 16, 64)
    with pytest.raises(RuntimeError, match="silu_mul needs even N and no topk weights"):
        torch.ops.strix.moe_gemm_bf16(c[:, :128], a, b, s, e, n, torch.ones(4, device=DEV), 1, 16, 64,
                                      True)
    with pytest.raises(RuntimeError, match="activation must be silu or gelu_tanh"):
        torch.ops.strix.moe_gemm_bf16(c[:, :128], a, b, s, e, n, None, 1, 16, 64, True, "relu")
    with pytest.raises(RuntimeError, match="expert_ids too short"):
        torch.ops.strix.moe_gemm_bf16(c, a, b, s, e[:0], n, None, 1, 16, 64)


# ---------------------------------------------------------------- the layer

@pytest.mark.parametrize("layout", ["sorted", "gather"])
@pytest.mark.parametrize("tokens", [256, 37, 1])
def test_fp8_layer_benchmark_geometry(tokens, layout):
    """Config 1: hidden 2048, 128 experts, top-8, intermediate 768, FP8 W8A8
    block-scaled. Indices (routing, permutation) bit-exact, output within 2e-2 x
    RMS of the oracle layer, in both layouts of the intermediate buffers."""
    layer = moe_fp8_layer(tokens=tokens, seed=3, device=DEV)
    out = strix.moe.fused_moe_fp8_w8a8(layer.x, layer.logits, layer.w13, layer.w13_scale,
                                       layer.w2, layer.w2_scale, layer.top_k, layout=layout)
    cpu = layer.to("cpu")
    ref, ids_ref, w_ref = M.moe_fp8_layer(cpu.x, cpu.logits, cpu.w13, cpu.w13_scale, cpu.w2,
                                          cpu.w2_scale, cpu.top_k)
    w, ids = strix.moe.route(layer.logits, layer.top_k)
    assert torch.equal(ids.cpu(), ids_ref)
    rms_check(out, ref, 2e-2)


@pytest.mark.parametrize("tokens,top_k,experts,block_m", [(1, 8, 128, 16), (37, 8, 128, 32),
                                                          (300, 4, 16, 64), (256, 8, 128, 128)])
def test_scatter_quantiser_equals_gather_quantiser(tokens, top_k, experts, block_m):
    """Same bytes and scales in every row below num_post_padded, and slot_pos is
    the inverse of sorted_ids."""
    g = torch.Generator().manual_seed(tokens)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(tokens)]).int()
    x = (torch.randn(tokens, 256, generator=g) * 3).bfloat16().to(DEV)
    x[0, 128:] = 0
    sorted_ids, expert_ids, num_post, slot_pos = strix.moe.align_with_positions(ids.to(DEV), block_m,
                                                                                experts)
    ref_sorted, _, ref_post = M.align(ids, block_m, experts)
    n_post = int(num_post.item())
    assert n_post == int(ref_post.item())
    assert torch.equal(sorted_ids.cpu()[:n_post], ref_sorted[:n_post])
    pos = slot_pos.cpu().long()
    assert torch.equal(sorted_ids.cpu()[pos].long(), torch.arange(tokens * top_k))
    cap, slots = sorted_ids.numel(), tokens * top_k
    qa = torch.full((cap, 256), 0x7F, dtype=torch.uint8, device=DEV).view(torch.float8_e4m3fn)
    sa = torch.full((cap, 2), -1.0, device=DEV)
    qb, sb = qa.clone(), sa.clone()
    torch.ops.strix.moe_act_quant_fp8_sorted(x, qa, sa, sorted_ids, num_post, top_k, slots)
    torch.ops.strix.moe_act_quant_fp8_scatter(x, qb, sb, slot_pos, sorted_ids, num_post, top_k)
    assert torch.equal(qa.view(torch.uint8)[:n_post], qb.view(torch.uint8)[:n_post])
    assert torch.equal(sa[:n_post], sb[:n_post])


def test_fused_layer_is_cuda_graph_capturable():
    """No host synchronisation and no allocation outside torch's caching allocator:
    the seven launches of the layer record into a CUDA graph, and a replay on new
    inputs (same shapes) matches the eager result bit for bit."""
    layer = moe_fp8_layer(tokens=64, seed=4, device=DEV)
    args = (layer.w13, layer.w13_scale, layer.w2, layer.w2_scale, layer.top_k)
    x, logits = layer.x.clone(), layer.logits.clone()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        strix.moe.fused_moe_fp8_w8a8(x, logits, *args)          # warm-up outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = strix.moe.fused_moe_fp8_w8a8(x, logits, *args)
    torch.cuda.synchronize()
    other = moe_fp8_layer(tokens=64, seed=5, device=DEV)
    x.copy_(other.x)
    logits.copy_(other.logits)
    graph.replay()
    torch.cuda.synchronize()
    eager = strix.moe.fused_moe_fp8_w8a8(other.x, other.logits, *args)
    assert torch.equal(out.view(torch.int16), eager.view(torch.int16))
