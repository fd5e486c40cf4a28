"""Dense W8A8 INT8 GEMM against the CPU oracle: the int32 sums bit for bit, the
bf16 output to its own rounding. Shapes follow the reference's
tests/test_w8a8_int8.py:84-85 ((n, k) in 2048x2048, 1024x2048, 256x4096; m in
6, 64, 300) plus ragged edges, decode rows and the 27B-like gate-up width."""

import ctypes

import pytest
import torch

import libstrix_b200 as strix  # noqa: F401  (registers torch.ops.strix)
from libstrix_b200 import _lib
from oracle import gemm as G

DEV = "cuda"


def make(m, n, k, seed=0):
    g = torch.Generator().manual_seed(seed * 7919 + m * 31 + n * 17 + k)
    a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    sa = torch.rand(m, generator=g) * 4e-2 + 1e-2
    sw = torch.rand(n, generator=g) * 9e-3 + 1e-3
    return a, sa, w, sw


def run(a, sa, w, sw, want_acc=True):
    acc = torch.empty(a.size(0), w.size(0), dtype=torch.int32, device=DEV) if want_acc else None
    out = torch.ops.strix.w8a8_int8_gemm(a.to(DEV), sa.to(DEV), w.to(DEV), sw.to(DEV), acc)
    torch.cuda.synchronize()
    flag = ctypes.c_int32(-1)
    assert _lib.load().strix_umma_status(ctypes.byref(flag)) == 0 and flag.value == 0
    return out.cpu(), (acc.cpu() if want_acc else None)


def check(m, n, k, seed=0):
    a, sa, w, sw = make(m, n, k, seed)
    out_ref, acc_ref = G.w8a8_int8_gemm(a, sa, w, sw)
    out, acc = run(a, sa, w, sw)
    assert torch.equal(acc, acc_ref), "int32 sums differ"
    # same fp32 products in the same order, one bf16 rounding: identical bits
    assert torch.equal(out.view(torch.int16), out_ref.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("n,k", [(2048, 2048), (1024, 2048), (256, 4096)])
@pytest.mark.parametrize("m", [1, 6, 16, 17, 33, 64, 65, 128, 300])
def test_matches_oracle(m, n, k):
    check(m, n, k)


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 8, 128), (3, 136, 128), (16, 120, 256), (64, 1000, 384),
                                   (100, 264, 128), (129, 257 * 8, 256), (257, 520, 1152),
                                   (1000, 776, 512)])
def test_ragged_edges(m, n, k):
    check(m, n, k, seed=1)


@pytest.mark.gpu
def test_extreme_values_do_not_overflow():
    """All operands +-127 at the 27B-like K: |sum| = 5120 * 127 * 127 < 2^31."""
    m, n, k = 130, 512, 5120
    a = torch.full((m, k), 127, dtype=torch.int8)
    a[::2] = -127
    w = torch.full((n, k), -127, dtype=torch.int8)
    w[::3] = 127
    sa, sw = torch.full((m,), 1e-2), torch.full((n,), 1e-3)
    out_ref, acc_ref = G.w8a8_int8_gemm(a, sa, w, sw)
    out, acc = run(a, sa, w, sw)
    assert torch.equal(acc, acc_ref) and acc.abs().max().item() == k * 127 * 127
    assert torch.equal(out.view(torch.int16), out_ref.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 16])
def test_gate_up_width_decode(m):
    """K = 5120, N = 34816 (a 27B-like MLP gate-up) at decode batch sizes."""
    check(m, 34816, 5120, seed=2)


@pytest.mark.gpu
def test_gate_up_width_prefill_properties():
    """M = 4096 at the full width: the CPU oracle covers a sample of rows and
    columns bit for bit; linearity in the scales covers the rest."""
    m, n, k = 4096, 34816, 5120
    a, sa, w, sw = make(m, n, k, seed=3)
    acc = torch.empty(m, n, dtype=torch.int32, device=DEV)
    ad, wd, sad, swd = a.to(DEV), w.to(DEV), sa.to(DEV), sw.to(DEV)
    out = torch.ops.strix.w8a8_int8_gemm(ad, sad, wd, swd, acc)
    rows = torch.arange(0, m, 61)
    cols = torch.arange(0, n, 127)
    ref = G.w8a8_int8_acc(a[rows], w[cols])
    assert torch.equal(acc[rows.to(DEV)][:, cols.to(DEV)].cpu(), ref)
    # every output is its own int32 sum times the two scales, rounded once
    expect = (acc.float() * sad[:, None] * swd[None, :]).to(torch.bfloat16)
    assert torch.equal(out.view(torch.int16), expect.view(torch.int16))
    # a row of ones against the sums: column totals agree with an int64 reduction on the host
    col_sum = acc[:, cols.to(DEV)].sum(0, dtype=torch.int64).cpu()
    assert torch.equal(col_sum, a.long().sum(0) @ w[cols].long().t())
    flag = ctypes.c_int32(-1)
    assert _lib.load().strix_umma_status(ctypes.byref(flag)) == 0 and flag.value == 0


@pytest.mark.gpu
def test_empty_batch():
    a, sa, w, sw = make(0, 256, 256)
    out, _ = run(a, sa, w, sw, want_acc=False)
    assert out.shape == (0, 256)


@pytest.mark.gpu
def test_argument_errors():
    a, sa, w, sw = (t.to(DEV) for t in make(4, 256, 256))
    op = torch.ops.strix.w8a8_int8_gemm
    with pytest.raises(RuntimeError):
        op(a[:, :200].contiguous(), sa, w[:, :200].contiguous(), sw)     # K % 128
    with pytest.raises(RuntimeError):
        op(a, sa[:3], w, sw)                                               # scale count
    with pytest.raises(RuntimeError):
        op(a.to(torch.uint8), sa, w, sw)                                   # dtype


def test_oracle_group_form_matches_reference_formula():
    """The group-quantised reference equals quantise -> exact int sums per
    group -> fp32 fold, the arithmetic the kernel form uses."""
    torch.manual_seed(0)
    m, n, k = 7, 40, 384
    x = torch.randn(m, k).to(torch.bfloat16)
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8)
    s = torch.rand(n) * 0.01 + 1e-4
    q, sg = G.act_quant_group_i8(x)
    acc = torch.einsum("mgk,ngk->mng", q.view(m, -1, 128).double(), w.view(n, -1, 128).double())
    folded = (acc * sg.double()[:, None, :]).sum(-1) * s.double()[None, :]
    ref = G.w8a8_group_reference(x, w, s)
    assert torch.allclose(folded.float(), ref, rtol=1e-4, atol=1e-4 * ref.abs().max().item())
