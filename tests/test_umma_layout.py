"""Pins the tcgen05 / TMEM conventions of the sm_100a kernels against a CPU
matmul (the analogue of the reference's tests/test_wmma_layout.py): operand
descriptors, swizzle, K advance, accumulator row/column mapping."""

import pytest
import torch

import libstrix_b200  # noqa: F401  (registers torch.ops.strix)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [16, 32, 64, 128, 256, 48, 208])
@pytest.mark.parametrize("k", [128, 256, 1024])
def test_int8_tile_is_bit_exact(n, k):
    g = torch.Generator().manual_seed(n + k)
    a = torch.randint(-128, 128, (128, k), generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int8)
    d = torch.ops.strix._umma_tile(a.cuda(), b.cuda())
    ref = a.to(torch.int32) @ b.to(torch.int32).t()
    assert torch.equal(d.cpu(), ref)


def test_int8_tile_is_not_transposed_or_permuted():
    """One-hot operands: D[m, j] = A[m, kk] * B[j, kk] isolates every index map."""
    k = 256
    a = torch.zeros(128, k, dtype=torch.int8)
    b = torch.zeros(64, k, dtype=torch.int8)
    for m in range(128):
        a[m, (m * 7) % k] = (m % 100) + 1
    for j in range(64):
        b[j, (j * 11 + 3) % k] = j + 1
    d = torch.ops.strix._umma_tile(a.cuda(), b.cuda())
    assert torch.equal(d.cpu(), a.to(torch.int32) @ b.to(torch.int32).t())


@pytest.mark.parametrize("n,k", [(16, 128), (64, 512), (256, 256)])
def test_e4m3_tile(n, k):
    g = torch.Generator().manual_seed(n)
    a = (torch.randn(128, k, generator=g) * 4).to(torch.float8_e4m3fn)
    b = (torch.randn(n, k, generator=g) * 4).to(torch.float8_e4m3fn)
    d = torch.ops.strix._umma_tile(a.cuda(), b.cuda())
    ref = a.float() @ b.float().t()
    torch.testing.assert_close(d.cpu(), ref, rtol=1e-3, atol=1e-2)
