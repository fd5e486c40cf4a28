"""CPU oracle for the dense quantized GEMMs - TEST INFRASTRUCTURE, not product code.

Restates the torch references the asf0/libstrix tests judge the dense kernels
with; see the package docstring for who may import this.
"""

from __future__ import annotations

import torch


def w8a8_int8_acc(a_q: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Exact int32 sums acc[m, n] = sum_k a_q[m, k] * w[n, k] of int8 operands.

    K * 127 * 127 stays far below 2^31 for every K a layer has, and below 2^53
    per fp64 partial sum, so the fp64 matmul (BLAS, fast) is exact; it is
    checked against an int64 matmul on a corner block."""
    acc = (a_q.double() @ w.double().t())
    m, n = min(8, a_q.size(0)), min(8, w.size(0))
    exact = a_q[:m].long() @ w[:n].long().t()
    assert torch.equal(acc[:m, :n].long(), exact)
    return acc.to(torch.int32)


def w8a8_int8_gemm(a_q, a_scale, w, w_scale):
    """(bf16 out [M, N], int32 acc [M, N]) of the per-token / per-channel W8A8
    GEMM: out = bf16(acc * a_scale[m] * w_scale[n]), the products taken in fp32
    in that order."""
    acc = w8a8_int8_acc(a_q, w)
    out = acc.float() * a_scale.float().reshape(-1, 1) * w_scale.float().reshape(1, -1)
    return out.to(torch.bfloat16), acc


def w8a8_group_reference(x: torch.Tensor, w_i8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 [M, N]: per-channel int8 weights times activations quantised to
    int8 per (row, 128-element group) - the reference of
    tests/test_w8a8_int8.py:50-58 for strix::w8a8_wmma_gemm
    (csrc/gemm/w8a8_wmma_gemm.hip:15-22)."""
    m, k = x.shape
    wf = w_i8.float() * scale.reshape(-1, 1)
    xg = x.float().reshape(m, k // 128, 128)
    sc = xg.abs().amax(-1, keepdim=True).clamp_min(1e-8) / 127
    xq = (xg / sc).round().clamp(-127, 127) * sc
    return xq.reshape(m, k) @ wf.t()


def act_quant_group_i8(x: torch.Tensor):
    """(q int8 [M, K], s fp32 [M, K/128]): the in-op activation quantiser of
    csrc/gemm/w8a8_wmma_gemm.hip:17-19 - s = max|x| / 127 over the group (1 if
    the group is all zero), q = clamp(rint(x / s), -127, 127)."""
    m, k = x.shape
    xg = x.float().reshape(m, k // 128, 128)
    amax = xg.abs().amax(-1, keepdim=True)
    s = torch.where(amax > 0, amax / 127, torch.ones_like(amax))
    q = torch.clamp(torch.round(xg / s), -127, 127).to(torch.int8)
    return q.reshape(m, k), s.reshape(m, k // 128)
