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


# ------------------------------------------------------------------ 4-bit formats
MX_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def mxfp4_dequant(w_u8: torch.Tensor, s_u8: torch.Tensor) -> torch.Tensor:
    """fp32 [..., N, K]: e2m1 nibbles (low nibble = even k) times 2^(scale - 127),
    a scale byte of 0 being the zero block - tests/test_mxfp4.py:29-47 with the
    kernel's zero-block rule of :65-70 and :118-127."""
    lut = torch.tensor(MX_VALUES, dtype=torch.float32)
    w = w_u8.to(torch.int32)

    def value(nib):
        v = lut[(nib & 7).long()]
        return torch.where((nib & 8) != 0, -v, v)

    out = torch.empty(*w_u8.shape[:-1], w_u8.size(-1) * 2, dtype=torch.float32)
    out[..., 0::2] = value(w & 15)
    out[..., 1::2] = value((w >> 4) & 15)
    scale = torch.pow(2.0, s_u8.float() - 127.0) * (s_u8 != 0)
    return out * scale.repeat_interleave(32, dim=-1)


def mxfp4_quantize(w: torch.Tensor):
    """fp32 [..., K] -> (uint8 [..., K/2] e2m1 nibbles, uint8 [..., K/32] e8m0), the
    quantiser benchmark config 5 states: per 32 elements scale = 2^ceil(log2(amax
    / 6)), elements rounded to the nearest e2m1 value (ties to the even mantissa),
    low nibble = even k. Written as a nearest-neighbour search over the decode
    table, so that it shares no arithmetic with the threshold form the workload
    generator uses. The MX format has no counterpart quantiser in the reference
    (its checkpoints come quantised); the decode it must invert is
    tests/test_mxfp4.py:28-45."""
    k = w.size(-1)
    g = w.float().reshape(*w.shape[:-1], k // 32, 32)
    amax = g.abs().amax(-1)
    e = torch.ceil(torch.log2(amax.double() / 6.0))
    byte = torch.where(amax > 0, (e + 127).clamp(1, 254), torch.zeros_like(e)).to(torch.int64)
    scale = torch.pow(2.0, (byte - 127).double())
    x = (g.double() / scale[..., None]).abs()
    lut = torch.tensor(MX_VALUES, dtype=torch.float64)
    dist = (x[..., None] - lut).abs()                       # [..., 32, 8]
    best = dist.min(-1, keepdim=True).values
    cand = dist == best                                     # one or (on a tie) two codes
    even = torch.tensor([c % 2 == 0 for c in range(8)])
    pick_even = (cand & even).any(-1)
    code = torch.where(pick_even, (cand & even).to(torch.uint8).argmax(-1),
                       cand.to(torch.uint8).argmax(-1)).to(torch.uint8)
    code = code | ((g < 0).to(torch.uint8) << 3)
    code = torch.where((byte == 0)[..., None], torch.zeros_like(code), code).reshape(*w.shape[:-1], k)
    return (code[..., 0::2] | (code[..., 1::2] << 4)).contiguous(), byte.to(torch.uint8)


def int4_pack(q: torch.Tensor) -> torch.Tensor:
    """[..., K] values 0..15 -> [..., K/2] bytes, low nibble = even k
    (tests/test_moe_wna16.py:44-46)."""
    return (q[..., 0::2] | (q[..., 1::2] << 4)).contiguous()


def int4_pack_exllama(q: torch.Tensor) -> torch.Tensor:
    """[..., K] values 0..15 -> [..., K/2] bytes in vLLM's ExLlama word order: every
    32-bit word holds eight consecutive elements, nibble i = element (0 2 4 6 1 3 5
    7)[i] - the layout the reference's dense int4 ops decode
    (csrc/gemm/w8a8_wmma_gemm.hip:128-132,278-291; its tests pack with vLLM's
    pack_skinny_int4, tests/test_w8a16.py:74-98, which is not available here, so this
    packer is pinned only by the format statement in the kernel source: parity
    unpinned)."""
    order = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7])
    k = q.size(-1)
    words = q.reshape(*q.shape[:-1], k // 8, 8)[..., order].to(torch.uint8)     # nibble i of each word
    return (words[..., 0::2] | (words[..., 1::2] << 4)).reshape(*q.shape[:-1], k // 2).contiguous()


def int4_dequant(w_u8: torch.Tensor, scales: torch.Tensor, group: int, exact: bool = False):
    """(nibble - 8) * scale per group, rounded to bf16 unless `exact`
    (tests/test_moe_wna16.py:48-62)."""
    q = torch.stack([(w_u8 & 0xF).float() - 8.0, ((w_u8 >> 4) & 0xF).float() - 8.0],
                    dim=-1).reshape(*w_u8.shape[:-1], -1)
    w = q * scales.float().repeat_interleave(group, dim=-1)
    return w if exact else w.to(torch.bfloat16)


def w8a16_reference(x, w_u8, scales, group_size):
    """fp32 [M, N] of excess-128 byte weights (tests/test_w8a16.py:9-17)."""
    w = w_u8.float() - 128.0
    k = w.size(1)
    s = scales.float()
    s = s.repeat_interleave(group_size, dim=1)[:, :k] if group_size else s.reshape(-1, 1)
    return x.float() @ (w * s).t()


def fp8_dequant(w: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """fp32 [N, K]: e4m3 times fp32 scales per channel [N] or per 128 x 128 block
    [ceil(N/128), K/128] (csrc/gemm/fp8_dequant.hip:63)."""
    n, k = w.shape
    if scales.dim() == 2 and scales.size(1) != 1:
        full = scales.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :k]
    else:
        full = scales.reshape(n, 1)
    return w.float() * full
