"""Oracle for the MoE path (router, permute, activation quant, grouped expert
GEMMs with the fused gate epilogue, combine), CPU torch, fp32.

Restates the in-test references of the asf0/libstrix test-suite:
  align()       tests/test_moe_gemm.py:9-31   (moe_align_block_size contract)
  reference()   tests/test_moe_gemm.py:34-42  (per-expert fp32 matmul)
  FP8 weights   tests/test_moe_fp8.py:17-29, tests/test_moe_fp8_raw.py:17-39
  act quant i8  tests/test_moe_w4a8.py:24-36
The router, the e4m3 activation quantiser and the combine are not in the
reference (vLLM's); they follow the benchmark configuration's wording: fp32
softmax -> top-k -> renormalise; per-token-per-128 e4m3 with scale amax/448;
fp32 sum of the top-k rows, one bf16 rounding.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

FP8_MAX = 448.0


def align(topk_ids: torch.Tensor, block_m: int, num_experts: int):
    """moe_align_block_size's contract (tests/test_moe_gemm.py:9-31): slot ids
    grouped by expert in ascending expert and ascending slot order, each run
    padded to block_m with the invalid id topk_ids.numel(); experts without
    tokens get no block; one spare partial block and one spare expert id follow
    num_post_padded."""
    flat = topk_ids.flatten()
    pad = flat.numel()
    sorted_ids, expert_ids = [], []
    for e in range(num_experts):
        ids = (flat == e).nonzero().flatten().tolist()
        if not ids:
            continue
        ids += [pad] * (-len(ids) % block_m)
        sorted_ids += ids
        expert_ids += [e] * (len(ids) // block_m)
    total = len(sorted_ids)
    sorted_ids += [pad] * (block_m // 2 + 3)
    expert_ids += [0]
    return (torch.tensor(sorted_ids, dtype=torch.int32),
            torch.tensor(expert_ids, dtype=torch.int32),
            torch.tensor([total], dtype=torch.int32))


def grouped_reference(a, b, topk_ids, top_k, weights=None):
    """out[slot] = a[slot // top_k] @ b[expert(slot)]^T in fp32, times the
    slot's routing weight if given (tests/test_moe_gemm.py:34-42). `b` is the
    dequantised weight [E, N, K] in any float dtype."""
    flat = topk_ids.flatten()
    out = torch.empty(flat.numel(), b.size(1))
    for e in flat.unique().tolist():
        slots = (flat == e).nonzero().flatten()
        out[slots] = a[slots // top_k].float() @ b[e].float().t()
    if weights is not None:
        out = out * weights.flatten()[:, None]
    return out


def gate_mul(h: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """[gate (N/2) ; up (N/2)] columns -> act(gate) * up (tests/test_moe_fp8.py:73-77)."""
    n = h.size(1)
    gate, up = h[:, : n // 2], h[:, n // 2:]
    act = F.silu(gate) if activation == "silu" else F.gelu(gate, approximate="tanh")
    return act * up


def make_fp8_weights(e, n, k, scheme, seed=0, keep_fp32=False):
    """Random e4m3 experts + scales as tests/test_moe_fp8.py:17-29: values
    randn*40 clamped to +-448; block scales fp32 [E, N/128, K/128] or channel
    scales [E, N], both rand*0.02+0.001. Returns (w_fp8, scales, dequantised),
    the latter bf16-rounded (the plain op's oracle) or fp32 (`keep_fp32`, the
    raw op's oracle, tests/test_moe_fp8_raw.py:17-28)."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn((e, n, k), generator=g) * 40).clamp(-448, 448).to(torch.float8_e4m3fn)
    if scheme == "block":
        scales = torch.rand((e, n // 128, k // 128), generator=g) * 0.02 + 0.001
        full = scales.repeat_interleave(128, 1).repeat_interleave(128, 2)
    else:
        scales = torch.rand((e, n), generator=g) * 0.02 + 0.001
        full = scales.reshape(e, n, 1)
    deq = w.float() * full
    return w, scales, deq if keep_fp32 else deq.to(torch.bfloat16)


def quantize_weight_fp8_block(w: torch.Tensor):
    """fp32 [E, N, K] -> e4m3 with one fp32 scale per 128x128 block, s = amax /
    448 (benchmark config 1: weights N(0, 0.02) quantised with block scales)."""
    e, n, k = w.shape
    blocks = w.view(e, n // 128, 128, k // 128, 128)
    s = blocks.abs().amax(dim=(2, 4)).clamp_min(1e-12) / FP8_MAX
    q = (blocks / s[:, :, None, :, None]).view(e, n, k).to(torch.float8_e4m3fn)
    return q, s.contiguous()


def dequant_fp8_block(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    return q.float() * s.repeat_interleave(128, -2).repeat_interleave(128, -1)


def act_quant_i8(x: torch.Tensor, group: int = 128):
    """Per (row, 128-group) symmetric int8: s = amax / 127 (1 for an all-zero
    group), q = clamp(round(x / s), +-127) (tests/test_moe_w4a8.py:24-36)."""
    g = x.float().view(x.size(0), -1, group)
    s = g.abs().amax(-1) / 127
    s = torch.where(s > 0, s, torch.ones_like(s))
    q = torch.clamp(torch.round(g / s[..., None]), -127, 127).view(x.shape).to(torch.int8)
    return q, s


def act_quant_fp8(x: torch.Tensor, group: int = 128):
    """Per (row, 128-group) e4m3: s = amax / 448 (1 for an all-zero group),
    q = e4m3(x / s) with round-to-nearest-even (config 1's activation form)."""
    g = x.float().view(x.size(0), -1, group)
    s = g.abs().amax(-1) / FP8_MAX
    s = torch.where(s > 0, s, torch.ones_like(s))
    q = (g / s[..., None]).clamp(-FP8_MAX, FP8_MAX).view(x.shape).to(torch.float8_e4m3fn)
    return q, s


def dequant_act(q: torch.Tensor, s: torch.Tensor, group: int = 128) -> torch.Tensor:
    return q.float() * s.repeat_interleave(group, dim=-1)


def router(logits: torch.Tensor, top_k: int):
    """fp32 softmax over experts -> top-k -> renormalise to sum 1."""
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, top_k, dim=-1)
    return ids.to(torch.int32), w / w.sum(-1, keepdim=True)


def moe_sum(c3: torch.Tensor) -> torch.Tensor:
    """[T, top_k, H] -> [T, H]: fp32 sum, one bf16 rounding."""
    return c3.float().sum(1).to(torch.bfloat16)


def moe_fp8_layer(x, logits, w13_q, w13_s, w2_q, w2_s, top_k):
    """Benchmark config 1 end to end (W8A8 FP8, block-scaled): router -> quantise
    activations per token per 128 -> gate-up GEMM -> SiLU-mul (rounded to bf16,
    as the fused epilogue writes it) -> quantise -> down GEMM x routing weight
    (rounded to bf16) -> sum over top-k. Every GEMM consumes the
    quantised-then-dequantised activations, the convention of
    tests/test_moe_w4a8.py:78-80."""
    ids, wts = router(logits, top_k)
    xq, xs = act_quant_fp8(x)
    h = grouped_reference(dequant_act(xq, xs), dequant_fp8_block(w13_q, w13_s), ids, top_k)
    act = gate_mul(h).to(torch.bfloat16)
    aq, as_ = act_quant_fp8(act)
    y = grouped_reference(dequant_act(aq, as_), dequant_fp8_block(w2_q, w2_s), ids, 1, wts)
    y = y.to(torch.bfloat16)
    return moe_sum(y.view(x.size(0), top_k, -1)), ids, wts


def moe_mxfp4_layer(x, logits, w13, w13_scale, w2, w2_scale, top_k, token_ids=None,
                    expert_offset=0):
    """Benchmark config 5 (MXFP4 experts, bf16 activations, W4A16 reading): router
    -> gate-up GEMM over the exactly dequantised weights -> SiLU-mul rounded to
    bf16 -> down GEMM x routing weight rounded to bf16 -> fp32 sum over top-k, one
    bf16 rounding. `token_ids` restricts the evaluation to a sample of tokens (the
    router still sees every row it is given); the weights are dequantised one
    expert at a time inside the loop. Weight tensors may hold a contiguous slice
    of the experts starting at `expert_offset` (slots routed elsewhere must not
    occur in the sample then). Returns (out bf16 [len(token_ids), H], ids, weights)."""
    from . import gemm as G

    ids, wts = router(logits, top_k)
    sel = torch.arange(x.size(0)) if token_ids is None else torch.as_tensor(token_ids)
    xs, ids_s, wts_s = x[sel].float(), ids[sel].long(), wts[sel]
    hidden = w2.size(1)
    y = torch.zeros(sel.numel(), top_k, hidden)
    for e in ids_s.unique().tolist():
        tok, slot = (ids_s == e).nonzero(as_tuple=True)
        le = e - expert_offset
        h = xs[tok] @ G.mxfp4_dequant(w13[le], w13_scale[le]).t()
        act = gate_mul(h).to(torch.bfloat16).float()
        out = act @ G.mxfp4_dequant(w2[le], w2_scale[le]).t()
        y[tok, slot] = (out * wts_s[tok, slot, None]).to(torch.bfloat16).float()
    return y.sum(1).to(torch.bfloat16), ids, wts
