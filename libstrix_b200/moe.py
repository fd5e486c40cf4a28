"""MoE layer built from the strix ops: route -> permute -> quantise -> gate-up
GEMM with the fused gate -> quantise -> down GEMM x routing weight -> combine.

The sequence is the reference's StrixFp8Experts.apply
(python/strix_vllm/moe.py:905-1014) with vLLM's router, moe_align_block_size
and moe_sum replaced by this library's kernels, and with the W8A8 activation
form of the benchmark configuration (e4m3 per token per 128).
"""

from __future__ import annotations

import torch

from . import _lib


# m-blocks the sorted-layout tcgen05 kernels index in one launch (kMaxMBlocks in
# csrc/moe_gemm_umma.cu); larger batches take the gather layout
MAX_SORTED_M_BLOCKS = 2048


def pick_block_m(tokens: int, top_k: int, experts: int) -> int:
    """Rows per m-block. Up to 16 rows per expert on average: the smaller of 16 /
    32 that holds an expert's share twice over, so most experts stream their
    weights exactly once (tokens as the MMA's N, 128 weight rows as its M).
    Beyond that 128, the tile of the wide tcgen05 kernel (tokens as the MMA's
    M, 256 weight rows as its N): measured faster from 32 rows per expert on
    (0.225 vs 0.234 ms at 512 tokens, 0.51 vs 0.99 ms at 4096)."""
    per_expert = tokens * top_k / max(experts, 1)
    for bm in (16, 32):
        if per_expert * 2 <= bm:
            return bm
    return 128


def route(logits: torch.Tensor, top_k: int, renormalize: bool = True):
    """(topk_weights fp32 [T, k], topk_ids int32 [T, k]) by softmax -> top-k -> renormalise."""
    t = logits.size(0)
    weights = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    ids = torch.empty(t, top_k, dtype=torch.int32, device=logits.device)
    torch.ops.strix.moe_topk_softmax(weights, ids, logits, renormalize)
    return weights, ids


def align(topk_ids: torch.Tensor, block_m: int, num_experts: int):
    """(sorted_ids, expert_ids, num_post_padded) with the moe_align_block_size contract."""
    lib = _lib.load()
    cap = lib.strix_moe_align_capacity(topk_ids.numel(), num_experts, block_m)
    sorted_ids = torch.empty(cap, dtype=torch.int32, device=topk_ids.device)
    expert_ids = torch.empty(cap // block_m, dtype=torch.int32, device=topk_ids.device)
    num_post = torch.empty(1, dtype=torch.int32, device=topk_ids.device)
    torch.ops.strix.moe_align_block_size(topk_ids, num_experts, block_m, sorted_ids, expert_ids,
                                         num_post)
    return sorted_ids, expert_ids, num_post


def align_with_positions(topk_ids: torch.Tensor, block_m: int, num_experts: int):
    """align() plus slot_pos int32 [numel]: the sorted position of every slot."""
    lib = _lib.load()
    cap = lib.strix_moe_align_capacity(topk_ids.numel(), num_experts, block_m)
    dev = topk_ids.device
    sorted_ids = torch.empty(cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(cap // block_m, dtype=torch.int32, device=dev)
    num_post = torch.empty(1, dtype=torch.int32, device=dev)
    slot_pos = torch.empty(topk_ids.numel(), dtype=torch.int32, device=dev)
    torch.ops.strix.moe_align_block_size_pos(topk_ids, num_experts, block_m, sorted_ids, expert_ids,
                                             num_post, slot_pos)
    return sorted_ids, expert_ids, num_post, slot_pos


def act_quant_fp8(x: torch.Tensor):
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    sa = torch.empty(x.size(0), x.size(1) // 128, dtype=torch.float32, device=x.device)
    torch.ops.strix.moe_act_quant_fp8(x, q, sa)
    return q, sa


class Fp8MoeWorkspace:
    """Intermediate buffers of one layer call, reusable across calls of one shape.
    With `sorted_rows` (the capacity of the sorted id list) the activation
    buffers are laid out by sorted position, the layout of the tcgen05 path."""

    def __init__(self, tokens, top_k, hidden, inter, device, sorted_rows=None):
        slots = tokens * top_k
        bf16, f32, f8 = torch.bfloat16, torch.float32, torch.float8_e4m3fn
        self.sorted_rows = sorted_rows
        in_rows = sorted_rows if sorted_rows is not None else tokens
        mid_rows = sorted_rows if sorted_rows is not None else slots
        self.xq = torch.empty(in_rows, hidden, dtype=f8, device=device)
        self.xs = torch.empty(in_rows, hidden // 128, dtype=f32, device=device)
        self.act = torch.empty(mid_rows, inter, dtype=bf16, device=device)
        self.aq = torch.empty(mid_rows, inter, dtype=f8, device=device)
        self.as_ = torch.empty(mid_rows, inter // 128, dtype=f32, device=device)
        self.y = torch.empty(slots, hidden, dtype=bf16, device=device)
        self.out = torch.empty(tokens, hidden, dtype=bf16, device=device)


class Fp8LayerWorkspace:
    """Scratch of the one-call layer launcher (strix_moe_fp8_layer) for one shape,
    plus the output rows."""

    def __init__(self, tokens, top_k, hidden, inter, experts, block_m, device, with_out=True):
        self.key = (tokens, top_k, hidden, inter, experts, block_m)
        self.nbytes = _lib.load().strix_moe_fp8_layer_workspace(*self.key)
        self.buf = torch.empty(self.nbytes + 256, dtype=torch.uint8, device=device)
        self.ptr = (self.buf.data_ptr() + 255) // 256 * 256
        self.out = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=device) if with_out else None


def workspace_for(tokens, top_k, hidden, inter, experts, block_m, device, layout="sorted"):
    """The workspace fused_moe_fp8_w8a8 wants for this shape, so that a caller
    can allocate it once."""
    if layout != "sorted":
        return Fp8MoeWorkspace(tokens, top_k, hidden, inter, device)
    return Fp8LayerWorkspace(tokens, top_k, hidden, inter, experts, block_m, device)


def fits_sorted_grid(slots: int, experts: int, block_m: int) -> bool:
    """Whether the padded id list of `slots` routed rows stays within the m-blocks
    one launch of the sorted-layout kernels may walk (MAX_SORTED_M_BLOCKS); above
    it the layer takes the gather layout. Host arithmetic only."""
    return _lib.load().strix_moe_align_capacity(slots, experts, block_m) // block_m <= MAX_SORTED_M_BLOCKS


def sorted_path_covers(w13, w13_scale, w2, w2_scale, block_m: int) -> bool:
    """Whether both GEMMs of the layer run on the tcgen05 sorted-layout kernel."""
    lib = _lib.load()

    def kind(w, s):
        return 2 if s.dim() == 3 and s.size(1) != w.size(1) else 1

    return bool(lib.strix_moe_gemm_fp8_sorted_covers(w13.size(1), w13.size(2), block_m, 1,
                                                     kind(w13, w13_scale))
                and lib.strix_moe_gemm_fp8_sorted_covers(w2.size(1), w2.size(2), block_m, 0,
                                                         kind(w2, w2_scale)))


def fused_moe_fp8_w8a8(x, logits, w13, w13_scale, w2, w2_scale, top_k, block_m=None, ws=None,
                       layout="auto"):
    """One MoE layer, FP8 W8A8 block-scaled. x bf16 [T, H]; logits fp32 [T, E];
    w13 e4m3 [E, 2I, H] + fp32 scales [E, 2I/128, H/128]; w2 e4m3 [E, H, I] +
    scales [E, H/128, I/128]. Returns bf16 [T, H]. Seven kernel launches, no
    host synchronisation. Where the sorted-layout tcgen05 kernels cover the shape the
    whole layer is ONE call into the library (strix_moe_fp8_layer); otherwise the
    router op, then experts_fp8_w8a8."""
    out = _layer_call(x, logits, None, None, w13, w13_scale, w2, w2_scale, top_k, block_m, ws, layout,
                      None, "silu")
    if out is not None:
        return out
    weights, ids = route(logits, top_k)
    return experts_fp8_w8a8(x, weights, ids, w13, w13_scale, w2, w2_scale, block_m=block_m, ws=ws,
                            layout="gather" if layout == "auto" else layout)


def _layer_call(x, logits, topk_weights, topk_ids, w13, w13_scale, w2, w2_scale, top_k, block_m, ws,
                layout, out, activation):
    """The layer through strix_moe_fp8_layer, or None where it does not apply."""
    t, h = x.shape
    e, n13, _ = w13.shape
    inter = n13 // 2
    bm = block_m or pick_block_m(t, top_k, e)
    lib = _lib.load()
    if layout not in ("auto", "sorted") or x.dtype != torch.bfloat16 or x.stride(1) != 1 or t == 0:
        return None
    f8 = torch.float8_e4m3fn
    if w13.dtype != f8 or w2.dtype != f8 or w13_scale.dtype != torch.float32 \
            or w2_scale.dtype != torch.float32 or w13.stride(2) != 1 or w2.stride(2) != 1 \
            or w13_scale.stride(-1) != 1 or w2_scale.stride(-1) != 1 \
            or (logits is not None and (logits.dtype != torch.float32 or logits.stride(1) != 1)):
        return None
    if not sorted_path_covers(w13, w13_scale, w2, w2_scale, bm) \
            or not fits_sorted_grid(t * top_k, e, bm):
        if layout == "sorted":
            raise RuntimeError("fused_moe_fp8_w8a8: geometry not covered by the sorted-layout kernels")
        return None
    if not isinstance(ws, Fp8LayerWorkspace) or ws.key != (t, top_k, h, inter, e, bm):
        ws = Fp8LayerWorkspace(t, top_k, h, inter, e, bm, x.device)
    out = ws.out if out is None else out
    block = w13_scale.dim() == 3 and w13_scale.size(1) != n13
    if topk_ids is not None:
        topk_ids = topk_ids.to(torch.int32).contiguous()
        topk_weights = topk_weights.to(torch.float32).contiguous()
    with torch.cuda.device(x.device):
        _lib.call("strix_moe_fp8_layer", out.data_ptr(), x.data_ptr(),
                  None if logits is None else logits.data_ptr(),
                  None if topk_weights is None else topk_weights.data_ptr(),
                  None if topk_ids is None else topk_ids.data_ptr(),
                  w13.data_ptr(), w13_scale.data_ptr(), w2.data_ptr(), w2_scale.data_ptr(), ws.ptr,
                  ws.nbytes, t, h, inter, e, top_k, bm, x.stride(0),
                  0 if logits is None else logits.stride(0), out.stride(0), w13.stride(0), w13.stride(1),
                  w13_scale.stride(0), w13_scale.stride(1) if block else 0, w2.stride(0), w2.stride(1),
                  w2_scale.stride(0), w2_scale.stride(1) if block else 0, 2 if block else 1,
                  2 if activation == "gelu_tanh" else 1, torch.cuda.current_stream().cuda_stream)
        _lib.after_tcgen05("fused_moe_fp8_w8a8")
    return out


def experts_fp8_w8a8(x, topk_weights, topk_ids, w13, w13_scale, w2, w2_scale, out=None,
                     block_m=None, ws=None, layout="auto", activation="silu"):
    """The experts of an FP8 W8A8 MoE layer for routing that is already decided
    (topk_weights fp32 / topk_ids int32 [T, k], e.g. by the serving framework's
    router): permute -> quantise -> gate-up GEMM with the fused gate -> quantise
    -> down GEMM x routing weight -> sum over top-k into `out` (bf16 [T, H]).
    The sequence is the reference's StrixFp8Experts.apply
    (python/strix_vllm/moe.py:905-1014) with e4m3 activations per (token, 128).

    layout "sorted" (the default where covered): the quantiser permutes the
    tokens into sorted order, both GEMMs run on tcgen05 with TMA-fed operands,
    the intermediate stays in sorted order and the down GEMM scatters to slot
    order for the combine. layout "gather": the GEMMs gather token rows by slot
    id themselves (the reference's op contract, mma.sync streaming kernels)."""
    t, h = x.shape
    e, n13, _ = w13.shape
    top_k = topk_ids.size(1)
    inter = n13 // 2
    if layout in ("auto", "sorted") and not isinstance(ws, Fp8MoeWorkspace):
        done = _layer_call(x, None, topk_weights, topk_ids, w13, w13_scale, w2, w2_scale, top_k,
                           block_m, ws, layout, out, activation)
        if done is not None:
            return done
    bm = block_m or pick_block_m(t, top_k, e)
    lib = _lib.load()
    if layout == "auto":
        layout = "sorted" if sorted_path_covers(w13, w13_scale, w2, w2_scale, bm) \
            and fits_sorted_grid(t * top_k, e, bm) else "gather"
    weights = topk_weights.to(torch.float32)
    ids = topk_ids.to(torch.int32).contiguous()
    ops = torch.ops.strix
    if layout == "sorted":
        sorted_ids, expert_ids, num_post, slot_pos = align_with_positions(ids, bm, e)
    else:
        sorted_ids, expert_ids, num_post = align(ids, bm, e)
    if layout == "sorted":
        cap = sorted_ids.numel()
        if ws is None or ws.sorted_rows != cap:
            ws = Fp8MoeWorkspace(t, top_k, h, inter, x.device, sorted_rows=cap)
        slots = t * top_k
        ops.moe_act_quant_fp8_scatter(x, ws.xq, ws.xs, slot_pos, sorted_ids, num_post, top_k)
        ops.moe_gemm_fp8_sorted(ws.act, ws.xq, ws.xs, w13, w13_scale, sorted_ids, expert_ids,
                                num_post, None, slots, bm, True, activation, True)
        ops.moe_act_quant_fp8_sorted(ws.act, ws.aq, ws.as_, None, num_post, 1, slots)
        ops.moe_gemm_fp8_sorted(ws.y, ws.aq, ws.as_, w2, w2_scale, sorted_ids, expert_ids,
                                num_post, weights.reshape(-1), slots, bm, False, "silu", False)
    else:
        if ws is None or ws.sorted_rows is not None:
            ws = Fp8MoeWorkspace(t, top_k, h, inter, x.device)
        ops.moe_act_quant_fp8(x, ws.xq, ws.xs)
        ops.moe_gemm_fp8_w8a8(ws.act, ws.xq, ws.xs, w13, w13_scale, sorted_ids, expert_ids,
                              num_post, None, top_k, bm, 64, True, activation)
        ops.moe_act_quant_fp8(ws.act, ws.aq, ws.as_)
        ops.moe_gemm_fp8_w8a8(ws.y, ws.aq, ws.as_, w2, w2_scale, sorted_ids, expert_ids, num_post,
                              weights.reshape(-1), 1, bm, 64, False, "silu")
    out = ws.out if out is None else out
    ops.moe_sum(ws.y.view(t, top_k, h), out)
    return out


def fused_moe_mxfp4(x, logits, w13, w13_scale, w2, w2_scale, top_k, block_m=None):
    """One MoE layer over MXFP4 experts (e2m1 nibbles, e8m0 scale per 32) and bf16
    activations: w13 uint8 [E, 2I, H/2] + scales [E, 2I, H/32], w2 uint8 [E, H, I/2]
    + scales [E, H, I/32]. route -> align -> permute into sorted order -> gate-up
    GEMM with SiLU-mul -> down GEMM x routing weight -> sum over top-k. From 32 rows
    per expert on (and where its tiles divide the shapes) the tcgen05 kernel over
    the sorted layout runs, below that the weight-streaming kernel. Six launches,
    no host synchronisation. Returns bf16 [T, H]."""
    t, h = x.shape
    e = w13.size(0)
    inter = w13.size(1) // 2
    lib = _lib.load()
    ops = torch.ops.strix
    weights, ids = route(logits, top_k)
    out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
    y = torch.empty(t * top_k, h, dtype=torch.bfloat16, device=x.device)
    wide_ok = bool(lib.strix_moe_gemm_mxfp4_sorted_covers(w13.size(1), w13.size(2) * 2, 128, 1)
                   and lib.strix_moe_gemm_mxfp4_sorted_covers(w2.size(1), w2.size(2) * 2, 128, 0))
    bm = block_m or (128 if wide_ok and t * top_k >= 32 * e else 64)
    if bm == 128 and wide_ok:
        sorted_ids, expert_ids, num_post, slot_pos = align_with_positions(ids, 128, e)
        cap = sorted_ids.numel()
        xs = torch.empty(cap, h, dtype=torch.bfloat16, device=x.device)
        act = torch.empty(cap, inter, dtype=torch.bfloat16, device=x.device)
        ops.moe_permute_bf16(x, xs, slot_pos, sorted_ids, num_post, top_k)
        ops.moe_gemm_mxfp4_sorted(act, xs, w13, w13_scale, sorted_ids, expert_ids, num_post, None,
                                  t * top_k, 128, True, "silu", True)
        ops.moe_gemm_mxfp4_sorted(y, act, w2, w2_scale, sorted_ids, expert_ids, num_post,
                                  weights.view(-1), t * top_k, 128, False, "silu", False)
    else:
        sorted_ids, expert_ids, num_post = align(ids, bm, e)
        act = torch.empty(t * top_k, inter, dtype=torch.bfloat16, device=x.device)
        ops.moe_gemm_mxfp4(act, x, w13, w13_scale, sorted_ids, expert_ids, num_post, None, top_k,
                           bm, 64, True, "silu")
        ops.moe_gemm_mxfp4(y, act, w2, w2_scale, sorted_ids, expert_ids, num_post, weights.view(-1),
                           1, bm, 64, False, "silu")
    ops.moe_sum(y.view(t, top_k, h), out)
    return out
