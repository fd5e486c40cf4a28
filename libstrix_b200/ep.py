"""Expert-parallel MoE: token dispatch -> local experts -> combine.

Every rank holds `experts_per_rank` consecutive experts and its own tokens. A
routed slot (token, k) travels to the rank that owns its expert, is computed
there with the grouped GEMMs of this library, and its result row travels back;
the source rank then sums a token's top-k rows. The exchange is two
`all_to_all_single` calls over the process group (NCCL over NVLink on GPUs,
gloo in the CPU tests): activation rows one way, result rows the other, plus one
small call for (local expert id, routing weight) pairs and one for the counts.

The reference has no expert parallelism (its experts refuse an `expert_map`,
python/strix_vllm/moe.py:193-210); this is the path the 8-GPU configuration
needs. The split sizes of an uneven all-to-all live on the host, so a layer call
synchronises once (the counts); everything else stays on the stream.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def dispatch_plan(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """(order, send_counts): slots sorted by destination rank (stable, so a
    rank's rows keep slot order) and the number of slots per destination."""
    dest = (topk_ids.reshape(-1) // experts_per_rank).to(torch.int64)
    order = torch.sort(dest, stable=True).indices
    send_counts = torch.bincount(dest, minlength=world)[:world]
    return order, send_counts


def ep_dispatch_combine(
    x: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    experts_per_rank: int,
    local_fn: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
    group=None,
    combine: Callable[[torch.Tensor], torch.Tensor] | None = None,
) -> torch.Tensor:
    """x [T, H]; topk_weights fp32 [T, k]; topk_ids int [T, k] (global expert
    ids). local_fn(rows [R, H], local_ids int32 [R], weights fp32 [R]) -> [R, H]
    computes `weights[r] * expert[local_ids[r]](rows[r])` for the rows this rank
    received. Returns [T, H]: for each token the sum of its k result rows
    (`combine`, default a float32 sum rounded to x's dtype)."""
    world = dist.get_world_size(group)
    t, k = topk_ids.shape
    h = x.size(1)
    if x.is_cuda and x.dtype == torch.bfloat16 and h % 8 == 0:
        return _dispatch_combine_cuda(x, topk_weights, topk_ids, experts_per_rank, local_fn, group)
    order, send_counts = dispatch_plan(topk_ids, experts_per_rank, world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    send_splits, recv_splits = send_counts.tolist(), recv_counts.tolist()   # the one host sync
    n_recv = sum(recv_splits)

    # rows and (local expert id, weight) of every slot, in dispatch order
    send_x = x.index_select(0, order // k)
    meta = torch.empty(t * k, 2, dtype=torch.float32, device=x.device)
    flat_ids = topk_ids.reshape(-1).index_select(0, order)
    meta[:, 0] = (flat_ids % experts_per_rank).to(torch.float32)
    meta[:, 1] = topk_weights.reshape(-1).to(torch.float32).index_select(0, order)
    recv_x = torch.empty(n_recv, h, dtype=x.dtype, device=x.device)
    recv_meta = torch.empty(n_recv, 2, dtype=torch.float32, device=x.device)
    dist.all_to_all_single(recv_x, send_x, recv_splits, send_splits, group=group)
    dist.all_to_all_single(recv_meta, meta, recv_splits, send_splits, group=group)

    y = local_fn(recv_x, recv_meta[:, 0].to(torch.int32), recv_meta[:, 1].contiguous())

    back = torch.empty(t * k, h, dtype=y.dtype, device=x.device)
    dist.all_to_all_single(back, y.contiguous(), send_splits, recv_splits, group=group)
    slots = torch.empty_like(back)
    slots.index_copy_(0, order, back)          # undo the dispatch order
    slots = slots.view(t, k, h)
    if combine is not None:
        return combine(slots)
    return slots.float().sum(1).to(x.dtype)


def _dispatch_combine_cuda(x, topk_weights, topk_ids, experts_per_rank, local_fn, group):
    """ep_dispatch_combine on the GPU with this library's kernels around the four
    collectives: the plan (slots grouped by destination rank, its inverse and the
    per-rank counts) is one launch of the align kernel with ranks as "experts" and
    block_m = 1; one launch packs the send rows and the (local expert, weight)
    pairs; the combine reads the returned rows through the inverse permutation."""
    from . import _lib

    world = dist.get_world_size(group)
    t, k = topk_ids.shape
    h = x.size(1)
    n = t * k
    dev = x.device
    i32 = dict(dtype=torch.int32, device=dev)
    ids = topk_ids.reshape(-1).to(torch.int32).contiguous()
    wts = topk_weights.reshape(-1).to(torch.float32).contiguous()
    dest = torch.div(ids, experts_per_rank, rounding_mode="floor").to(torch.int32)
    order = torch.empty(max(n, 1), **i32)
    blocks = torch.empty(max(n, 1), **i32)
    n_post = torch.empty(1, **i32)
    slot_pos = torch.empty(max(n, 1), **i32)
    counts = torch.empty(world, **i32)
    stream = torch.cuda.current_stream().cuda_stream
    with torch.cuda.device(dev):
        _lib.call("strix_moe_align_counts", dest.data_ptr(), order.data_ptr(), blocks.data_ptr(),
                  n_post.data_ptr(), slot_pos.data_ptr(), counts.data_ptr(), n, world, 1,
                  order.numel(), blocks.numel(), stream)
    send_counts = counts.to(torch.int64)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    send_splits, recv_splits = send_counts.tolist(), recv_counts.tolist()   # the one host sync
    n_recv = sum(recv_splits)

    # a send row = the token's `h` bf16 values + 16 bytes holding (local expert id,
    # routing weight) as two floats, so one collective carries both
    hp = h + 8
    send = torch.empty(n, hp, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.call("strix_ep_pack", x.data_ptr(), send.data_ptr(), send.data_ptr() + 2 * h,
                  order.data_ptr(), ids.data_ptr(), wts.data_ptr(), n, h, k, experts_per_rank,
                  x.stride(0), hp, hp // 2, stream)
    recv = torch.empty(n_recv, hp, dtype=torch.bfloat16, device=dev)
    dist.all_to_all_single(recv, send, recv_splits, send_splits, group=group)
    recv_meta = recv[:, h:h + 4].view(torch.float32)

    y = local_fn(recv[:, :h], recv_meta[:, 0].to(torch.int32), recv_meta[:, 1].contiguous())

    back = torch.empty(n, h, dtype=torch.bfloat16, device=dev)
    dist.all_to_all_single(back, y.contiguous(), send_splits, recv_splits, group=group)
    out = torch.empty(t, h, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.call("strix_moe_sum_gather", back.data_ptr(), slot_pos.data_ptr(), out.data_ptr(), t, k, h,
                  back.stride(0) if n else h, out.stride(0), stream)
    return out


def local_experts_mxfp4(w13, w13_scale, w2, w2_scale, block_m: int | None = None):
    """local_fn over this rank's MXFP4 experts: w13 uint8 [E, 2I, H/2] with e8m0
    scales [E, 2I, H/32], w2 uint8 [E, H, I/2] with scales [E, H, I/32]. Gate-up
    GEMM with SiLU-mul, down GEMM times the routing weight; the received rows
    are tokens with one expert each. From 32 rows per expert on (and where its
    tiles divide the shapes) the tensor-core kernel over the sorted layout runs,
    below that the weight-streaming kernel."""
    from . import _lib
    from . import moe as _moe

    e = w13.size(0)
    inter = w13.size(1) // 2
    hidden = w2.size(1)
    ops = torch.ops.strix
    lib = _lib.load()
    wide_ok = bool(lib.strix_moe_gemm_mxfp4_sorted_covers(w13.size(1), w13.size(2) * 2, 128, 1)
                   and lib.strix_moe_gemm_mxfp4_sorted_covers(w2.size(1), w2.size(2) * 2, 128, 0))

    def run(rows, local_ids, weights):
        r = rows.size(0)
        dev = rows.device
        y = torch.empty(r, hidden, dtype=torch.bfloat16, device=dev)
        if r == 0:
            return y
        bm = block_m or (128 if wide_ok and r >= 32 * e else 64)
        if bm == 128 and wide_ok:
            sorted_ids, expert_ids, num_post, slot_pos = _moe.align_with_positions(
                local_ids.view(r, 1).contiguous(), 128, e)
            cap = sorted_ids.numel()
            xs = torch.empty(cap, rows.size(1), dtype=torch.bfloat16, device=dev)
            act = torch.empty(cap, inter, dtype=torch.bfloat16, device=dev)
            ops.moe_permute_bf16(rows, xs, slot_pos, sorted_ids, num_post, 1)
            ops.moe_gemm_mxfp4_sorted(act, xs, w13, w13_scale, sorted_ids, expert_ids, num_post, None,
                                      r, 128, True, "silu", True)
            ops.moe_gemm_mxfp4_sorted(y, act, w2, w2_scale, sorted_ids, expert_ids, num_post, weights,
                                      r, 128, False, "silu", False)
            return y
        sorted_ids, expert_ids, num_post = _moe.align(local_ids.view(r, 1), bm, e)
        act = torch.empty(r, inter, dtype=torch.bfloat16, device=dev)
        ops.moe_gemm_mxfp4(act, rows, w13, w13_scale, sorted_ids, expert_ids, num_post, None, 1,
                           bm, 64, True, "silu")
        ops.moe_gemm_mxfp4(y, act, w2, w2_scale, sorted_ids, expert_ids, num_post, weights, 1,
                           bm, 64, False, "silu")
        return y

    return run


def local_experts_fp8(w13, w13_scale, w2, w2_scale, block_m: int | None = None):
    """local_fn over this rank's FP8 W8A8 block-scaled experts (w13 e4m3 [E, 2I, H]
    with fp32 scales [E, 2I/128, H/128], w2 e4m3 [E, H, I] with [E, H/128, I/128]):
    the sorted-layout tcgen05 path of moe.fused_moe_fp8_w8a8, the received rows
    being tokens with one expert each."""
    from . import moe as _moe

    e = w13.size(0)
    inter = w13.size(1) // 2
    hidden = w2.size(1)
    ops = torch.ops.strix
    f8 = torch.float8_e4m3fn

    def run(rows, local_ids, weights):
        r = rows.size(0)
        dev = rows.device
        y = torch.empty(r, hidden, dtype=torch.bfloat16, device=dev)
        if r == 0:
            return y
        bm = block_m or _moe.pick_block_m(r, 1, e)
        if not _moe.sorted_path_covers(w13, w13_scale, w2, w2_scale, bm):
            raise RuntimeError("local_experts_fp8: geometry not covered by the sorted-layout kernel")
        sorted_ids, expert_ids, num_post, slot_pos = _moe.align_with_positions(
            local_ids.view(r, 1).contiguous(), bm, e)
        cap = sorted_ids.numel()
        xq = torch.empty(cap, rows.size(1), dtype=f8, device=dev)
        xs = torch.empty(cap, rows.size(1) // 128, dtype=torch.float32, device=dev)
        act = torch.empty(cap, inter, dtype=torch.bfloat16, device=dev)
        aq = torch.empty(cap, inter, dtype=f8, device=dev)
        as_ = torch.empty(cap, inter // 128, dtype=torch.float32, device=dev)
        ops.moe_act_quant_fp8_scatter(rows, xq, xs, slot_pos, sorted_ids, num_post, 1)
        ops.moe_gemm_fp8_sorted(act, xq, xs, w13, w13_scale, sorted_ids, expert_ids, num_post, None,
                                r, bm, True, "silu", True)
        ops.moe_act_quant_fp8_sorted(act, aq, as_, None, num_post, 1, r)
        ops.moe_gemm_fp8_sorted(y, aq, as_, w2, w2_scale, sorted_ids, expert_ids, num_post, weights,
                                r, bm, False, "silu", False)
        return y

    return run


def ep_moe_fp8(x, logits, w13, w13_scale, w2, w2_scale, top_k, group=None, block_m=None):
    """One expert-parallel FP8 W8A8 block-scaled MoE layer; arguments as
    ep_moe_mxfp4 with the FP8 weight tensors of this rank's experts."""
    from . import moe as _moe

    weights, ids = _moe.route(logits, top_k)
    t, h = x.shape

    def combine(slots):
        out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
        torch.ops.strix.moe_sum(slots, out)
        return out

    return ep_dispatch_combine(x, weights, ids, w13.size(0),
                               local_experts_fp8(w13, w13_scale, w2, w2_scale, block_m), group,
                               combine)


def ep_moe_mxfp4(x, logits, w13, w13_scale, w2, w2_scale, top_k, group=None, block_m=None):
    """One expert-parallel MXFP4 MoE layer. x bf16 [T_local, H]; logits fp32
    [T_local, E_global]; the weight tensors hold this rank's E_global / world
    experts. Router and combine run on this rank's tokens, the experts where
    they live. Returns bf16 [T_local, H]."""
    from . import moe as _moe

    weights, ids = _moe.route(logits, top_k)
    t, h = x.shape

    def combine(slots):
        out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
        torch.ops.strix.moe_sum(slots, out)
        return out

    return ep_dispatch_combine(x, weights, ids, w13.size(0),
                               local_experts_mxfp4(w13, w13_scale, w2, w2_scale, block_m),
                               group, combine)
