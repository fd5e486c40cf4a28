"""Expert-parallel MoE: token dispatch -> local experts -> combine.

Every rank holds `experts_per_rank` consecutive experts and its own tokens. A
token travels to every rank that owns one of its top-k experts, is computed
there with the grouped GEMMs of this library, and one partial row per (token,
rank) travels back; the source rank sums them.

Two exchanges are implemented:

  * peer memory (the GPU path, `EpContext`): this library's own kernels write
    payload rows, metadata, counts and epoch flags straight into the peers'
    buffers over NVLink (csrc/ep_exchange.cu). No host synchronisation, no
    collective call per layer; a token is sent once per destination rank; the
    FP8 layer quantises before dispatch (e4m3 bytes + per-128 scales travel, a
    quarter of the bf16 payload is saved twice over); received rows are scattered
    straight into the expert-sorted layout of the tcgen05 GEMMs.
  * collectives (`ep_dispatch_combine`): `all_to_all_single` over the process
    group with split sizes on the host - the portable form, which the CPU tests
    run over gloo and which serves as fallback where peer mappings are refused.

The reference has no expert parallelism (its experts refuse an `expert_map`,
python/strix_vllm/moe.py:193-210); this is the path the 8-GPU configuration
needs.
"""

from __future__ import annotations

import ctypes
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


# --------------------------------------------------------------- peer memory
def _no_mark(name: str) -> None:
    pass


class _RawCuda:
    """A cudaMalloc allocation presented through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}


_BUFFERS = ("recv", "meta", "counts", "flags", "ret", "rflags")


class _ExpertWeights(ctypes.Structure):
    """strix_expert_weights of the header."""
    _fields_ = [("w13", ctypes.c_void_p), ("w13_scale", ctypes.c_void_p), ("w2", ctypes.c_void_p),
                ("w2_scale", ctypes.c_void_p)] + \
               [(n, ctypes.c_int64) for n in ("w13_stride_e", "w13_stride_n", "s13_stride_e", "s13_stride_n",
                                              "w2_stride_e", "w2_stride_n", "s2_stride_e", "s2_stride_n",
                                              "experts", "hidden", "inter")] + \
               [("kind", ctypes.c_int32), ("gate_act", ctypes.c_int32)]


class _Exchange(ctypes.Structure):
    """strix_ep_exchange of the header."""
    _fields_ = [(n, ctypes.c_int64) for n in ("world", "rank", "cap", "top_k", "row_bytes", "hidden",
                                              "epoch", "round_robin")] + \
               [("placement", ctypes.c_void_p), ("experts_global", ctypes.c_int64)] + \
               [("peer_" + n, ctypes.POINTER(ctypes.c_void_p)) for n in _BUFFERS] + \
               [(n, ctypes.c_void_p) for n in ("ticket", "ids", "weights", "rows_per_source", "y", "tok_pos",
                                               "counts")]


def _expert_weights(w13, w13_scale, w2, w2_scale, kind: int) -> _ExpertWeights:
    e, n13 = w13.size(0), w13.size(1)
    hidden, inter = w2.size(1), n13 // 2
    block = kind == 2
    per_row = kind == 0 or block     # scale tensors with a row stride ([E, N, K/32] or [E, N/128, K/128])
    return _ExpertWeights(
        w13.data_ptr(), w13_scale.data_ptr(), w2.data_ptr(), w2_scale.data_ptr(),
        w13.stride(0), w13.stride(1), w13_scale.stride(0), w13_scale.stride(1) if per_row else 0,
        w2.stride(0), w2.stride(1), w2_scale.stride(0), w2_scale.stride(1) if per_row else 0,
        e, hidden, inter, kind, 1)


class EpContext:
    """One rank's buffers for the peer-memory exchange, plus the addresses of
    every peer's buffers as this rank sees them.

    cap: tokens a source rank may send (its token count at most); row_bytes: the
    payload row (a multiple of 16); hidden: width of the result rows (bf16).
    Build with `EpContext.create(group, ...)` (one per process, CUDA IPC between
    the ranks of one node) or `EpContext.emulate(world, ...)` (all ranks in this
    process on one device, for tests: the phases of the ranks then run in
    lockstep, never concurrently)."""

    def __init__(self, world, rank, cap, top_k, row_bytes, hidden, device):
        from . import _lib

        self.world, self.rank, self.cap, self.top_k = world, rank, cap, top_k
        self.row_bytes, self.hidden, self.device = row_bytes, hidden, torch.device(device)
        self.epoch = 0
        self._lib = _lib
        self._imported: list[int] = []
        meta_ints = 1 + 2 * top_k
        sizes = {"recv": world * cap * row_bytes, "meta": world * cap * meta_ints * 4,
                 "counts": 256, "flags": 256, "ret": world * cap * hidden * 2, "rflags": 256}
        self.ptr: dict[str, int] = {}
        self.t: dict[str, torch.Tensor] = {}
        with torch.cuda.device(self.device):
            for name, nbytes in sizes.items():
                p = ctypes.c_void_p()
                _lib.call("strix_peer_alloc", ctypes.byref(p), nbytes)
                self.ptr[name] = p.value
                self.t[name] = torch.as_tensor(_RawCuda(p.value, nbytes), device=self.device)
        self.peer: dict[str, list[int]] = {}
        i32 = dict(dtype=torch.int32, device=self.device)
        self.ticket = torch.zeros(2, **i32)
        self.ids = torch.empty(world * cap, top_k, **i32)
        self.weights = torch.empty(world * cap, top_k, dtype=torch.float32, device=self.device)
        self.rows_per_source = torch.zeros(world, **i32)
        self.y = torch.empty(world * cap * top_k, hidden, dtype=torch.bfloat16, device=self.device)
        self.tok_pos = torch.empty(world, cap, **i32)    # used as [world, tokens] of the call
        self.counts = torch.empty(world, **i32)

    # ---- construction
    @classmethod
    def create(cls, group, cap, top_k, row_bytes, hidden, device):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ctx = cls(world, rank, cap, top_k, row_bytes, hidden, device)
        handles = {}
        for name in _BUFFERS:
            h = (ctypes.c_uint8 * 64)()
            ctx._lib.call("strix_peer_export", ctx.ptr[name], h)
            handles[name] = bytes(h)
        gathered = [None] * world
        dist.all_gather_object(gathered, handles, group=group)
        with torch.cuda.device(ctx.device):
            for name in _BUFFERS:
                ptrs = []
                for r in range(world):
                    if r == rank:
                        ptrs.append(ctx.ptr[name])
                        continue
                    p = ctypes.c_void_p()
                    ctx._lib.call("strix_peer_import", gathered[r][name], ctypes.byref(p))
                    ctx._imported.append(p.value)
                    ptrs.append(p.value)
                ctx.peer[name] = ptrs
        dist.barrier(group=group)
        return ctx

    @classmethod
    def emulate(cls, world, cap, top_k, row_bytes, hidden, device):
        ctxs = [cls(world, r, cap, top_k, row_bytes, hidden, device) for r in range(world)]
        for c in ctxs:
            for name in _BUFFERS:
                c.peer[name] = [o.ptr[name] for o in ctxs]
        return ctxs

    def close(self):
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self._imported:
                self._lib.call("strix_peer_unimport", p)
            self._imported = []
            self.t = {}
            for name, p in self.ptr.items():
                self._lib.call("strix_peer_free", p)
            self.ptr = {}

    def _ptrs(self, name):
        return (ctypes.c_void_p * self.world)(*self.peer[name])

    # ---- the exchange phases (each enqueues kernels on the current stream)
    def dispatch(self, payload: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                 experts_per_rank: int, mark=_no_mark, placement: torch.Tensor | None = None):
        """payload [T, row_bytes worth of elements] (last dim contiguous) goes to every
        rank that owns one of the token's experts (experts_per_rank < 0: round-robin
        placement, expert e on rank e mod world; `placement`: a table from
        placement_table() instead). `mark(name)` is called after each kernel is
        enqueued (a hook for per-phase timing)."""
        t, k = topk_ids.shape
        assert k == self.top_k and t <= self.cap
        assert payload.size(1) * payload.element_size() == self.row_bytes and payload.stride(1) == 1
        self.epoch += 1
        self.tokens = t
        ids = topk_ids.to(torch.int32).contiguous()
        wts = topk_weights.to(torch.float32).contiguous()
        stream = torch.cuda.current_stream().cuda_stream
        call = self._lib.call
        with torch.cuda.device(self.device):
            table = None if placement is None else placement.data_ptr()
            call("strix_ep_plan", ids.data_ptr(), self.tok_pos.data_ptr(), self.counts.data_ptr(), t, k,
                 experts_per_rank, self.world, table, stream)
            mark("plan")
            call("strix_ep_dispatch", payload.data_ptr(), ids.data_ptr(), wts.data_ptr(),
                 self.tok_pos.data_ptr(), self.counts.data_ptr(), self._ptrs("recv"), self._ptrs("meta"),
                 self._ptrs("counts"), self._ptrs("flags"), self.ticket.data_ptr(), t, self.row_bytes,
                 payload.stride(0) * payload.element_size(), k, experts_per_rank, self.world, self.rank,
                 self.cap, self.epoch, table, stream)
            mark("dispatch")

    def receive(self, spin_limit: int = 0):
        """Waits (on the device) for every source; returns (rows uint8 [world * cap,
        row_bytes], ids int32 [world * cap, top_k] with -1 where nothing arrived,
        weights fp32 of the same shape)."""
        stream = torch.cuda.current_stream().cuda_stream
        with torch.cuda.device(self.device):
            self._lib.call("strix_ep_prepare", self.ptr["meta"], self.ptr["counts"], self.ptr["flags"],
                           self.ids.data_ptr(), self.weights.data_ptr(), self.rows_per_source.data_ptr(),
                           self.world, self.cap, self.top_k, self.epoch, spin_limit, stream)
        rows = self.t["recv"][: self.world * self.cap * self.row_bytes].view(self.world * self.cap,
                                                                             self.row_bytes)
        return rows, self.ids, self.weights

    def send_back(self, y: torch.Tensor):
        """y bf16 [world * cap * top_k, hidden], slot order, weighted: one summed row
        per received token goes back to its source."""
        stream = torch.cuda.current_stream().cuda_stream
        with torch.cuda.device(self.device):
            self._lib.call("strix_ep_return", y.data_ptr(), self.ids.data_ptr(), self.ptr["meta"],
                           self.ptr["counts"], self._ptrs("ret"), self._ptrs("rflags"),
                           self.ticket.data_ptr() + 4, self.world, self.rank, self.cap, self.top_k,
                           self.hidden, y.stride(0), self.epoch, stream)

    def combine(self, out: torch.Tensor | None = None, spin_limit: int = 0) -> torch.Tensor:
        """Waits for every rank's return; out[t] = sum of token t's partial rows."""
        t = self.tokens
        if out is None:
            out = torch.empty(t, self.hidden, dtype=torch.bfloat16, device=self.device)
        stream = torch.cuda.current_stream().cuda_stream
        with torch.cuda.device(self.device):
            self._lib.call("strix_ep_combine", self.ptr["ret"], self.ptr["rflags"], self.tok_pos.data_ptr(),
                           out.data_ptr(), t, self.hidden, out.stride(0) if t else self.hidden, self.world,
                           self.cap, self.epoch, spin_limit, stream)
        return out

    def layer(self, x, logits, w13, w13_scale, w2, w2_scale, kind: int, block_m: int,
              out: torch.Tensor | None = None, spin_limit: int = 0, round_robin: bool = False,
              placement: torch.Tensor | None = None) -> torch.Tensor:
        """One expert-parallel layer as ONE call into the library (strix_ep_moe_layer):
        router, payload, dispatch, this rank's experts over what it receives, return
        and combine. kind 0 MXFP4 experts over bf16 rows, 1 / 2 FP8 W8A8 experts
        (channel / block scales) over e4m3 rows."""
        t, h = x.shape
        assert t <= self.cap and h == self.hidden and x.stride(1) == 1 and logits.stride(1) == 1
        assert x.dtype == torch.bfloat16 and logits.dtype == torch.float32
        self.epoch += 1
        self.tokens = t
        if out is None:
            out = torch.empty(t, h, dtype=torch.bfloat16, device=self.device)
        keep = {n: self._ptrs(n) for n in _BUFFERS}        # host arrays the struct points into
        ex = _Exchange(self.world, self.rank, self.cap, self.top_k, self.row_bytes, self.hidden, self.epoch,
                       int(round_robin), None if placement is None else placement.data_ptr(),
                       logits.size(1), *[ctypes.cast(keep[n], ctypes.POINTER(ctypes.c_void_p)) for n in _BUFFERS],
                       self.ticket.data_ptr(), self.ids.data_ptr(), self.weights.data_ptr(),
                       self.rows_per_source.data_ptr(), self.y.data_ptr(), self.tok_pos.data_ptr(),
                       self.counts.data_ptr())
        wt = _expert_weights(w13, w13_scale, w2, w2_scale, kind)
        lib = self._lib.load()
        need = lib.strix_ep_moe_layer_workspace(ctypes.byref(wt), ctypes.byref(ex), block_m)
        if need < 0:
            raise RuntimeError(lib.strix_last_error().decode())
        ws = getattr(self, "_layer_ws", None)
        if ws is None or ws.numel() < need + 256:
            ws = self._layer_ws = torch.empty(need + 256, dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            self._lib.call("strix_ep_moe_layer", out.data_ptr(), x.data_ptr(), logits.data_ptr(),
                           ctypes.byref(wt), ctypes.byref(ex), (ws.data_ptr() + 255) // 256 * 256, need, t,
                           x.stride(0), logits.stride(0), out.stride(0) if t else h, block_m, spin_limit,
                           torch.cuda.current_stream().cuda_stream)
            self._lib.after_tcgen05("ep_moe_layer")
        return out

    def status(self, reset: bool = False) -> int:
        flag = ctypes.c_int32(-1)
        with torch.cuda.device(self.device):
            self._lib.call("strix_ep_status", ctypes.byref(flag), int(reset))
        return flag.value


def _experts_mxfp4_on_received(ctx: EpContext, w13, w13_scale, w2, w2_scale, mark=_no_mark):
    """The received tokens through this rank's MXFP4 experts; returns y in slot order."""
    from . import moe as _moe

    rows, ids, weights = ctx.receive()
    mark("receive_wait")
    e = w13.size(0)
    inter = w13.size(1) // 2
    ops = torch.ops.strix
    sorted_ids, expert_ids, num_post, slot_pos = _moe.align_with_positions(ids, 128, e)
    mark("align")
    cap_s = sorted_ids.numel()
    dev = ctx.device
    xs = torch.empty(cap_s, ctx.row_bytes // 2, dtype=torch.bfloat16, device=dev)
    act = torch.empty(cap_s, inter, dtype=torch.bfloat16, device=dev)
    ops.moe_permute_rows(rows, xs.view(torch.uint8), slot_pos, sorted_ids, num_post, ctx.top_k)
    mark("permute")
    n_slots = ids.numel()
    ops.moe_gemm_mxfp4_sorted(act, xs, w13, w13_scale, sorted_ids, expert_ids, num_post, None, n_slots,
                              128, True, "silu", True)
    mark("gemm_gate_up")
    ops.moe_gemm_mxfp4_sorted(ctx.y, act, w2, w2_scale, sorted_ids, expert_ids, num_post,
                              weights.view(-1), n_slots, 128, False, "silu", False)
    mark("gemm_down")
    return ctx.y


def _experts_fp8_on_received(ctx: EpContext, w13, w13_scale, w2, w2_scale, block_m, mark=_no_mark):
    """The received (already quantised) tokens through this rank's FP8 experts."""
    from . import moe as _moe

    rows, ids, weights = ctx.receive()
    mark("receive_wait")
    e, n13, h = w13.shape
    inter = n13 // 2
    if mark is _no_mark and w13_scale.stride(-1) == 1 and w2_scale.stride(-1) == 1:
        # no phase timing wanted: the five launches as ONE call into the library
        from . import _lib
        n_rows, key = ids.size(0), (ids.size(0), ctx.top_k, h, inter, e, block_m)
        ws = getattr(ctx, "_fp8_ws", None)
        if ws is None or ws.key != key:
            ws = ctx._fp8_ws = _moe.Fp8LayerWorkspace(n_rows, ctx.top_k, h, inter, e, block_m, ctx.device,
                                                      with_out=False)
        block = w13_scale.dim() == 3 and w13_scale.size(1) != n13
        _lib.call("strix_moe_fp8_experts_on_rows", ctx.y.data_ptr(), rows.data_ptr(), weights.data_ptr(),
                  ids.data_ptr(), w13.data_ptr(), w13_scale.data_ptr(), w2.data_ptr(), w2_scale.data_ptr(),
                  ws.ptr, ws.nbytes, n_rows, h, inter, e, ctx.top_k, block_m, rows.stride(0),
                  ctx.y.stride(0), w13.stride(0), w13.stride(1), w13_scale.stride(0),
                  w13_scale.stride(1) if block else 0, w2.stride(0), w2.stride(1), w2_scale.stride(0),
                  w2_scale.stride(1) if block else 0, 2 if block else 1, 1,
                  torch.cuda.current_stream().cuda_stream)
        _lib.after_tcgen05("ep_moe_fp8")
        return ctx.y
    ops = torch.ops.strix
    f8 = torch.float8_e4m3fn
    sorted_ids, expert_ids, num_post, slot_pos = _moe.align_with_positions(ids, block_m, e)
    mark("align")
    cap_s = sorted_ids.numel()
    dev = ctx.device
    srt = torch.empty(cap_s, ctx.row_bytes, dtype=torch.uint8, device=dev)
    ops.moe_permute_rows(rows, srt, slot_pos, sorted_ids, num_post, ctx.top_k)
    mark("permute")
    xq, xs = srt[:, :h].view(f8), srt[:, h:h + h // 32].view(torch.float32)
    act = torch.empty(cap_s, inter, dtype=torch.bfloat16, device=dev)
    aq = torch.empty(cap_s, inter, dtype=f8, device=dev)
    as_ = torch.empty(cap_s, inter // 128, dtype=torch.float32, device=dev)
    n_slots = ids.numel()
    ops.moe_gemm_fp8_sorted(act, xq, xs, w13, w13_scale, sorted_ids, expert_ids, num_post, None, n_slots,
                            block_m, True, "silu", True)
    mark("gemm_gate_up")
    ops.moe_act_quant_fp8_sorted(act, aq, as_, None, num_post, 1, n_slots)
    mark("act_quant")
    ops.moe_gemm_fp8_sorted(ctx.y, aq, as_, w2, w2_scale, sorted_ids, expert_ids, num_post,
                            weights.view(-1), n_slots, block_m, False, "silu", False)
    mark("gemm_down")
    return ctx.y


_CONTEXTS: dict[tuple, EpContext] = {}


def context_for(group, tokens, top_k, row_bytes, hidden, device) -> EpContext:
    """The cached EpContext of this (group, payload shape). It is built on first use
    - a collective: every rank must reach it together - with a capacity of the
    largest token count over the ranks at that moment; later calls may bring
    fewer tokens, never more (build an EpContext of your own for a larger batch)."""
    key = (id(group), top_k, row_bytes, hidden, str(device))
    ctx = _CONTEXTS.get(key)
    if ctx is None:
        if not dist.is_initialized():       # a single process: the rank exchanges with itself
            ctx = _CONTEXTS[key] = EpContext.emulate(1, max(tokens, 1), top_k, row_bytes, hidden, device)[0]
        else:
            ctx = _CONTEXTS[key] = EpContext.create(group, _capacity(tokens, group), top_k, row_bytes,
                                                    hidden, device)
    if tokens > ctx.cap:
        raise RuntimeError(f"{tokens} tokens exceed the exchange capacity {ctx.cap} set at first use")
    return ctx


def close_contexts() -> None:
    for ctx in _CONTEXTS.values():
        ctx.close()
    _CONTEXTS.clear()


def fp8_row_bytes(hidden: int) -> int:
    """Bytes of an FP8 payload row: `hidden` e4m3 bytes, hidden / 128 fp32 scales,
    padded to whole 16-byte chunks."""
    return (hidden + hidden // 32 + 15) // 16 * 16


def fp8_payload(x: torch.Tensor, buf: torch.Tensor | None = None):
    """(payload uint8 [T, fp8_row_bytes(H)], q view, scale view): x quantised to e4m3
    per (token, 128 group) with the fp32 scales behind each row's bytes - what the
    FP8 layer sends instead of bf16 rows."""
    t, h = x.shape
    row = fp8_row_bytes(h)
    if buf is None or buf.size(0) != t or buf.size(1) != row or buf.device != x.device:
        buf = torch.zeros(t, row, dtype=torch.uint8, device=x.device)
    q, s = buf[:t, :h].view(torch.float8_e4m3fn), buf[:t, h:h + h // 32].view(torch.float32)
    torch.ops.strix.moe_act_quant_fp8(x, q, s)
    return buf[:t], q, s


def ep_moe_fp8(x, logits, w13, w13_scale, w2, w2_scale, top_k, group=None, block_m=None,
               exchange="auto", ctx=None, mark=_no_mark, placement="contiguous"):
    """One expert-parallel FP8 W8A8 block-scaled MoE layer. x bf16 [T_local, H];
    logits fp32 [T_local, E_global]; the weight tensors hold this rank's E_global /
    world experts. Returns bf16 [T_local, H]. exchange: "peer" (this library's
    kernels over peer memory), "nccl" (all_to_all_single) or "auto" (peer on CUDA;
    a single rank runs the fused single-GPU layer, which is the same computation
    without an exchange). placement: which rank owns which expert - "contiguous"
    (rank r holds the experts [r E/N, (r + 1) E/N)) or "round_robin" (rank r holds r,
    r + N, r + 2N, ...: its local expert i is global expert i N + r), which balances
    a load that is skewed along the expert index, or a `Placement` (any assignment,
    hot experts replicated: `Placement.balanced(loads, world, slots_per_rank)`); the
    weight tensors then hold placement.ranks[rank] in that order. Peer exchange only."""
    from . import moe as _moe

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rr = _round_robin(placement, exchange, x)
    table = placement.table(x.device) if isinstance(placement, Placement) else None
    t, h = x.shape
    if world == 1 and exchange == "auto" and ctx is None:
        return _moe.fused_moe_fp8_w8a8(x, logits, w13, w13_scale, w2, w2_scale, top_k, block_m=block_m)
    if exchange == "nccl" or not x.is_cuda:
        weights, ids = _moe.route(logits, top_k)

        def combine(slots):
            out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
            torch.ops.strix.moe_sum(slots, out)
            return out

        return ep_dispatch_combine(x, weights, ids, w13.size(0),
                                   local_experts_fp8(w13, w13_scale, w2, w2_scale, block_m), group,
                                   combine)
    e_local = w13.size(0)
    row_bytes = fp8_row_bytes(h)
    if ctx is None:
        ctx = context_for(group, t, top_k, row_bytes, h, x.device)
    bm = block_m or _moe.pick_block_m(t * ctx.world, top_k, e_local * ctx.world)
    if not _moe.sorted_path_covers(w13, w13_scale, w2, w2_scale, bm):
        raise RuntimeError("ep_moe_fp8: geometry not covered by the sorted-layout kernel")
    if mark is _no_mark and _one_call_ok(x, logits, w13_scale, w2_scale):
        block = w13_scale.dim() == 3 and w13_scale.size(1) != w13.size(1)
        return ctx.layer(x, logits, w13, w13_scale, w2, w2_scale, 2 if block else 1, bm, round_robin=rr,
                         placement=table)
    weights, ids = _moe.route(logits, top_k)
    mark("route")
    payload, _, _ = fp8_payload(x, getattr(ctx, "_payload", None))
    ctx._payload = payload          # the padding bytes were zeroed once, at allocation
    mark("quantise")
    ctx.dispatch(payload, weights, ids, -e_local if rr else e_local, mark, placement=table)
    y = _experts_fp8_on_received(ctx, w13, w13_scale, w2, w2_scale, bm, mark)
    ctx.send_back(y)
    mark("return")
    out = ctx.combine()
    mark("combine_wait")
    return out


def ep_moe_mxfp4(x, logits, w13, w13_scale, w2, w2_scale, top_k, group=None, block_m=None,
                 exchange="auto", ctx=None, mark=_no_mark, placement="contiguous"):
    """One expert-parallel MXFP4 MoE layer. x bf16 [T_local, H]; logits fp32
    [T_local, E_global]; the weight tensors hold this rank's E_global / world
    experts. Router and combine run on this rank's tokens, the experts where
    they live. Returns bf16 [T_local, H]. `exchange` and `placement` as in
    ep_moe_fp8."""
    from . import _lib
    from . import moe as _moe

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rr = _round_robin(placement, exchange, x)
    table = placement.table(x.device) if isinstance(placement, Placement) else None
    t, h = x.shape
    lib = _lib.load()
    wide_ok = bool(lib.strix_moe_gemm_mxfp4_sorted_covers(w13.size(1), w13.size(2) * 2, 128, 1)
                   and lib.strix_moe_gemm_mxfp4_sorted_covers(w2.size(1), w2.size(2) * 2, 128, 0))
    if world == 1 and exchange == "auto" and ctx is None and x.is_cuda:
        return _moe.fused_moe_mxfp4(x, logits, w13, w13_scale, w2, w2_scale, top_k, block_m=block_m)
    peer = exchange != "nccl" and x.is_cuda and wide_ok and (h * 2) % 16 == 0
    if peer and mark is _no_mark and _one_call_ok(x, logits, w13_scale, w2_scale):
        if ctx is None:
            ctx = context_for(group, t, top_k, h * 2, h, x.device)
        return ctx.layer(x, logits, w13, w13_scale, w2, w2_scale, 0, 128, round_robin=rr, placement=table)
    weights, ids = _moe.route(logits, top_k)
    if not peer:
        def combine(slots):
            out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
            torch.ops.strix.moe_sum(slots, out)
            return out

        return ep_dispatch_combine(x, weights, ids, w13.size(0),
                                   local_experts_mxfp4(w13, w13_scale, w2, w2_scale, block_m),
                                   group, combine)
    if ctx is None:
        ctx = context_for(group, t, top_k, h * 2, h, x.device)
    mark("route")
    ctx.dispatch(x, weights, ids, -w13.size(0) if rr else w13.size(0), mark, placement=table)
    y = _experts_mxfp4_on_received(ctx, w13, w13_scale, w2, w2_scale, mark)
    ctx.send_back(y)
    mark("return")
    out = ctx.combine()
    mark("combine_wait")
    return out


class Placement:
    """Which rank holds which expert, as a table: `ranks[r]` lists the global experts
    rank r holds, in the order of its weight tensors (its local expert i is global
    expert ranks[r][i]). An expert may appear on several ranks: a replicated hot
    expert, whose tokens are spread over the copies (token t goes to copy t mod
    copies). `table(device)` is the int32 tensor the exchange kernels read."""

    def __init__(self, ranks: list[list[int]], experts: int):
        self.ranks, self.experts, self.world = [list(r) for r in ranks], experts, len(ranks)
        where: list[list[int]] = [[] for _ in range(experts)]
        for r, held in enumerate(self.ranks):
            for i, e in enumerate(held):
                where[e].append((r << 16) | i)
        if any(not w for w in where):
            raise ValueError("every expert needs a rank")
        self.max_copies = max(len(w) for w in where)
        self.where = where
        self._tables: dict[str, torch.Tensor] = {}

    def table(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self._tables:
            stride = 1 + self.max_copies
            rows = [[len(w)] + w + [-1] * (self.max_copies - len(w)) for w in self.where]
            flat = [self.experts, stride] + [v for row in rows for v in row]
            self._tables[key] = torch.tensor(flat, dtype=torch.int32, device=device)
        return self._tables[key]

    def rank_of(self, topk_ids: torch.Tensor) -> torch.Tensor:
        """The rank that serves each slot of topk_ids [T, k] (token t = row t): the
        table's rule, on whatever device the ids are."""
        dev = topk_ids.device
        tab = self.table(dev)[2:].view(self.experts, 1 + self.max_copies)
        e = topk_ids.long()
        t = torch.arange(e.size(0), device=dev).view(-1, 1).expand_as(e)
        copy = t % tab[e, 0].long()
        return tab[e, 1 + copy] >> 16

    @classmethod
    def balanced(cls, loads, world: int, slots_per_rank: int | None = None) -> "Placement":
        """Longest-processing-time placement of `loads` (expected routed slots per
        expert) with at most `slots_per_rank` experts per rank (default: experts /
        world, no copies). Spare slots are spent on copies of whichever expert has the
        largest load per copy; copies of one expert go to different ranks."""
        loads = [float(v) for v in loads]
        experts = len(loads)
        per = slots_per_rank or -(-experts // world)
        if per * world < experts:
            raise ValueError("not enough expert slots")
        copies = [1] * experts
        for _ in range(per * world - experts):
            e = max(range(experts), key=lambda i: loads[i] / copies[i])
            if copies[e] >= world or loads[e] / copies[e] <= sum(loads) / (world * per):
                break
            copies[e] += 1
        items = sorted(((loads[e] / copies[e], e) for e in range(experts) for _ in range(copies[e])),
                       reverse=True)
        ranks: list[list[int]] = [[] for _ in range(world)]
        total = [0.0] * world
        for w, e in items:
            free = [r for r in range(world) if len(ranks[r]) < per and e not in ranks[r]]
            r = min(free, key=lambda i: total[i])
            ranks[r].append(e)
            total[r] += w
        return cls(ranks, experts)


def _round_robin(placement, exchange: str, x) -> bool:
    if isinstance(placement, Placement):
        if exchange == "nccl" or not x.is_cuda:
            raise ValueError("a placement table needs the peer-memory exchange")
        return False
    if placement not in ("contiguous", "round_robin"):
        raise ValueError(f"placement must be 'contiguous', 'round_robin' or a Placement, got {placement!r}")
    if placement == "round_robin" and (exchange == "nccl" or not x.is_cuda):
        raise ValueError("round_robin placement needs the peer-memory exchange")
    return placement == "round_robin"


def _one_call_ok(x, logits, w13_scale, w2_scale) -> bool:
    """Layouts strix_ep_moe_layer takes as they are."""
    return x.dtype == torch.bfloat16 and x.stride(1) == 1 and logits.dtype == torch.float32 \
        and logits.stride(1) == 1 and w13_scale.stride(-1) == 1 and w2_scale.stride(-1) == 1


def _capacity(tokens: int, group) -> int:
    """Rows a source may send: the largest token count over the ranks (one small
    collective with a host read, at context creation only)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return max(tokens, 1)
    dev = torch.device("cuda", torch.cuda.current_device())
    n = torch.tensor([tokens], dtype=torch.int64, device=dev)
    dist.all_reduce(n, op=dist.ReduceOp.MAX, group=group)
    return max(int(n.item()), 1)
