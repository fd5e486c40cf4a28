"""Expert-parallel dispatch / combine on CPU ranks (gloo, world size 2): the
bookkeeping of libstrix_b200.ep against a single-process computation, with a
plain torch expert function standing in for the GPU kernels. The GPU test runs
the MXFP4 experts through the same code on however many GPUs are visible."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

E_GLOBAL, TOP_K, H = 8, 3, 16


def expert_weights():
    g = torch.Generator().manual_seed(7)
    return torch.randn(E_GLOBAL, H, H, generator=g) / H ** 0.5


def rank_inputs(rank, tokens):
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(tokens, H, generator=g)
    ids = torch.stack([torch.randperm(E_GLOBAL, generator=g)[:TOP_K] for _ in range(tokens)]) \
        if tokens else torch.zeros(0, TOP_K, dtype=torch.int64)
    w = torch.rand(tokens, TOP_K, generator=g)
    return x, w, ids.int()


def dense_reference(x, w, ids):
    wts = expert_weights()
    out = torch.zeros_like(x)
    for t in range(x.size(0)):
        for j in range(ids.size(1)):
            out[t] += w[t, j] * (wts[ids[t, j]] @ x[t])
    return out


def _worker(rank, world, port, tokens_per_rank, skew, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from libstrix_b200 import ep

        per = E_GLOBAL // world
        wts = expert_weights()[rank * per:(rank + 1) * per]
        x, w, ids = rank_inputs(rank, tokens_per_rank[rank])
        if skew:                      # every slot of every rank goes to rank 0's experts
            ids = ids % per
        seen = {}

        def local_fn(rows, local_ids, weights):
            seen["rows"] = rows.size(0)
            assert local_ids.dtype == torch.int32 and bool((local_ids < per).all())
            y = torch.einsum("rij,rj->ri", wts[local_ids.long()], rows)
            return y * weights[:, None]

        out = ep.ep_dispatch_combine(x, w, ids, per, local_fn)
        ref = dense_reference(x, w, ids)
        err = float((out - ref).abs().max()) if out.numel() else 0.0
        results[rank] = (err, seen["rows"])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens_per_rank,skew", [([5, 9], False), ([0, 7], False), ([6, 6], True)])
def test_dispatch_combine_two_ranks(tokens_per_rank, skew):
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29600 + (os.getpid() + sum(tokens_per_rank) + int(skew)) % 300
    mp.spawn(_worker, args=(2, port, tokens_per_rank, skew, results), nprocs=2, join=True)
    assert set(results.keys()) == {0, 1}
    for rank in (0, 1):
        err, rows = results[rank]
        assert err < 1e-5, f"rank {rank}: max error {err}"
    total = sum(tokens_per_rank) * TOP_K
    assert results[0][1] + results[1][1] == total           # every slot was computed once
    if skew:
        assert results[1][1] == 0                            # and where its expert lives


def test_dispatch_plan_is_stable_and_counts():
    from libstrix_b200 import ep

    ids = torch.tensor([[5, 0], [1, 6], [7, 2]])
    order, counts = ep.dispatch_plan(ids, 4, 2)
    assert counts.tolist() == [3, 3]
    assert order.tolist() == [1, 2, 5, 0, 3, 4]              # rank 0's slots first, in slot order


def test_placement_table_and_balancing():
    """Host logic of expert placement: the table the kernels read, the rank each slot
    goes to, and the balanced placement with copies of hot experts."""
    from libstrix_b200 import ep

    pl = ep.Placement([[0, 1, 2], [3, 4, 0], [5, 6], [7, 0]], 8)
    tab = pl.table("cpu")
    assert tab[:2].tolist() == [8, 4]                              # experts, row stride (1 + 3 copies)
    rows = tab[2:].view(8, 4)
    assert rows[0].tolist() == [3, (0 << 16) | 0, (1 << 16) | 2, (3 << 16) | 1]
    assert rows[5].tolist() == [1, (2 << 16) | 0, -1, -1]
    ids = torch.tensor([[0, 5], [0, 3], [0, 7], [0, 1]], dtype=torch.int32)
    assert pl.rank_of(ids).tolist() == [[0, 2], [1, 1], [3, 3], [0, 0]]   # token t -> copy t mod 3
    with pytest.raises(ValueError, match="every expert needs a rank"):
        ep.Placement([[0], [1]], 3)
    # one expert with 40 % of the load: no placement without copies can balance 4 ranks
    loads = [400.0] + [600.0 / 15] * 15
    plain = ep.Placement.balanced(loads, 4)
    spare = ep.Placement.balanced(loads, 4, slots_per_rank=5)

    def ratio(p):
        per = [0.0] * p.world
        for e, where in enumerate(p.where):
            for w in where:
                per[w >> 16] += loads[e] / len(where)
        return max(per) / (sum(per) / p.world)

    assert all(len(r) == 4 for r in plain.ranks) and ratio(plain) > 1.5
    assert all(len(r) <= 5 for r in spare.ranks) and ratio(spare) < 1.1
    assert len(spare.where[0]) >= 2 and len({w >> 16 for w in spare.where[0]}) == len(spare.where[0])


@pytest.mark.gpu
def test_ep_moe_mxfp4_matches_oracle_on_visible_gpus():
    """World size 1 on one GPU (the all-to-alls degenerate to copies): the
    whole EP path against the CPU oracle of the MXFP4 layer."""
    from libstrix_b200 import ep
    from oracle import gemm as G
    from oracle import moe as M

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29711", RANK="0", WORLD_SIZE="1")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        t, e, k, hid, inter = 70, 8, 2, 256, 128
        g = torch.Generator().manual_seed(0)
        x = torch.randn(t, hid, generator=g).bfloat16()
        logits = torch.randn(t, e, generator=g)
        w13 = torch.randint(0, 256, (e, 2 * inter, hid // 2), generator=g, dtype=torch.uint8)
        s13 = torch.randint(118, 124, (e, 2 * inter, hid // 32), generator=g, dtype=torch.uint8)
        w2 = torch.randint(0, 256, (e, hid, inter // 2), generator=g, dtype=torch.uint8)
        s2 = torch.randint(118, 124, (e, hid, inter // 32), generator=g, dtype=torch.uint8)
        out = ep.ep_moe_mxfp4(x.cuda(), logits.cuda(), w13.cuda(), s13.cuda(), w2.cuda(), s2.cuda(), k)
        ids, wts = M.router(logits, k)
        h1 = M.gate_mul(M.grouped_reference(x, G.mxfp4_dequant(w13, s13), ids, k, None), "silu")
        h1 = h1.bfloat16()
        y = M.grouped_reference(h1, G.mxfp4_dequant(w2, s2), ids, 1, wts).bfloat16()
        ref = y.view(t, k, hid).float().sum(1)
        err = (out.float().cpu() - ref).abs()
        rms = ref.pow(2).mean().sqrt()
        assert bool((err <= 2e-2 * rms + ref.abs() * 2.0 ** -8).all()), f"{err.max()} vs rms {rms}"
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_ep_moe_fp8_equals_the_single_rank_layer():
    """World size 1: the EP path with FP8 local experts against the fused layer
    and the CPU oracle (same kernels, different permutation bookkeeping)."""
    import libstrix_b200 as strix
    from libstrix_b200 import ep
    from libstrix_b200.workloads import moe_fp8_layer
    from oracle import moe as M

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29712", RANK="0", WORLD_SIZE="1")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        layer = moe_fp8_layer(tokens=70, seed=2, device="cuda")
        out = ep.ep_moe_fp8(layer.x, layer.logits, layer.w13, layer.w13_scale, layer.w2,
                            layer.w2_scale, layer.top_k)
        cpu = layer.to("cpu")
        ref, _, _ = M.moe_fp8_layer(cpu.x, cpu.logits, cpu.w13, cpu.w13_scale, cpu.w2, cpu.w2_scale,
                                    cpu.top_k)
        err = (out.float().cpu() - ref.float()).abs()
        rms = ref.float().pow(2).mean().sqrt()
        assert bool((err <= 2e-2 * rms + ref.float().abs() * 2.0 ** -8).all()), f"{err.max()} vs {rms}"
        fused = strix.moe.fused_moe_fp8_w8a8(layer.x, layer.logits, layer.w13, layer.w13_scale,
                                             layer.w2, layer.w2_scale, layer.top_k)
        torch.testing.assert_close(out.float(), fused.float(), rtol=2e-2, atol=2e-2)
    finally:
        dist.destroy_process_group()


def _gpu_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from libstrix_b200 import ep
        from libstrix_b200 import moe as smoe

        e, k, hid, inter = 8, 2, 256, 128
        per = e // world
        g = torch.Generator().manual_seed(0)          # the same experts on every rank
        w13 = torch.randint(0, 256, (e, 2 * inter, hid // 2), generator=g, dtype=torch.uint8).to(dev)
        s13 = torch.randint(118, 124, (e, 2 * inter, hid // 32), generator=g, dtype=torch.uint8).to(dev)
        w2 = torch.randint(0, 256, (e, hid, inter // 2), generator=g, dtype=torch.uint8).to(dev)
        s2 = torch.randint(118, 124, (e, hid, inter // 32), generator=g, dtype=torch.uint8).to(dev)
        gr = torch.Generator().manual_seed(100 + rank)  # each rank's own tokens
        t = 50 + 30 * rank
        x = torch.randn(t, hid, generator=gr).bfloat16().to(dev)
        logits = torch.randn(t, e, generator=gr).to(dev)
        lo = rank * per
        out = ep.ep_moe_mxfp4(x, logits, w13[lo:lo + per].contiguous(), s13[lo:lo + per].contiguous(),
                              w2[lo:lo + per].contiguous(), s2[lo:lo + per].contiguous(), k)
        # the same layer without parallelism: all experts here, this rank's tokens
        weights, ids = smoe.route(logits, k)
        run = ep.local_experts_mxfp4(w13, s13, w2, s2)
        rows = x.repeat_interleave(k, 0)
        y = run(rows, ids.reshape(-1).to(torch.int32), weights.reshape(-1).contiguous())
        ref = torch.empty(t, hid, dtype=torch.bfloat16, device=dev)
        torch.ops.strix.moe_sum(y.view(t, k, hid), ref)
        torch.cuda.synchronize()
        results[rank] = float((out.float() - ref.float()).abs().max()), float(ref.float().abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ep_moe_mxfp4_two_gpus_equals_unsharded_layer():
    """Two NCCL ranks, each with its own tokens and half of the experts, against
    the same layer computed on one rank with all experts: a row's result does not
    depend on where or in which m-block it was computed."""
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_gpu_worker, args=(2, 29741, results), nprocs=2, join=True)
    for rank in (0, 1):
        err, peak = results[rank]
        assert err <= 1e-2 * peak, f"rank {rank}: max error {err} vs peak {peak}"


# ------------------------------------------------- peer-memory exchange (GPU kernels)
def _bound_ok(out, ref):
    err = (out.float().cpu() - ref.float()).abs()
    rms = ref.float().pow(2).mean().sqrt()
    return bool((err <= 2e-2 * rms + ref.float().abs() * 2.0 ** -8).all()), float(err.max()), float(rms)


@pytest.mark.gpu
@pytest.mark.parametrize("placement", ["contiguous", "round_robin", "table"])
@pytest.mark.parametrize("kind", ["mxfp4", "fp8"])
@pytest.mark.parametrize("tokens_per_rank", [[70, 0, 33, 128], [1, 1, 1, 1]])
def test_peer_exchange_with_emulated_ranks(kind, tokens_per_rank, placement):
    _emulated_exchange(kind, tokens_per_rank, placement)


@pytest.mark.gpu
def test_peer_exchange_eight_emulated_ranks_balanced_placement():
    """Eight ranks, sixteen experts of which one draws a third of the load: the
    balanced placement (three expert slots per rank) replicates it, and the layer
    still matches the oracle of the unsharded layer."""
    from libstrix_b200 import ep

    loads = [40.0] + [80.0 / 15] * 15
    place = ep.Placement.balanced(loads, 8, slots_per_rank=3)
    assert len(place.where[0]) >= 2
    _emulated_exchange("mxfp4", [5, 0, 9, 1, 33, 2, 7, 64], "table", world=8, e_global=16, place=place)


def _emulated_exchange(kind, tokens_per_rank, placement, world=4, e_global=8, place=None):
    """Four ranks emulated in one process on one GPU (the phases of all ranks run in
    lockstep, so no kernel ever waits for one that has not been launched): plan,
    dispatch, receive, local experts, return and combine against the CPU oracle of
    the unsharded layer, with the experts in contiguous blocks per rank, placed
    round-robin (expert e on rank e mod 4), or by a table in which expert 0 has three
    copies (its tokens are spread over them) and the ranks hold 3, 3, 2 and 2 experts."""
    from libstrix_b200 import ep
    from libstrix_b200 import moe as smoe
    from libstrix_b200.workloads import moe_fp8_layer, moe_mxfp4_layer
    from oracle import moe as M

    dev = torch.device("cuda", 0)
    k, hid, inter = 2, 256, 128
    per = e_global // world
    rr = placement == "round_robin"
    if placement == "table" and place is None:
        place = ep.Placement([[0, 1, 2], [3, 4, 0], [5, 6], [7, 0]], e_global)
    table = place.table(dev) if place else None
    total = sum(tokens_per_rank)
    if kind == "mxfp4":
        layer = moe_mxfp4_layer(tokens=256, hidden=hid, experts=e_global, top_k=k, inter=inter, seed=3)
        ref, _, _ = M.moe_mxfp4_layer(layer.x[:total], layer.logits[:total], layer.w13, layer.w13_scale,
                                      layer.w2, layer.w2_scale, k)
        row_bytes = hid * 2
    else:
        layer = moe_fp8_layer(tokens=256, hidden=hid, experts=e_global, top_k=k, inter=inter, seed=3)
        ref, _, _ = M.moe_fp8_layer(layer.x[:total], layer.logits[:total], layer.w13, layer.w13_scale,
                                    layer.w2, layer.w2_scale, k)
        row_bytes = ep.fp8_row_bytes(hid)
    g = layer.to(dev)
    ctxs = ep.EpContext.emulate(world, max(tokens_per_rank), k, row_bytes, hid, dev)
    try:
        offs = [sum(tokens_per_rank[:r]) for r in range(world + 1)]
        for rounds in range(2):                       # twice: the epoch stamps must carry over
            for r, ctx in enumerate(ctxs):
                x, logits = g.x[offs[r]:offs[r + 1]], g.logits[offs[r]:offs[r + 1]]
                weights, ids = smoe.route(logits, k)
                payload = x if kind == "mxfp4" else ep.fp8_payload(x)[0]
                ctx.dispatch(payload, weights, ids, -per if rr else per, placement=table)
            for r, ctx in enumerate(ctxs):
                sl = slice(r, None, world) if rr else slice(r * per, (r + 1) * per)
                if place:
                    sl = torch.tensor(place.ranks[r], device=dev)
                if kind == "mxfp4":
                    y = ep._experts_mxfp4_on_received(ctx, g.w13[sl].contiguous(), g.w13_scale[sl].contiguous(),
                                                      g.w2[sl].contiguous(), g.w2_scale[sl].contiguous())
                else:
                    y = ep._experts_fp8_on_received(ctx, g.w13[sl].contiguous(), g.w13_scale[sl].contiguous(),
                                                    g.w2[sl].contiguous(), g.w2_scale[sl].contiguous(), 128)
                ctx.send_back(y)
            outs = [ctx.combine() for ctx in ctxs]
            torch.cuda.synchronize()
            assert ctxs[0].status() == 0
            # every token reached each rank that owns one of its experts exactly once
            got = torch.stack([c.rows_per_source for c in ctxs]).cpu()       # [dest, src]
            ids_all, _ = M.router(layer.logits[:total], k)
            for r in range(world):
                mine = ids_all[offs[r]:offs[r + 1]] % world if rr else ids_all[offs[r]:offs[r + 1]] // per
                if place:
                    mine = place.rank_of(ids_all[offs[r]:offs[r + 1]])
                for d in range(world):
                    assert int(got[d, r]) == int((mine == d).any(-1).sum())
            for r in range(world):
                if tokens_per_rank[r] == 0:
                    assert outs[r].shape == (0, hid)
                    continue
                ok, err, rms = _bound_ok(outs[r], ref[offs[r]:offs[r + 1]])
                assert ok, f"round {rounds} rank {r}: max err {err} vs rms {rms}"
    finally:
        for c in ctxs:
            c.close()


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["mxfp4", "fp8"])
@pytest.mark.parametrize("tokens", [70, 1])
def test_one_call_layer_on_a_single_rank(kind, tokens):
    """strix_ep_moe_layer (router, payload, dispatch, experts, return, combine in one
    call) on a world of one - the rank sends to itself, so every wait is for a kernel
    launched earlier on the same stream - against the CPU oracle, twice in a row
    (the epoch stamps carry over) and with fewer tokens than the capacity."""
    from libstrix_b200 import ep
    from libstrix_b200.workloads import moe_fp8_layer, moe_mxfp4_layer
    from oracle import moe as M

    dev = torch.device("cuda", 0)
    e, k, hid, inter = 8, 2, 256, 128
    if kind == "mxfp4":
        layer = moe_mxfp4_layer(tokens=128, hidden=hid, experts=e, top_k=k, inter=inter, seed=5)
        oracle, row_bytes, code, bm = M.moe_mxfp4_layer, hid * 2, 0, 128
    else:
        layer = moe_fp8_layer(tokens=128, hidden=hid, experts=e, top_k=k, inter=inter, seed=5)
        oracle, row_bytes, code, bm = M.moe_fp8_layer, ep.fp8_row_bytes(hid), 2, 128
    g = layer.to(dev)
    ctx = ep.EpContext.emulate(1, 100, k, row_bytes, hid, dev)[0]
    try:
        for n in (tokens, min(tokens + 20, 100)):
            ref, _, _ = oracle(layer.x[:n], layer.logits[:n], layer.w13, layer.w13_scale, layer.w2,
                               layer.w2_scale, k)
            out = ctx.layer(g.x[:n], g.logits[:n], g.w13, g.w13_scale, g.w2, g.w2_scale, code, bm)
            torch.cuda.synchronize()
            assert ctx.status() == 0
            ok, err, rms = _bound_ok(out, ref)
            assert ok, f"{n} tokens: max err {err} vs rms {rms}"
    finally:
        ctx.close()


@pytest.mark.gpu
def test_peer_exchange_waits_are_bounded():
    """A flag that nothing sets: the receive and combine kernels give up after the
    given number of polls, raise the status word and deliver empty input."""
    from libstrix_b200 import ep

    dev = torch.device("cuda", 0)
    ctx = ep.EpContext.emulate(2, 8, 2, 64, 32, dev)[0]     # its "peer" never dispatches
    try:
        ctx.epoch, ctx.tokens = 5, 4
        ctx.tok_pos = torch.zeros(2, 4, dtype=torch.int32, device=dev)
        _, ids, _ = ctx.receive(spin_limit=50)
        torch.cuda.synchronize()
        assert ctx.status(reset=True) == 1 and bool((ids == -1).all())
        out = ctx.combine(spin_limit=50)
        torch.cuda.synchronize()
        assert ctx.status(reset=True) == 2 and bool((out == 0).all())
        assert ctx.status() == 0
    finally:
        ctx.close()


@pytest.mark.gpu
def test_masked_expert_ids_have_no_position():
    """Slots whose expert id is -1 (masked) or out of range get slot_pos -1 and are
    skipped by the scatter kernels."""
    from libstrix_b200 import moe as smoe

    ids = torch.tensor([[0, -1], [3, 1], [-1, -1], [2, 9]], dtype=torch.int32, device="cuda")
    sorted_ids, expert_ids, num_post, slot_pos = smoe.align_with_positions(ids, 4, 4)
    pos = slot_pos.cpu().tolist()
    assert [p >= 0 for p in pos] == [True, False, True, True, False, False, True, False]
    assert int(num_post) == 16
    srt = sorted_ids.cpu()[:16].view(4, 4)
    assert srt[:, 0].tolist() == [0, 3, 6, 2] and bool((srt[:, 1:] == 8).all())
    x = torch.arange(4 * 8, dtype=torch.float32, device="cuda").view(4, 8).bfloat16()
    y = torch.full((sorted_ids.numel(), 8), -1.0, dtype=torch.bfloat16, device="cuda")
    torch.ops.strix.moe_permute_bf16(x, y, slot_pos, sorted_ids, num_post, 2)
    assert torch.equal(y[pos[0]], x[0]) and torch.equal(y[pos[2]], x[1]) and torch.equal(y[pos[6]], x[3])
