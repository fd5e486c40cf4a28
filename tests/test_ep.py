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
