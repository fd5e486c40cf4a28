#!/usr/bin/env python
"""Benchmark of the libstrix_b200 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Primary workload (config 3 of the baseline): paged decode attention over an
int8 KV cache - 64 sequences per GPU, one query token each, 32 query heads / 4 KV
heads, head_dim 128, block_size 16, context lengths ~ U[1024, 65536], block
tables a random permutation of the physical blocks. One step = one pass of the
kernel over the whole batch. Metric: algorithmic KV bytes read per second
(every live key's K and V rows and their two fp32 scales), summed over GPUs.
With N > 1 (torchrun) every rank owns an independent batch of 64 sequences
(no data-path collective; "weak" scaling).

`value` is timed with the inputs resident in HBM; `e2e` is the same metric
through the public call (libstrix_b200.attn_decode) with the step's inputs
(queries, sequence lengths, block table) in pinned host memory, copied in
inside the timed region, and the output copied back; the KV cache is resident
state, like model weights. `--impl reference` times the CPU oracle (the
reference's torch implementation restated, oracle/attention.py) on the host
cores over a bounded sample of the same batch.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "int8-KV paged decode attention, algorithmic KV bytes read per second"
UNIT = "GB/s"
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of the decode kernel,
# from an ncu capture of the 32-sequence case (committed summary under profiles/)
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = (1_183_573_248 + 16_128_000) / 1_182_370_464
WORKLOAD = ("decode_attn_int8kv B=64/gpu Hq=32 Hkv=4 D=128 block=16 ctx~U[1024,65536] "
            "shuffled block table")


def measured_peaks() -> tuple[float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu)], stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
        except OSError:
            self.proc = None

    def stop(self) -> dict | None:
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [r.split(", ") for r in Path(self.path).read_text().splitlines() if r.strip()]
        os.unlink(self.path)
        rows = [r for r in rows if len(r) >= 9]
        if not rows:
            return None
        sm = [float(r[1]) for r in rows]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            for name, v in zip(names, r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][2]),
                "reasons": sorted(reasons), "samples": len(rows)}


def cpu_oracle_sample(batch, nseq_sample: int, repeats: int = 1):
    """Times the CPU oracle on the first `nseq_sample` sequences of the batch.
    Returns (GB/s, seconds, threads, description, output)."""
    from oracle import attention as A

    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    lens = batch.seq_lens[:nseq_sample].cpu()
    parts, tables, ofs = [], [], 0
    maxb = max((int(x) + 15) // 16 for x in lens)
    table = torch.zeros(nseq_sample, maxb, dtype=torch.int32)
    for n in range(nseq_sample):
        nb = (int(lens[n]) + 15) // 16
        parts.append(batch.block_table[n, :nb].long().cpu())
        table[n, :nb] = torch.arange(ofs, ofs + nb, dtype=torch.int32)
        ofs += nb
    blocks = torch.cat(parts).to(batch.key_cache.device)
    kc, vc = batch.key_cache[blocks].cpu(), batch.value_cache[blocks].cpu()
    ks, vs = batch.k_scale[blocks].cpu(), batch.v_scale[blocks].cpu()
    q = batch.q[:nseq_sample].cpu()
    best, out = float("inf"), None
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = A.decode_reference(q, kc, vc, ks, vs, lens, table, batch.scale)
        best = min(best, time.perf_counter() - t0)
    nbytes = int(lens.sum()) * kc.size(2) * (2 * q.size(-1) + 8)
    desc = (f"first {nseq_sample} of 64 sequences ({int(lens.sum())} keys, {nbytes / 1e6:.0f} MB "
            f"of KV), torch fp32 on {threads} threads, dequantise + dense softmax")
    return nbytes / best / 1e9, best, threads, desc, out


def run_reference(args, rank: int) -> None:
    """--impl reference: the CPU oracle on the host cores, rank 0 only."""
    if rank != 0:
        return
    from libstrix_b200.workloads import decode_batch

    # A bounded sample of the seed-0 batch: its first sequences, cut so that the
    # whole run (warm-up + steps) stays near two minutes of CPU time. The cut is
    # calibrated on one 8,192-key sequence.
    gen = torch.Generator().manual_seed(0)
    all_lens = torch.randint(1024, 65536 + 1, (64,), generator=gen, dtype=torch.int64).tolist()
    cal = decode_batch(ctx_lens=[8192], seed=0)
    cpu_oracle_sample(cal, 1)
    _, cal_sec, _, _, _ = cpu_oracle_sample(cal, 1)
    budget = int(8192 / cal_sec * 120.0 / max(1, args.warmup + args.steps))
    budget = max(4096, min(budget, 160_000))
    lens, left = [], budget
    for n in all_lens:
        if left <= 0 or len(lens) == 4:
            break
        lens.append(min(n, left))
        left -= lens[-1]
    batch = decode_batch(ctx_lens=lens, seed=0)
    times, gbs = [], []
    for i in range(args.warmup + args.steps):
        v, sec, threads, desc, _ = cpu_oracle_sample(batch, len(lens))
        if i >= args.warmup:
            times.append(sec)
            gbs.append(v)
    value = statistics.mean(gbs)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * statistics.mean(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": desc},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--num-splits", type=int, default=0, help="0 = fixed 1024-key segments")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx-hi", type=int, default=65536)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-moe", action="store_true", help="skip the MoE FP8 layer runs")
    ap.add_argument("--only", choices=["moe", "gemm", "prefill", "ep"], default=None,
                    help="run one secondary section alone (for profiling) and print its JSON")
    ap.add_argument("--moe-tokens", type=int, nargs="*", default=[256, 4096])
    ap.add_argument("--gemm-m", type=int, nargs="*", default=[1, 16, 4096])
    ap.add_argument("--prefill-tokens", type=int, nargs="*", default=[2048, 65536])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist

    import libstrix_b200 as strix
    from libstrix_b200.workloads import decode_batch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.only == "ep":
        res = bench_ep_moe(args, dev, rank, world)
        if rank == 0:
            print(json.dumps({"ep": res}), flush=True)
        if dist.is_initialized():
            dist.destroy_process_group()
        return
    if args.only is not None:
        if rank == 0:
            section = {"moe": bench_moe_fp8, "gemm": bench_gemm_w8a8,
                       "prefill": bench_attn_prefill}[args.only]
            print(json.dumps({args.only: section(args, dev, not args.no_cpu_baseline)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # weak scaling: every rank holds a batch with the SAME context lengths (seed 0), so
    # the per-GPU work is fixed as N grows; the tensors are each rank's own
    batch = decode_batch(batch=args.batch, ctx_hi=args.ctx_hi, seed=0, device=dev)
    kv_bytes = batch.kv_bytes
    out = torch.empty_like(batch.q)
    nseg = strix._lib.load().strix_attn_decode_segments(
        args.num_splits, batch.block_table.size(1), 16)
    launches_per_step = 2 if nseg > 1 else 1

    def step():
        strix.attn_decode(out, batch.q, batch.key_cache, batch.value_cache, batch.seq_lens,
                          batch.block_table, batch.scale, args.num_splits, -1, batch.k_scale,
                          batch.v_scale)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()

    # ---- kernel-resident timing: K steps, CUDA events on the launching stream
    sampler = ClockSampler(local_rank)
    sampler.start()
    # keep the GPU busy long enough for nvidia-smi to see clocks under load
    t_end = time.perf_counter() + 0.6
    while time.perf_counter() < t_end:
        step()
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    clocks = sampler.stop()

    # ---- end to end: step inputs from pinned host memory, output read back
    q_h = batch.q.cpu().pin_memory()
    sl_h = batch.seq_lens.cpu().pin_memory()
    bt_h = batch.block_table.cpu().pin_memory()
    out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    q_d, sl_d, bt_d = torch.empty_like(batch.q), torch.empty_like(batch.seq_lens), \
        torch.empty_like(batch.block_table)

    def e2e_step():
        q_d.copy_(q_h, non_blocking=True)
        sl_d.copy_(sl_h, non_blocking=True)
        bt_d.copy_(bt_h, non_blocking=True)
        strix.attn_decode(out, q_d, batch.key_cache, batch.value_cache, sl_d, bt_d, batch.scale,
                          args.num_splits, -1, batch.k_scale, batch.v_scale)
        out_h.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    # ---- reduce over ranks: max time, summed bytes
    stats = torch.tensor([total_ms, e2e_ms, float(kv_bytes)], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = stats.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = stats.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms, all_bytes = tmax[0].item(), tmax[1].item(), tsum[2].item()
    else:
        all_bytes = float(kv_bytes)

    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = all_bytes / (ms_per_step * 1e-3) / 1e9
        e2e_value = all_bytes / (e2e_ms / args.steps * 1e-3) / 1e9
        peak, peak_kind = measured_peaks()
        # the dominant kernel's own duration: the step minus nothing else on the
        # stream (the reduce kernel is included; it is < 2 % of the step)
        achieved = kv_bytes / (statistics.mean(per_step) * 1e-3) / 1e9 if world == 1 else \
            value / world
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 mma / f32 softmax over int8 KV",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "kv_bytes_per_gpu": kv_bytes,
                       "segments": int(nseg), "l2": "inputs (2.2 GB) larger than the 126 MB L2",
                       "timing": "cuda events, max over ranks"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         # DRAM read + write bytes per launch: measured with ncu on the 32-sequence
                         # case (1,183.6 + 16.1 MB for 1,182.4 MB algorithmic) and scaled by the keys
                         "traffic": kv_bytes * DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE,
                         "traffic_note": "ncu capture at batch 32 scaled to this launch by its keys",
                         "peak_kind": peak_kind,
                         "frac_of_8TBps": achieved / 8000.0},
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": int(q_h.nbytes + sl_h.nbytes + bt_h.nbytes),
                    "d2h_bytes_per_step": int(out_h.nbytes)},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            v, sec, threads, desc, ref = cpu_oracle_sample(batch, 4)
            diff = (out[:4].float().cpu() - ref).abs()
            rms = ref.pow(2).mean().sqrt().item()
            # bound: 2e-2 x RMS plus the bf16 output quantum (half an ulp, at most 2^-8 |ref|)
            ok = bool((diff <= 2e-2 * rms + ref.abs() * 2.0 ** -8).all())
            worst = int(diff.argmax())
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": desc, "seconds": sec}
            line["parity"] = {"max_abs_err": diff.max().item(), "ref_rms": rms,
                              "ref_at_max_err": ref.view(-1)[worst].item(),
                              "max_abs_ref": ref.abs().max().item(), "ok": ok}
        if world == 1 and not args.no_moe:
            del batch
            torch.cuda.empty_cache()
            line["moe_fp8"] = bench_moe_fp8(args, dev, not args.no_cpu_baseline)
            line["gpu_launches"] += line["moe_fp8"]["gpu_launches"]
            line["gemm_w8a8_int8"] = bench_gemm_w8a8(args, dev, not args.no_cpu_baseline)
            line["gpu_launches"] += line["gemm_w8a8_int8"]["gpu_launches"]
            line["attn_prefill"] = bench_attn_prefill(args, dev, not args.no_cpu_baseline)
            line["gpu_launches"] += line["attn_prefill"]["gpu_launches"]
    # the expert-parallel MXFP4 layer runs on every rank (it is a collective)
    ep_res = None if args.no_moe else bench_ep_moe(args, dev, rank, world)
    if rank == 0:
        if ep_res is not None:
            line["ep_moe_mxfp4"] = ep_res
            line["gpu_launches"] += ep_res["gpu_launches"]
        print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


def bench_moe_fp8(args, dev, with_cpu: bool) -> dict:
    """The MoE half of the compound metric: one FP8 W8A8 block-scaled layer at
    256 tokens (config 1: hidden 2048, 128 experts, top-8, intermediate 768) and,
    for the tensor-bound regime, at 4096 tokens. At 256 tokens every expert is
    hit with ~16 rows, so the layer is bound by streaming the 604 MB of expert
    weights once: GB/s of weight bytes against the HBM roofline is reported
    beside TFLOP/s. Weights (604 MB) exceed the 126 MB L2."""
    import libstrix_b200 as strix
    from libstrix_b200.moe import pick_block_m, workspace_for
    from libstrix_b200.workloads import moe_fp8_layer

    peak, peak_kind = measured_peaks()
    out = {"config": "MoE FP8 W8A8 block-scaled, H=2048 E=128 top-8 I=768", "gpu_launches": 0,
           "runs": []}
    for tokens in args.moe_tokens:
        layer = moe_fp8_layer(tokens=tokens, seed=0, device=dev)
        ws = workspace_for(tokens, layer.top_k, 2048, 768, 128, pick_block_m(tokens, layer.top_k, 128), dev)

        def step():
            return strix.moe.fused_moe_fp8_w8a8(layer.x, layer.logits, layer.w13, layer.w13_scale,
                                                layer.w2, layer.w2_scale, layer.top_k, ws=ws)

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            res = step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        # the same seven launches replayed from a CUDA graph (how a serving loop runs
        # decode steps): an empty kernel costs 5 us per eager launch on this system
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                step()
        torch.cuda.synchronize()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms_graph = e0.elapsed_time(e1) / args.steps
        del graph
        gbs = layer.weight_bytes / (ms * 1e-3) / 1e9
        run = {"tokens": tokens, "ms_per_layer": ms, "tflops": layer.flops / (ms * 1e-3) / 1e12,
               "ms_per_layer_cuda_graph": ms_graph,
               "tflops_cuda_graph": layer.flops / (ms_graph * 1e-3) / 1e12,
               "weight_gbs_cuda_graph": layer.weight_bytes / (ms_graph * 1e-3) / 1e9,
               "weight_gbs": gbs, "weight_bytes": layer.weight_bytes,
               "block_m": pick_block_m(tokens, layer.top_k, 128),
               "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s",
                            "frac": gbs / peak, "peak_kind": peak_kind}}
        out["gpu_launches"] += 7 * args.steps
        if with_cpu and tokens == 256:
            from oracle import moe as M

            cpu = layer.to("cpu")
            threads = len(os.sched_getaffinity(0))
            torch.set_num_threads(threads)
            t0 = time.perf_counter()
            ref, _, _ = M.moe_fp8_layer(cpu.x, cpu.logits, cpu.w13, cpu.w13_scale, cpu.w2,
                                        cpu.w2_scale, cpu.top_k)
            sec = time.perf_counter() - t0
            diff = (res.float().cpu() - ref.float()).abs()
            rms = ref.float().pow(2).mean().sqrt().item()
            run["cpu_baseline"] = {"value": layer.flops / sec / 1e12, "unit": "TFLOP/s",
                                   "cores": threads, "kind": "port", "seconds": sec,
                                   "sample": "the whole 256-token layer, torch fp32 incl. dequantisation"}
            run["parity"] = {"max_abs_err": diff.max().item(), "ref_rms": rms,
                             "ok": bool((diff <= 2e-2 * rms + ref.float().abs() * 2.0 ** -8).all())}
        out["runs"].append(run)
        del layer, ws
        torch.cuda.empty_cache()
    return out


def bench_gemm_w8a8(args, dev, with_cpu: bool) -> dict:
    """Dense W8A8 INT8 GEMM of config 2: K=5120, N=34816 (a 27B-like MLP gate-up),
    M in {1, 16, 4096}. The decode rows (M <= 16) stream the 178 MB of weights
    once per launch - HBM roofline; every launch reads another of six weight
    copies (1.07 GB in rotation, far beyond the 126 MB L2). M = 4096 is tensor
    bound: TOPS against twice the measured bf16 peak (the int8 rate is nominally
    twice the bf16 rate; no int8 library GEMM was measured on this pool)."""
    from oracle import gemm as G

    hbm, peak_kind = measured_peaks()
    f = ROOT / "MEASURED_PEAKS.json"
    bf16 = float(json.loads(f.read_text())["bf16_tflops"]) if f.exists() else 1590.0
    n, k, copies = 34816, 5120, 6
    g = torch.Generator(device=dev).manual_seed(0)
    ws = [torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8, device=dev)
          for _ in range(copies)]
    sw = torch.rand(n, generator=g, device=dev) * 9e-3 + 1e-3
    out = {"config": "dense W8A8 INT8 GEMM K=5120 N=34816, int32-exact sums, bf16 out",
           "gpu_launches": 0, "runs": []}
    op = torch.ops.strix.w8a8_int8_gemm
    for m in args.gemm_m:
        a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8, device=dev)
        sa = torch.rand(m, generator=g, device=dev) * 4e-2 + 1e-2
        for i in range(max(args.warmup, 3)):
            res = op(a, sa, ws[i % copies], sw)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            res = op(a, sa, ws[i % copies], sw)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        byts = n * k + m * k + 2 * m * n
        tops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        gbs = byts / (ms * 1e-3) / 1e9
        roof = ({"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                 "peak_kind": peak_kind} if m <= 64 else
                {"bound": "tensor", "achieved": tops, "peak": 2 * bf16, "unit": "TOP/s",
                 "frac": tops / (2 * bf16), "peak_kind": "2 x measured bf16 (derived)"})
        run = {"m": m, "ms_per_launch": ms, "tops": tops, "gbs": gbs, "bytes": byts,
               "roofline": roof}
        out["gpu_launches"] += args.steps
        if with_cpu and m == 16:
            last = ws[(args.steps - 1) % copies]
            rows = torch.arange(0, n, 17, device=dev)
            t0 = time.perf_counter()
            ref, acc = G.w8a8_int8_gemm(a.cpu(), sa.cpu(), last[rows].cpu(), sw[rows].cpu())
            sec = time.perf_counter() - t0
            run["cpu_baseline"] = {"value": 2.0 * m * rows.numel() * k / sec / 1e12, "unit": "TOP/s",
                                   "cores": torch.get_num_threads(), "kind": "port",
                                   "seconds": sec, "sample": f"M=16, every 17th output channel ({rows.numel()})"}
            run["parity"] = {"bit_exact_bf16": bool(torch.equal(res[:, rows].cpu().view(torch.int16),
                                                                ref.view(torch.int16)))}
        out["runs"].append(run)
    return out


def bench_ep_moe(args, dev, rank: int, world: int) -> dict:
    """Config 5: MXFP4 MoE layer, gpt-oss-120B-like (hidden 2880, 128 experts, top-4,
    intermediate 2880), 8192 tokens in total, expert-parallel over the ranks:
    each rank holds 8192 / N tokens and 128 / N experts; tokens move by NCCL
    all-to-all (dispatch and combine). Router logits N(0,1) plus a Zipf(1.1)
    per-expert bias. Strong scaling: the total work is fixed. Time = max over
    ranks of the CUDA-event time; TFLOP/s counts 2 x slots x (2I x H + H x I)."""
    import torch.distributed as dist

    from libstrix_b200 import ep

    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29517")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    tokens_total, hid, inter, experts, top_k = 8192, 2880, 2880, 128, 4
    t_local, e_local = tokens_total // world, experts // world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x = torch.randn(t_local, hid, generator=g, device=dev, dtype=torch.bfloat16)
    zipf = torch.log(1.0 / torch.arange(1, experts + 1, device=dev, dtype=torch.float32) ** 1.1)
    zipf = zipf[torch.randperm(experts, generator=torch.Generator(device=dev).manual_seed(7), device=dev)]
    logits = torch.randn(t_local, experts, generator=g, device=dev) + zipf
    w13 = torch.randint(0, 256, (e_local, 2 * inter, hid // 2), generator=g, device=dev, dtype=torch.uint8)
    s13 = torch.randint(118, 124, (e_local, 2 * inter, hid // 32), generator=g, device=dev, dtype=torch.uint8)
    w2 = torch.randint(0, 256, (e_local, hid, inter // 2), generator=g, device=dev, dtype=torch.uint8)
    s2 = torch.randint(118, 124, (e_local, hid, inter // 32), generator=g, device=dev, dtype=torch.uint8)

    def step():
        return ep.ep_moe_mxfp4(x, logits, w13, s13, w2, s2, top_k)

    steps = max(2, min(args.steps, 10))
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ok = bool(torch.isfinite(out.float()).all())
    flops = 2.0 * tokens_total * top_k * (2 * inter * hid + hid * inter)
    ms = ms.item()
    fp8 = _bench_ep_fp8(dev, rank, world, steps)
    return {"fp8": fp8,
            "config": "MXFP4 MoE, H=2880 E=128 top-4 I=2880, 8192 tokens, EP over ranks, Zipf(1.1) bias",
            "n_gpus": world, "scaling": "strong", "ms_per_layer": ms,
            "tflops": flops / (ms * 1e-3) / 1e12, "tokens_per_s": tokens_total / (ms * 1e-3),
            "weight_bytes_per_rank": int(w13.numel() + s13.numel() + w2.numel() + s2.numel()),
            "finite": ok, "gpu_launches": 5 * steps,
            "exchange": "NCCL all_to_all_single x4 per layer (counts, rows, ids+weights, results)"}


def _bench_ep_fp8(dev, rank: int, world: int, steps: int) -> dict:
    """The FP8 W8A8 layer of config 1 (H=2048, E=128, top-8, I=768) expert-parallel:
    4096 tokens in total, 4096 / N per rank, 128 / N experts per rank; local
    experts on the sorted-layout tcgen05 kernels. Strong scaling."""
    import torch.distributed as dist

    from libstrix_b200 import ep
    from libstrix_b200.workloads import moe_fp8_layer

    tokens_total, experts = 4096, 128
    layer = moe_fp8_layer(tokens=tokens_total // world, seed=10 + rank, device=dev)
    e_local = experts // world
    lo = rank * e_local
    w13, s13 = layer.w13[lo:lo + e_local].contiguous(), layer.w13_scale[lo:lo + e_local].contiguous()
    w2, s2 = layer.w2[lo:lo + e_local].contiguous(), layer.w2_scale[lo:lo + e_local].contiguous()
    x, logits, top_k = layer.x, layer.logits, layer.top_k
    flops_total = layer.flops * world
    del layer
    torch.cuda.empty_cache()

    def step():
        return ep.ep_moe_fp8(x, logits, w13, s13, w2, s2, top_k)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = ms.item()
    return {"config": "FP8 W8A8 MoE, H=2048 E=128 top-8 I=768, 4096 tokens, EP over ranks",
            "n_gpus": world, "scaling": "strong", "ms_per_layer": ms,
            "tflops": flops_total / (ms * 1e-3) / 1e12, "tokens_per_s": tokens_total / (ms * 1e-3),
            "finite": bool(torch.isfinite(out.float()).all())}


def bench_attn_prefill(args, dev, with_cpu: bool) -> dict:
    """Causal GQA prefill of config 4: one sequence of 2048 and of 65536 tokens, 40
    query / 8 KV heads, head 128, int8 paged cache (block 16, shuffled table)
    written from bf16 N(0,1) values with per-token-per-head scales. Tensor bound:
    FLOPs = 4 x Hq x D x T (T + 1) / 2 (QK^T and PV over the causal half) against
    the measured bf16 peak. Q + out (1.3 GB at 65536 tokens) exceed the L2."""
    import libstrix_b200 as strix
    from oracle import attention as A

    f = ROOT / "MEASURED_PEAKS.json"
    bf16 = float(json.loads(f.read_text())["bf16_tflops"]) if f.exists() else 1590.0
    hq, hkv, hd, bs = 40, 8, 128, 16
    out = {"config": "causal GQA prefill, Hq=40 Hkv=8 D=128 block=16, int8 KV", "gpu_launches": 0,
           "runs": []}
    g = torch.Generator(device=dev).manual_seed(0)
    for t in args.prefill_tokens:
        nblk = (t + bs - 1) // bs
        kv = torch.randn(nblk, bs, hkv, 2 * hd, generator=g, device=dev, dtype=torch.bfloat16)
        kq, ks = A.quantize_kv(kv[..., :hd])
        vq, vs = A.quantize_kv(kv[..., hd:])
        del kv
        table = torch.randperm(nblk, generator=g, device=dev).int().view(1, nblk)
        q = torch.randn(t, hq, hd, generator=g, device=dev, dtype=torch.bfloat16)
        o = torch.empty_like(q)
        cu = torch.tensor([0, t], dtype=torch.int32, device=dev)
        sl = torch.tensor([t], dtype=torch.int32, device=dev)
        scale = hd ** -0.5

        def step():
            strix.attn_prefill(o, q, kq, vq, cu, sl, table, scale, 1, -1, ks, vs)

        steps = max(2, min(args.steps, 5 if t > 8192 else args.steps))
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        flops = 4.0 * hq * hd * t * (t + 1) / 2
        tf = flops / (ms * 1e-3) / 1e12
        run = {"tokens": t, "ms": ms, "tflops": tf, "flops": flops,
               "roofline": {"bound": "tensor", "achieved": tf, "peak": bf16, "unit": "TFLOP/s",
                            "frac": tf / bf16, "peak_kind": "measured bf16 (cuBLAS burst)"}}
        out["gpu_launches"] += steps
        if with_cpu and t <= 2048:
            n_q = 256   # the last 256 queries against the whole context
            t0 = time.perf_counter()
            kx, vx = (kq.float() * ks[..., None]).cpu(), (vq.float() * vs[..., None]).cpu()
            ref = A.attention_reference(q[-n_q:].cpu(), kx, vx, torch.tensor([0, n_q], dtype=torch.int32),
                                        sl.cpu(), table.cpu(), scale)
            sec = time.perf_counter() - t0
            diff = (o[-n_q:].float().cpu() - ref).abs()
            rms = ref.pow(2).mean().sqrt().item()
            run["cpu_baseline"] = {"value": 4.0 * hq * hd * n_q * (t - n_q / 2) / sec / 1e12,
                                   "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                   "seconds": sec, "sample": f"last {n_q} of {t} queries"}
            run["parity"] = {"max_abs_err": diff.max().item(), "ref_rms": rms,
                             "ok": bool((diff <= 2e-2 * rms + ref.abs() * 2.0 ** -8).all())}
        out["runs"].append(run)
        del q, o, kq, vq, ks, vs
        torch.cuda.empty_cache()
    return out


if __name__ == "__main__":
    main()
