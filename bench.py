#!/usr/bin/env python
"""Benchmark of the libstrix_b200 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (config 3 of the baseline): paged decode attention over an
int8 KV cache - a batch of 64 sequences, one query token each, 32 query heads /
4 KV heads, head_dim 128, block_size 16, context lengths ~ U[1024, 65536], block
tables a random permutation of the physical blocks. One step = one pass of the
kernel over the batch. Metric: algorithmic KV bytes read per second (every live
key's K and V rows and their two fp32 scales). With N > 1 (torchrun) the 64
sequences are sharded over the ranks, balanced by their context lengths (no
data-path collective; "strong" scaling: the batch is fixed); the same line
carries the weak-scaling figure (64 sequences per GPU) as `decode_weak`.

`value` is timed with the inputs resident in HBM; `e2e` is the same metric
through the public call (libstrix_b200.attn_decode) with the step's inputs
(queries, sequence lengths, block table) in pinned host memory, copied in inside
the timed region, and the output copied back; the KV cache is resident state,
like model weights.

The other half of the baseline's compound metric and the remaining configs ride
in the same JSON line: `moe_fp8` (config 1: FP8 W8A8 MoE layer at 256 and 4096
tokens), `gemm_w8a8_int8` (config 2), `attn_prefill` (config 4), `ep_moe`
(config 5: MXFP4 MoE layer, expert-parallel over the ranks, plus the FP8 layer
through the same exchange), each with its roofline, parity against the CPU
oracle and, where it is cheap, the oracle's CPU time.

`--impl reference` times the CPU oracle (the reference's torch implementation
restated, oracle/attention.py) on the host cores over a bounded sample of the
same batch; it loads none of this library's native code.
"""

from __future__ import annotations

import argparse
import importlib.util
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
WORKLOAD = ("decode_attn_int8kv B=64 Hq=32 Hkv=4 D=128 block=16 ctx~U[1024,65536] "
            "shuffled block table")


def load_workloads():
    """libstrix_b200/workloads.py by file path: it has no native dependency, and the
    reference arm must not load the library."""
    spec = importlib.util.spec_from_file_location("strix_workloads", ROOT / "libstrix_b200" / "workloads.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["strix_workloads"] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks() -> dict:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm": float(d["hbm_gbs"]), "bf16": float(d["bf16_tflops"]), "kind": "measured"}
    return {"hbm": 6650.0, "bf16": 1590.0, "kind": "fallback"}


_DENSE_PEAKS: dict = {}


def dense_8bit_peaks(dev) -> dict:
    """fp8 and int8 dense matmul rates of this GPU, measured the way the bf16 peak
    was (library GEMM, 8192^3, best of 10, CUDA events): the denominators of the
    8-bit tensor rooflines. Falls back to 2 x the measured bf16 peak, labelled."""
    if _DENSE_PEAKS:
        return _DENSE_PEAKS
    n = 8192
    bf16 = measured_peaks()["bf16"]

    def best_of(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12

    try:
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        _DENSE_PEAKS["fp8"] = best_of(lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one,
                                                               out_dtype=torch.bfloat16))
        _DENSE_PEAKS["fp8_kind"] = "measured (torch._scaled_mm 8192^3, best of 10)"
        del a, b
    except Exception as e:  # noqa: BLE001
        _DENSE_PEAKS["fp8"], _DENSE_PEAKS["fp8_kind"] = 2 * bf16, f"2 x measured bf16 (derived: {type(e).__name__})"
    try:
        a = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
        b = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8).t()
        _DENSE_PEAKS["int8"] = best_of(lambda: torch._int_mm(a, b))
        _DENSE_PEAKS["int8_kind"] = "measured (torch._int_mm 8192^3, best of 10)"
        del a, b
    except Exception as e:  # noqa: BLE001
        _DENSE_PEAKS["int8"], _DENSE_PEAKS["int8_kind"] = 2 * bf16, f"2 x measured bf16 (derived: {type(e).__name__})"
    torch.cuda.empty_cache()
    return _DENSE_PEAKS


def parity_stats(out: torch.Tensor, ref: torch.Tensor) -> dict:
    """Error of `out` against the oracle `ref` (fp32, CPU): the bound the tests use
    (2e-2 x RMS plus the bf16 output quantum, half an ulp <= 2^-8 |ref|) and the
    strict figures beside it - the share of elements inside 2e-2 x RMS alone, and
    the largest error against the oracle rounded to the output's bf16."""
    out, ref = out.float().cpu(), ref.float().cpu()
    err = (out - ref).abs()
    rms = ref.pow(2).mean().sqrt().item()
    err_b = (out - ref.bfloat16().float()).abs()
    return {"ok": bool((err <= 2e-2 * rms + ref.abs() * 2.0 ** -8).all()),
            "max_abs_err": err.max().item(), "ref_rms": rms,
            "max_err_over_rms": err.max().item() / max(rms, 1e-30),
            "frac_within_2e-2_rms": (err <= 2e-2 * rms).float().mean().item(),
            "max_err_over_rms_vs_bf16_rounded_oracle": err_b.max().item() / max(rms, 1e-30),
            "frac_within_2e-2_rms_vs_bf16_rounded_oracle": (err_b <= 2e-2 * rms).float().mean().item()}


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


def batch_context_lengths() -> list[int]:
    """The 64 context lengths of the seed-0 batch (U[1024, 65536])."""
    gen = torch.Generator().manual_seed(0)
    return torch.randint(1024, 65536 + 1, (64,), generator=gen, dtype=torch.int64).tolist()


def shard_sequences(lens: list[int], world: int) -> list[list[int]]:
    """Sequence indices per rank, balanced by the sum of context lengths (longest
    first onto the lightest rank)."""
    shards: list[list[int]] = [[] for _ in range(world)]
    load = [0] * world
    for i in sorted(range(len(lens)), key=lambda i: -lens[i]):
        r = min(range(world), key=lambda r: load[r])
        shards[r].append(i)
        load[r] += lens[i]
    return [sorted(s) for s in shards]


def cpu_oracle_sample(batch, nseq_sample: int, repeats: int = 1):
    """Times the CPU oracle on the first `nseq_sample` sequences of the batch.
    Returns (GB/s, seconds, threads, description, output)."""
    from oracle import attention as A

    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    lens = batch.seq_lens[:nseq_sample].cpu()
    parts, ofs = [], 0
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
    desc = (f"first {nseq_sample} sequences of the batch ({int(lens.sum())} keys, {nbytes / 1e6:.0f} MB "
            f"of KV), torch fp32 on {threads} threads, dequantise + dense softmax")
    return nbytes / best / 1e9, best, threads, desc, out


def run_reference(args, rank: int) -> None:
    """--impl reference: the CPU oracle on the host cores, rank 0 only."""
    if rank != 0:
        return
    wl = load_workloads()

    # A bounded sample of the seed-0 batch: its first sequences, cut so that the
    # whole run (warm-up + steps) stays near two minutes of CPU time. The cut is
    # calibrated on one 8,192-key sequence.
    all_lens = batch_context_lengths()
    cal = wl.decode_batch(ctx_lens=[8192], seed=0)
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
    batch = wl.decode_batch(ctx_lens=lens, seed=0)
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
        "ms_per_step": 1e3 * statistics.mean(times), "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": desc},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_decode(strix, batch, args, world, dist, local_rank, sample_clocks: bool):
    """(total ms over K steps, per-step ms list, e2e total ms, clocks, out, launches per
    step, h2d bytes, d2h bytes) for one rank's batch."""
    out = torch.empty_like(batch.q)
    nseg = strix._lib.load().strix_attn_decode_segments_n(batch.q.size(0), args.num_splits,
                                                          batch.block_table.size(1), 16)
    launches = 2 if nseg > 1 else 1

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
    # The timed step is a replay of the captured call (the op neither synchronises nor
    # allocates outside torch's pool, so it records as it is): a shard of 8 sequences
    # runs for 0.1 ms, which the Python call path alone does not sustain.
    graphed = False
    if not args.no_graph:
        eager_step = step
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                eager_step()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                eager_step()
            graphed = True
        except Exception as exc:                      # a capture that fails falls back to eager calls
            print(f"bench: decode graph capture failed ({exc}); timing eager calls", file=sys.stderr)
            torch.cuda.synchronize()
        if graphed:
            def step():
                graph.replay()

            for _ in range(3):
                step()
        barrier()
    time_decode.graphed = graphed
    sampler = ClockSampler(local_rank) if sample_clocks else None
    if sampler:
        sampler.start()
        t_end = time.perf_counter() + 0.6      # long enough for nvidia-smi to see clocks under load
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
    clocks = sampler.stop() if sampler else None

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
    return (total_ms, per_step, e0.elapsed_time(e1), clocks, out, launches, int(nseg),
            int(q_h.nbytes + sl_h.nbytes + bt_h.nbytes), int(out_h.nbytes))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--num-splits", type=int, default=0, help="0 = fixed 1024-key segments")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="time eager calls of the decode op instead of replays of its CUDA graph")
    ap.add_argument("--no-moe", action="store_true", help="skip the MoE / GEMM / prefill / EP sections")
    ap.add_argument("--only", choices=["moe", "gemm", "prefill", "ep", "decode_bf16"], default=None,
                    help="run one secondary section alone (for profiling) and print its JSON")
    ap.add_argument("--moe-tokens", type=int, nargs="*", default=[256, 4096])
    ap.add_argument("--gemm-m", type=int, nargs="*", default=[1, 16, 4096])
    ap.add_argument("--prefill-tokens", type=int, nargs="*", default=[2048, 65536])
    ap.add_argument("--ep-exchange", default="auto", choices=["auto", "peer", "nccl"])
    ap.add_argument("--ep-placement", default="balanced", choices=["balanced", "round_robin", "contiguous"],
                    help="which rank owns which expert in the expert-parallel sections")
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
    with_cpu = not args.no_cpu_baseline
    if args.only == "ep":
        res = bench_ep_moe(args, dev, rank, world, with_cpu)
        if rank == 0:
            print(json.dumps({"ep": res}), flush=True)
        if dist.is_initialized():
            dist.destroy_process_group()
        return
    if args.only is not None:
        if rank == 0:
            section = {"moe": bench_moe_fp8, "gemm": bench_gemm_w8a8,
                       "prefill": bench_attn_prefill, "decode_bf16": bench_decode_bf16kv}[args.only]
            print(json.dumps({args.only: section(args, dev, with_cpu)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- headline: the 64-sequence batch, sharded over the ranks by context length
    lens = batch_context_lengths()[:args.batch]
    mine = shard_sequences(lens, world)[rank]
    batch = decode_batch(ctx_lens=[lens[i] for i in mine], seed=rank, device=dev)
    kv_bytes = batch.kv_bytes
    total_ms, per_step, e2e_ms, clocks, out, launches, nseg, h2d, d2h = time_decode(
        strix, batch, args, world, dist, local_rank, sample_clocks=True)

    stats = torch.tensor([total_ms, e2e_ms, float(kv_bytes), float(h2d), float(d2h)],
                         dtype=torch.float64, device=dev)
    if world > 1:
        tmax, tsum = stats.clone(), stats.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms = tmax[0].item(), tmax[1].item()
        all_bytes, h2d_all, d2h_all = tsum[2].item(), int(tsum[3].item()), int(tsum[4].item())
        max_bytes = tmax[2].item()
    else:
        all_bytes, h2d_all, d2h_all, max_bytes = float(kv_bytes), h2d, d2h, float(kv_bytes)

    line = None
    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = all_bytes / (ms_per_step * 1e-3) / 1e9
        e2e_value = all_bytes / (e2e_ms / args.steps * 1e-3) / 1e9
        peaks = measured_peaks()
        # the dominant kernel's own duration: this rank's step (the reduce kernel is
        # included; it is a few percent of the step)
        achieved = kv_bytes / (statistics.mean(per_step) * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "f16 mma / f32 softmax over int8 KV", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sequences_per_rank": len(mine),
                       "kv_bytes_rank0": kv_bytes, "kv_bytes_total": all_bytes,
                       "shard_balance_max_over_mean": max_bytes / (all_bytes / world),
                       "segments": nseg,
                       "l2": f"each rank's KV ({kv_bytes / 1e6:.0f} MB on rank 0) exceeds the 126 MB L2",
                       "timing": "cuda events, max over ranks",
                       "launch": "replays of the op's CUDA graph (value); eager calls with host copies (e2e)"
                                 if getattr(time_decode, "graphed", False) else "eager op calls"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm"],
                         # DRAM read + write bytes per launch: measured with ncu on the 32-sequence
                         # case (1,183.6 + 16.1 MB for 1,182.4 MB algorithmic) and scaled by the keys
                         "traffic": kv_bytes * DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE,
                         "traffic_note": "ncu capture at batch 32 scaled to this launch by its keys",
                         "peak_kind": peaks["kind"], "frac_of_8TBps": achieved / 8000.0},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_all,
                    "d2h_bytes_per_step": d2h_all},
            "gpu_launches": launches * args.steps,
            "clocks": clocks,
        }
        if with_cpu:
            n_s = min(4, len(mine)) if world == 1 else 1
            v, sec, threads, desc, ref = cpu_oracle_sample(batch, n_s)
            line["parity"] = parity_stats(out[:n_s], ref)
            if world == 1:
                line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                                        "sample": desc, "seconds": sec}
    del batch, out
    torch.cuda.empty_cache()

    # ---- weak scaling beside it: 64 sequences on every GPU
    if world > 1 and not args.no_moe:
        wb = decode_batch(ctx_lens=lens, seed=100 + rank, device=dev)
        w_ms, _, _, _, _, _, _, _, _ = time_decode(strix, wb, args, world, dist, local_rank, False)
        wstats = torch.tensor([w_ms, float(wb.kv_bytes)], dtype=torch.float64, device=dev)
        wmax, wsum = wstats.clone(), wstats.clone()
        dist.all_reduce(wmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(wsum, op=dist.ReduceOp.SUM)
        if rank == 0:
            line["decode_weak"] = {"sequences_per_gpu": len(lens), "ms_per_step": wmax[0].item() / args.steps,
                                   "value": wsum[1].item() / (wmax[0].item() / args.steps * 1e-3) / 1e9,
                                   "unit": UNIT, "scaling": "weak"}
        del wb
        torch.cuda.empty_cache()

    if rank == 0 and world == 1 and not args.no_moe:
        moe = bench_moe_fp8(args, dev, with_cpu)
        gemm = bench_gemm_w8a8(args, dev, with_cpu)
        pre = bench_attn_prefill(args, dev, with_cpu)
        # the MoE half of the compound metric sits right behind the headline keys
        head = {k: line[k] for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step")}
        dbf = bench_decode_bf16kv(args, dev, with_cpu)
        line = {**head, "moe_fp8": moe, **{k: v for k, v in line.items() if k not in head},
                "gemm_w8a8_int8": gemm, "attn_prefill": pre, "attn_decode_bf16kv": dbf}
        line["gpu_launches"] += (moe["gpu_launches"] + gemm["gpu_launches"] + pre["gpu_launches"]
                                 + dbf["gpu_launches"])
    # the expert-parallel layers run on every rank (they exchange tokens)
    ep_res = None if args.no_moe else bench_ep_moe(args, dev, rank, world, with_cpu)
    if rank == 0:
        if ep_res is not None:
            line["ep_moe"] = ep_res
            line["gpu_launches"] += ep_res["gpu_launches"]
        print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


def bench_decode_bf16kv(args, dev, with_cpu: bool) -> dict:
    """Decode attention over bf16 caches (no scales): the first 32 sequences of the
    headline batch, their int8 caches dequantised once outside the timed region. The
    bytes are the K and V rows of every key (2 x 2 bytes x head x KV heads)."""
    import libstrix_b200 as strix
    from libstrix_b200.workloads import decode_batch

    lens = batch_context_lengths()[:min(args.batch, 32)]
    b = decode_batch(ctx_lens=lens, seed=7, device=dev)
    kc = torch.empty(b.key_cache.shape, dtype=torch.bfloat16, device=dev)
    vc = torch.empty_like(kc)
    chunk = 4096                                   # blocks per pass: bounds the fp32 temporaries
    for lo in range(0, kc.size(0), chunk):
        sl = slice(lo, lo + chunk)
        kc[sl] = (b.key_cache[sl].float() * b.k_scale[sl][..., None]).bfloat16()
        vc[sl] = (b.value_cache[sl].float() * b.v_scale[sl][..., None]).bfloat16()
    out = torch.empty_like(b.q)
    out8 = torch.empty_like(b.q)
    strix.attn_decode(out8, b.q, b.key_cache, b.value_cache, b.seq_lens, b.block_table, b.scale,
                      0, -1, b.k_scale, b.v_scale)
    nseg = strix._lib.load().strix_attn_decode_segments_n(b.q.size(0), 0, b.block_table.size(1), 16)
    kv_heads, head = kc.size(-2), kc.size(-1)
    nbytes = int(b.seq_lens.sum()) * kv_heads * head * 2 * 2

    def step():
        strix.attn_decode(out, b.q, kc, vc, b.seq_lens, b.block_table, b.scale, 0, -1)

    ms = _timed(step, args.steps, max(args.warmup, 3))
    peaks = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    diff = (out.float() - out8.float()).abs().max().item()
    return {"workload": f"{len(lens)} sequences of the headline batch, bf16 K/V rows, block 16",
            "ms_per_step": ms, "value": gbs, "unit": UNIT, "kv_bytes": nbytes, "segments": int(nseg),
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm"], "peak_kind": peaks["kind"]},
            "max_abs_diff_vs_int8_kv_path": diff,
            "l2": f"{nbytes / 1e6:.0f} MB of rows per step exceed the 126 MB L2",
            "gpu_launches": (2 if nseg > 1 else 1) * args.steps}


def bench_moe_fp8(args, dev, with_cpu: bool) -> dict:
    """The MoE half of the compound metric: one FP8 W8A8 block-scaled layer at
    256 tokens (config 1: hidden 2048, 128 experts, top-8, intermediate 768) and,
    for the tensor-bound regime, at 4096 tokens. At 256 tokens every expert is
    hit with ~16 rows, so the layer is bound by streaming the 604 MB of expert
    weights once: GB/s of weight bytes against the HBM roofline. At 4096 tokens
    TFLOP/s against the measured fp8 matmul rate. Weights (604 MB) exceed the L2.
    `e2e`: the same layer through fused_moe_fp8_w8a8 with x and the router logits
    in pinned host memory, copied in, and the output copied back, every step."""
    import libstrix_b200 as strix
    from libstrix_b200.moe import pick_block_m, workspace_for
    from libstrix_b200.workloads import moe_fp8_layer
    from oracle import moe as M

    peaks = measured_peaks()
    fp8 = dense_8bit_peaks(dev)
    out = {"config": "MoE FP8 W8A8 block-scaled, H=2048 E=128 top-8 I=768", "gpu_launches": 0, "runs": []}
    for tokens in args.moe_tokens:
        layer = moe_fp8_layer(tokens=tokens, seed=0, device=dev)
        ws = workspace_for(tokens, layer.top_k, 2048, 768, 128, pick_block_m(tokens, layer.top_k, 128), dev)

        def step(x=layer.x, logits=layer.logits):
            return strix.moe.fused_moe_fp8_w8a8(x, logits, layer.w13, layer.w13_scale,
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
        # the same launches replayed from a CUDA graph (how a serving loop runs decode steps)
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
        # end to end: inputs from pinned host memory, output back
        x_h, lg_h = layer.x.cpu().pin_memory(), layer.logits.cpu().pin_memory()
        o_h = torch.empty(res.shape, dtype=res.dtype).pin_memory()
        x_d, lg_d = torch.empty_like(layer.x), torch.empty_like(layer.logits)

        def e2e_step():
            x_d.copy_(x_h, non_blocking=True)
            lg_d.copy_(lg_h, non_blocking=True)
            o_h.copy_(step(x_d, lg_d), non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for _ in range(3):
            e2e_step()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        ms_e2e = e0.elapsed_time(e1) / args.steps
        gbs = layer.weight_bytes / (ms * 1e-3) / 1e9
        tf = layer.flops / (ms * 1e-3) / 1e12
        roof = ({"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                 "frac": gbs / peaks["hbm"], "peak_kind": peaks["kind"]} if tokens < 2048 else
                {"bound": "tensor", "achieved": tf, "peak": fp8["fp8"], "unit": "TFLOP/s",
                 "frac": tf / fp8["fp8"], "peak_kind": fp8["fp8_kind"]})
        run = {"tokens": tokens, "ms": ms, "tflops": tf, "weight_gbs": gbs, "ms_cuda_graph": ms_graph,
               "block_m": pick_block_m(tokens, layer.top_k, 128), "roofline": roof,
               "e2e": {"value": layer.flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": ms_e2e,
                       "h2d_bytes_per_step": int(x_h.nbytes + lg_h.nbytes),
                       "d2h_bytes_per_step": int(o_h.nbytes)}}
        out["gpu_launches"] += 7 * 2 * args.steps
        if with_cpu:
            threads = len(os.sched_getaffinity(0))
            torch.set_num_threads(threads)
            cpu = layer.to("cpu")
            sample = torch.arange(tokens) if tokens <= 256 else torch.arange(0, tokens, tokens // 32)
            t0 = time.perf_counter()
            ref, _, _ = M.moe_fp8_layer(cpu.x[sample], cpu.logits[sample], cpu.w13, cpu.w13_scale,
                                        cpu.w2, cpu.w2_scale, cpu.top_k)
            sec = time.perf_counter() - t0
            run["parity"] = parity_stats(res[sample.to(dev)], ref)
            run["parity"]["sample"] = f"{sample.numel()} of {tokens} tokens"
            if tokens <= 256:
                run["cpu_baseline"] = {"value": layer.flops / sec / 1e12, "unit": "TFLOP/s",
                                       "cores": threads, "kind": "port", "seconds": sec,
                                       "sample": "the whole 256-token layer, torch fp32 incl. dequantisation"}
            del cpu
        out["runs"].append(run)
        del layer, ws
        torch.cuda.empty_cache()
    return out


def bench_gemm_w8a8(args, dev, with_cpu: bool) -> dict:
    """Dense W8A8 INT8 GEMM of config 2: K=5120, N=34816 (a 27B-like MLP gate-up),
    M in {1, 16, 4096}. The decode rows (M <= 16) stream the 178 MB of weights
    once per launch - HBM roofline; every launch reads another of six weight
    copies (1.07 GB in rotation, far beyond the 126 MB L2). M = 4096 is tensor
    bound: TOPS against the int8 matmul rate measured on this GPU."""
    from oracle import gemm as G

    peaks = measured_peaks()
    i8 = dense_8bit_peaks(dev)
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
        roof = ({"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                 "frac": gbs / peaks["hbm"], "peak_kind": peaks["kind"]} if m <= 64 else
                {"bound": "tensor", "achieved": tops, "peak": i8["int8"], "unit": "TOP/s",
                 "frac": tops / i8["int8"], "peak_kind": i8["int8_kind"]})
        run = {"m": m, "ms": ms, "tops": tops, "gbs": gbs, "bytes": byts, "roofline": roof}
        out["gpu_launches"] += args.steps
        if with_cpu:
            last = ws[(args.steps - 1) % copies]
            rows = torch.arange(0, n, 17 if m <= 64 else 257, device=dev)
            mrows = torch.arange(0, m, max(1, m // 16), device=dev)
            t0 = time.perf_counter()
            ref, _ = G.w8a8_int8_gemm(a[mrows].cpu(), sa[mrows].cpu(), last[rows].cpu(), sw[rows].cpu())
            sec = time.perf_counter() - t0
            got = res[mrows][:, rows].cpu()
            run["parity"] = {"bit_exact_bf16": bool(torch.equal(got.view(torch.int16), ref.view(torch.int16))),
                             "sample": f"{mrows.numel()} rows x {rows.numel()} output channels"}
            if m == 16:
                run["cpu_baseline"] = {"value": 2.0 * mrows.numel() * rows.numel() * k / sec / 1e12,
                                       "unit": "TOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                       "seconds": sec, "sample": f"M=16, every 17th output channel ({rows.numel()})"}
        out["runs"].append(run)
    return out


def _timed(fn, steps: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _phase_times(layer_fn, reps: int = 5) -> dict:
    """Mean CUDA-event time between the marks a layer sets (layer_fn(mark) runs one
    layer and calls mark(name) after each phase is enqueued)."""
    acc: dict[str, float] = {}
    for it in range(reps + 1):
        marks = []
        start = torch.cuda.Event(enable_timing=True)
        start.record()

        def mark(name):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((name, ev))

        layer_fn(mark)
        torch.cuda.synchronize()
        if it:
            prev = start
            for name, ev in marks:
                acc[name] = acc.get(name, 0.0) + prev.elapsed_time(ev) / reps
                prev = ev
    return {k: round(v, 4) for k, v in acc.items()}


def bench_ep_moe(args, dev, rank: int, world: int, with_cpu: bool) -> dict:
    """Config 5: MXFP4 MoE layer, gpt-oss-120B-like (hidden 2880, 128 experts, top-4,
    intermediate 2880), 8192 tokens in total, expert-parallel over the ranks: each
    rank holds 8192 / N tokens and 128 / N experts. Weights N(0, 0.02) quantised to
    e2m1 with e8m0 scales per 32; router logits N(0,1) plus a Zipf(1.1) per-expert
    bias. Tokens move through this library's peer-memory exchange (or NCCL
    all-to-all with --ep-exchange nccl). Expert placement (--ep-placement): the Zipf
    bias makes one expert draw 22 % of all slots, more than a rank's share from 8
    ranks on, so the default is `balanced`: a placement table computed from the
    router's load on a seeded calibration batch (not the timed tokens), one spare
    expert slot per rank, the spare slots holding copies of the hottest experts whose
    tokens are spread over the copies. `contiguous` (blocks) and `round_robin` have
    no copies; the load ratios of all three are reported. Strong scaling: the total
    work is fixed.
    Time = max over ranks of the CUDA-event time; TFLOP/s counts 2 x slots x
    (2I x H + H x I). Rank 0 checks a sample of its tokens against the CPU oracle
    (the experts they need are regenerated from their seeds). A second entry runs
    the FP8 W8A8 layer of config 1 at 4096 tokens through the same exchange."""
    import torch.distributed as dist

    from libstrix_b200 import ep
    from libstrix_b200.workloads import moe_mxfp4_layer
    from oracle import moe as M

    tokens_total, hid, inter, experts, top_k = 8192, 2880, 2880, 128, 4
    t_local, e_local = tokens_total // world, experts // world
    exchange = args.ep_exchange
    placement = "contiguous" if world == 1 or exchange == "nccl" else args.ep_placement
    place = placement
    if placement == "balanced":
        # expected load per expert: the router over a calibration batch of the same distribution
        from libstrix_b200.workloads import zipf_bias
        g = torch.Generator().manual_seed(4242)
        cal = (torch.randn(8192, experts, generator=g) + zipf_bias(experts, 1.1)).to(dev)
        from libstrix_b200 import moe as smoe_cal
        loads = torch.bincount(smoe_cal.route(cal, top_k)[1].flatten().long(), minlength=experts).tolist()
        place = ep.Placement.balanced(loads, world, slots_per_rank=e_local + 1)
        mine = place.ranks[rank]
    else:
        mine = list(range(rank, experts, world)) if placement == "round_robin" else \
            list(range(rank * e_local, (rank + 1) * e_local))
    layer = moe_mxfp4_layer(tokens=tokens_total, hidden=hid, experts=experts, top_k=top_k, inter=inter,
                            seed=0, device=dev, expert_list=mine,
                            token_lo=rank * t_local, token_hi=(rank + 1) * t_local)

    def step():
        return ep.ep_moe_mxfp4(layer.x, layer.logits, layer.w13, layer.w13_scale, layer.w2,
                               layer.w2_scale, top_k, exchange=exchange, placement=place)

    steps = max(2, min(args.steps, 10))
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step()
    e1.record()
    torch.cuda.synchronize()
    ms_t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms = ms_t.item()
    flops = 2.0 * tokens_total * top_k * (2 * inter * hid + hid * inter)

    # load: routed slots per expert rank (Zipf skew), max over mean
    from libstrix_b200 import moe as smoe

    _, ids = smoe.route(layer.logits, top_k)
    flat = ids.reshape(-1).long()
    per_rank_blocks = torch.bincount(flat // e_local, minlength=world).to(torch.float64)
    per_rank_rr = torch.bincount(flat % world, minlength=world).to(torch.float64)
    if world > 1:
        dist.all_reduce(per_rank_blocks, op=dist.ReduceOp.SUM)
        dist.all_reduce(per_rank_rr, op=dist.ReduceOp.SUM)
    per_rank = per_rank_rr if placement == "round_robin" else per_rank_blocks
    if placement == "balanced":
        per_rank = torch.bincount(place.rank_of(ids).reshape(-1).long(), minlength=world).to(torch.float64)
        if world > 1:
            dist.all_reduce(per_rank, op=dist.ReduceOp.SUM)
    res = {"config": "MXFP4 MoE, H=2880 E=128 top-4 I=2880, 8192 tokens, EP over ranks, Zipf(1.1) bias, "
                     "weights N(0,0.02) -> e2m1 / e8m0 per 32",
           "n_gpus": world, "scaling": "strong", "ms_per_layer": ms,
           "tflops": flops / (ms * 1e-3) / 1e12, "tokens_per_s": tokens_total / (ms * 1e-3),
           "roofline": {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12 / world,
                        "peak": measured_peaks()["bf16"], "unit": "TFLOP/s per GPU",
                        "frac": flops / (ms * 1e-3) / 1e12 / world / measured_peaks()["bf16"],
                        "peak_kind": "measured bf16 (the kernel runs kind::f16 on decoded weights)"},
           "slots_per_rank_max_over_mean": (per_rank.max() / per_rank.mean()).item(),
           "expert_placement": placement,
           "slots_per_rank_max_over_mean_if_contiguous": (per_rank_blocks.max() / per_rank_blocks.mean()).item(),
           "slots_per_rank_max_over_mean_if_round_robin": (per_rank_rr.max() / per_rank_rr.mean()).item(),
           "experts_held_per_rank": len(mine),
           "exchange": ("none (one rank: the fused single-GPU layer)" if world == 1 and exchange == "auto"
                        else "NCCL all_to_all_single" if exchange == "nccl"
                        else "peer-memory kernels over NVLink (CUDA IPC), no host synchronisation"),
           "gpu_launches": (6 if world == 1 else 11) * steps}
    if world > 1 and exchange != "nccl":
        dist.barrier()
        res["phases_ms_rank0"] = _phase_times(lambda mark: ep.ep_moe_mxfp4(
            layer.x, layer.logits, layer.w13, layer.w13_scale, layer.w2, layer.w2_scale, top_k,
            exchange=exchange, mark=mark, placement=place))
        res["ep_status"] = next(iter(ep._CONTEXTS.values())).status()
    # parity on rank 0: a sample of its tokens against the oracle over regenerated experts
    if with_cpu and rank == 0:
        sample = torch.arange(0, t_local, max(1, t_local // 8))[:8]
        ids_s = ids[sample.to(dev)].cpu().long()
        need = sorted(set(ids_s.reshape(-1).tolist()))
        lo, hi = need[0], need[-1] + 1
        full = {k: None for k in ("w13", "w13_scale", "w2", "w2_scale")}
        shapes = {"w13": (2 * inter, hid // 2), "w13_scale": (2 * inter, hid // 32),
                  "w2": (hid, inter // 2), "w2_scale": (hid, inter // 32)}
        for k, shp in shapes.items():
            full[k] = torch.zeros(hi - lo, *shp, dtype=torch.uint8)
        for e in need:
            one = moe_mxfp4_layer(tokens=256, hidden=hid, experts=experts, top_k=top_k, inter=inter, seed=0,
                                  device=dev, expert_lo=e, expert_hi=e + 1, token_lo=0, token_hi=256)
            for k in shapes:
                full[k][e - lo] = getattr(one, k)[0].cpu()
        ref, _, _ = M.moe_mxfp4_layer(layer.x.cpu(), layer.logits.cpu(), full["w13"], full["w13_scale"],
                                      full["w2"], full["w2_scale"], top_k, token_ids=sample,
                                      expert_offset=lo)
        res["parity"] = parity_stats(out[sample.to(dev)], ref)
        res["parity"]["sample"] = f"{sample.numel()} tokens of rank 0, {len(need)} experts regenerated"
    del layer, out
    torch.cuda.empty_cache()
    res["fp8"] = _bench_ep_fp8(args, dev, rank, world, steps, with_cpu)
    return res


def _bench_ep_fp8(args, dev, rank: int, world: int, steps: int, with_cpu: bool) -> dict:
    """The FP8 W8A8 layer of config 1 (H=2048, E=128, top-8, I=768) expert-parallel:
    4096 tokens in total, 4096 / N per rank, 128 / N experts per rank; e4m3 rows and
    their scales travel (quantise before dispatch). Strong scaling."""
    import torch.distributed as dist

    from libstrix_b200 import ep
    from libstrix_b200.workloads import moe_fp8_layer
    from oracle import moe as M

    tokens_total, experts = 4096, 128
    layer = moe_fp8_layer(tokens=tokens_total, seed=10, device=dev)     # the same layer on every rank
    t_local, e_local = tokens_total // world, experts // world
    lo, t0 = rank * e_local, rank * t_local
    placement = "contiguous" if world == 1 or args.ep_exchange == "nccl" else args.ep_placement
    placement = "contiguous" if placement == "balanced" else placement   # this router has no bias
    own = slice(rank, None, world) if placement == "round_robin" else slice(lo, lo + e_local)
    w13, s13 = layer.w13[own].contiguous(), layer.w13_scale[own].contiguous()
    w2, s2 = layer.w2[own].contiguous(), layer.w2_scale[own].contiguous()
    x, logits, top_k = layer.x[t0:t0 + t_local].contiguous(), layer.logits[t0:t0 + t_local].contiguous(), layer.top_k
    flops_total = layer.flops

    def step():
        return ep.ep_moe_fp8(x, logits, w13, s13, w2, s2, top_k, exchange=args.ep_exchange,
                             placement=placement)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step()
    e1.record()
    torch.cuda.synchronize()
    ms_t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms = ms_t.item()
    res = {"config": "FP8 W8A8 MoE, H=2048 E=128 top-8 I=768, 4096 tokens, EP over ranks",
           "n_gpus": world, "scaling": "strong", "ms_per_layer": ms,
           "tflops": flops_total / (ms * 1e-3) / 1e12, "tokens_per_s": tokens_total / (ms * 1e-3),
           "expert_placement": placement}
    if world > 1 and args.ep_exchange != "nccl":
        dist.barrier()
        res["phases_ms_rank0"] = _phase_times(lambda mark: ep.ep_moe_fp8(
            x, logits, w13, s13, w2, s2, top_k, exchange=args.ep_exchange, mark=mark, placement=placement))
    if with_cpu and rank == 0:
        cpu = layer.to("cpu")
        sample = torch.arange(0, t_local, max(1, t_local // 16))[:16]
        ref, _, _ = M.moe_fp8_layer(cpu.x[t0 + sample], cpu.logits[t0 + sample], cpu.w13, cpu.w13_scale,
                                    cpu.w2, cpu.w2_scale, cpu.top_k)
        res["parity"] = parity_stats(out[sample.to(dev)], ref)
        res["parity"]["sample"] = f"{sample.numel()} tokens of rank 0"
    ep.close_contexts()
    return res


def bench_attn_prefill(args, dev, with_cpu: bool) -> dict:
    """Causal GQA prefill of config 4: one sequence of 2048 and of 65536 tokens, 40
    query / 8 KV heads, head 128, int8 paged cache (block 16, shuffled table)
    written by this library's KV writer from bf16 N(0,1) values with
    per-token-per-head scales. Tensor bound: FLOPs = 4 x Hq x D x T (T + 1) / 2
    (QK^T and PV over the causal half) against the measured bf16 peak. Q + out
    (1.3 GB at 65536 tokens) exceed the L2. Parity: at 2048 tokens the last 256
    queries, at 65536 tokens every 256th 64-query tile and the last one, against
    the CPU oracle (a tile = the last 64 queries of the context that ends with it)."""
    import libstrix_b200 as strix
    from oracle import attention as A

    peaks = measured_peaks()
    hq, hkv, hd, bs = 40, 8, 128, 16
    out = {"config": "causal GQA prefill, Hq=40 Hkv=8 D=128 block=16, int8 KV", "gpu_launches": 0,
           "runs": []}
    g = torch.Generator(device=dev).manual_seed(0)
    for t in args.prefill_tokens:
        nblk = (t + bs - 1) // bs
        table = torch.randperm(nblk, generator=g, device=dev).int().view(1, nblk)
        # the cache is written by the product kernel: token i -> slot table[i / 16] * 16 + i % 16
        kq = torch.zeros(nblk, bs, hkv, hd, dtype=torch.int8, device=dev)
        vq = torch.zeros_like(kq)
        ks = torch.zeros(nblk, bs, hkv, device=dev)
        vs = torch.zeros_like(ks)
        pos = torch.arange(t, device=dev)
        slots = table[0, pos // bs].long() * bs + pos % bs
        for a in range(0, t, 8192):
            kv = torch.randn(min(8192, t - a), hkv, 2 * hd, generator=g, device=dev, dtype=torch.bfloat16)
            strix.kv_write_int8(kv[..., :hd], kv[..., hd:], kq, vq, ks, vs, slots[a:a + 8192])
        q = torch.randn(t, hq, hd, generator=g, device=dev, dtype=torch.bfloat16)
        o = torch.empty_like(q)
        cu = torch.tensor([0, t], dtype=torch.int32, device=dev)
        sl = torch.tensor([t], dtype=torch.int32, device=dev)
        scale = hd ** -0.5

        def step():
            strix.attn_prefill(o, q, kq, vq, cu, sl, table, scale, 1, -1, ks, vs)

        steps = max(2, min(args.steps, 5 if t > 8192 else args.steps))
        ms = _timed(step, steps)
        flops = 4.0 * hq * hd * t * (t + 1) / 2
        tf = flops / (ms * 1e-3) / 1e12
        run = {"tokens": t, "ms": ms, "tflops": tf, "flops": flops,
               "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16"], "unit": "TFLOP/s",
                            "frac": tf / peaks["bf16"], "peak_kind": f"{peaks['kind']} bf16 (cuBLAS burst)"}}
        out["gpu_launches"] += 2 * steps
        if with_cpu:
            kx, vx = (kq.float() * ks[..., None]).cpu(), (vq.float() * vs[..., None]).cpu()
            tiles = [(t - 256, t)] if t <= 2048 else \
                [(i * 64, i * 64 + 64) for i in sorted(set(range(0, t // 64, 256)) | {t // 64 - 1})]
            t0 = time.perf_counter()
            stats, work = [], 0.0
            for a, b in tiles:
                ref = A.attention_reference(q[a:b].cpu(), kx, vx, torch.tensor([0, b - a], dtype=torch.int32),
                                            torch.tensor([b], dtype=torch.int32), table.cpu(), scale)
                stats.append(parity_stats(o[a:b], ref))
                work += 4.0 * hq * hd * (b - a) * (a + b) / 2
            sec = time.perf_counter() - t0
            par = {k: (all(s[k] for s in stats) if k == "ok" else
                       min(s[k] for s in stats) if k.startswith("frac") else max(s[k] for s in stats))
                   for k in stats[0]}
            par["sample"] = f"{len(tiles)} query tiles ({sum(b - a for a, b in tiles)} queries)"
            run["parity"] = par
            run["cpu_baseline"] = {"value": work / sec / 1e12, "unit": "TFLOP/s",
                                   "cores": torch.get_num_threads(), "kind": "port", "seconds": sec,
                                   "sample": par["sample"]}
        out["runs"].append(run)
        del q, o, kq, vq, ks, vs
        torch.cuda.empty_cache()
    return out


if __name__ == "__main__":
    main()
