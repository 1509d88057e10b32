#!/usr/bin/env python
"""Benchmark of the decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one decode step of one layer for one ragged batch (K/V projection of the new tokens on
tensor cores + RoPE + write-back, split-KV attention streamed from the KV pool, LSE merge).
Workload: the OPT-6.7B layer configuration (hidden 4096, 32 MHA heads, head_dim 128, no RoPE),
16 requests with context lengths uniform in [512, 8192], 16-token pages, randomly permuted page
table; seeded synthetic tensors (there are no model weights or traces on the machine).

Reported on one JSON line:
  value  - host-KV GB/s: KV bytes attended per second with the KV pool in page-locked HOST memory,
           streamed over the host link by the kernel inside the timed region (X, Q and the lengths
           already on the device)
  e2e    - the same through the public Python API, with every step also copying X, Q and the
           lengths host->device from pinned memory and the output back
  roofline     - the KV-streaming kernel of those steps: algorithmic KV bytes per launch / its mean
                 launch duration (CUDA events on the launching stream) against the pinned
                 host->device copy rate measured in the same run with all ranks copying at once
  hbm          - the same step with the pool resident in HBM, against the measured HBM copy peak
  cpu_baseline - the CPU restatement of the reference's torch path, timed on the host cores
  clocks, gpu_launches
With N > 1 (torchrun) the layer's 32 KV heads are partitioned over the ranks (32 / N each, every rank
its own host pool, no data-path collective: the same total work at every N), and two more objects
are added: multi_gpu_check (head shard and both forms of the sequence split against the oracle on a
small case) and seq_split (one 1M-token request split by sequence, merged with NCCL or by the
fused peer-memory exchange).

--impl reference times the reference's torch attention path, restated for the CPU in fp32
(oracle/), on the host cores for the same configuration.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from directkv_b200 import workloads  # noqa: E402

CFG_ID = 1
PAGE = 16
METRIC = "decode_attention_host_kv_gbps"
UNIT = "GB/s"


def c2_lengths():
    """Request lengths of the batch.  Every rank gets the same ones: under head sharding all ranks serve the same
    requests (each its own KV heads), so the per-GPU work is identical; contents and page placement differ."""
    # +1: the token decoded in this step (its K/V are projected, stored and attended too)
    return [n + 1 for n in workloads.ragged_lengths_uniform(16, 512, 8192, seed=4234 + CFG_ID)]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [x for x in sm if x > 0.5 * (max(mx) if mx else 1)] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def workload_config(world: int, lens):
    """The `config` object of the JSON line; both arms (this engine, --impl reference) print the same one."""
    shape = workloads.OPT_6_7B
    return {
        "workload": "opt-6.7b layer decode, 16 ragged requests ctx U[512,8192], 16-token permuted pages",
        "kv_pool": "page-locked host memory, read over the host link inside the timed region",
        "kv_bytes_per_step": workloads.kv_bytes(shape, lens), "tokens": int(sum(lens)), "page_size": PAGE,
        "parallelism": (f"kv-head partition x{world}: {shape.nh_kv // world} of the layer's {shape.nh_kv} KV heads and one "
                        f"host pool per rank, no data-path collective (total work fixed)"),
        "l2": "inputs larger than L2 (0.98 GB of KV per step vs 126 MB)",
    }


def cpu_reference_time(steps: int, warmup: int, lens, budget_s: float = 150.0):
    """Times the reference's torch attention path (fp32, CPU, all host threads) on the whole batch.  `steps` timed
    passes after `warmup` untimed ones; the loop stops early only when the time budget is spent, and returns how
    many passes it timed."""
    from oracle import directkv_oracle as orc

    torch.set_num_threads(os.cpu_count() or 1)
    shape = workloads.OPT_6_7B
    case = workloads.make_decode_case(shape, lens, PAGE, CFG_ID, "cpu", kv_on_host=True)
    args = (case["x"], case["wk"], case["wv"], case["q"], case["k_pool"], case["v_pool"], case["page_table"], lens,
            PAGE, None, shape.scale)
    t_start = time.perf_counter()
    for _ in range(warmup):
        orc.decode_layer(*args)
    done, t0 = 0, time.perf_counter()
    while done < steps:
        orc.decode_layer(*args)
        done += 1
        if time.perf_counter() - t_start > budget_s:
            break
    dt = (time.perf_counter() - t0) / done
    nbytes = workloads.kv_bytes(shape, lens)
    sample = f"all {len(lens)} requests ({sum(lens)} tokens) per step, {done} steps after {warmup} warm-ups"
    return nbytes / dt / 1e9, dt * 1e3, torch.get_num_threads(), sample, done


def run_reference(args, rank, world):
    """--impl reference: the reference's own implementation of the path that runs here - its torch attention path
    (gather by slot + scaled_dot_product_attention; the kernel is sm_90a-only), restated in fp32 for the CPU - on
    the whole batch, all host threads, with the --steps / --warmup given.  Under torchrun rank 0 alone runs."""
    if rank != 0:
        return
    lens = c2_lengths()
    gbs, ms, cores, sample, done = cpu_reference_time(args.steps, args.warmup, lens)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": done,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(world, lens),
        "note": "reference's torch attention path (gather by slot + scaled_dot_product_attention) restated in fp32 "
                "on the CPU; the reference's own kernel is sm_90a-only",
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)



# ---------------------------------------------------------------------------------------------------
# Configuration sweep (the five benchmark configurations): one JSON row per configuration and mode.
# ---------------------------------------------------------------------------------------------------
def _median_ms(fn, iters, warm, sync):
    """Median of per-call CUDA-event times (the reference times its kernels the same way:
    benchmarks/bench_smpv2_perf.py:59-71 - warm-ups, then events around the call)."""
    for _ in range(warm):
        fn()
    sync()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        sync()
        ts.append(a.elapsed_time(b))
    _median_ms.last = ts
    return statistics.median(ts), min(ts)


_median_ms.last = []

# Columns of the reference's long-context benchmark (benchmarks/bench_offload_longctx.py:65-71).  Its rows come from a
# served model; the rows written here time the 32 attention layers of one decoded token (synthetic weights, no MLP),
# which is the part of a token's latency that this engine owns, and say so in the `system` / `model` fields.
LONGCTX_CSV_HEADER = ["system", "model", "seq_length", "mean_latency_s", "p50_latency_s", "p90_latency_s", "p99_latency_s",
                      "mean_e2e_latency_s", "p50_e2e_latency_s", "p90_e2e_latency_s", "p99_e2e_latency_s",
                      "gpu_memory_peak_mb", "memory_saving_pct", "throughput_tps"]


def write_longctx_csv(path, rows):
    import csv

    exists = os.path.exists(path)
    with open(path, "a", newline="") as f:
        w = csv.DictWriter(f, fieldnames=LONGCTX_CSV_HEADER)
        if not exists:
            w.writeheader()
        for r in rows:
            w.writerow({k: r.get(k, "") for k in LONGCTX_CSV_HEADER})


def _pct(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(q * (len(xs) - 1))))]


def _graphed(fn, n=1):
    """Captures n calls of fn (the per-layer launch sequence) in one CUDA graph and returns the replay."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(n):
            fn()
    return g.replay


def _oracle_picks(lens, seed=0):
    """Requests a full-size run is checked on: the longest, the shortest and two seeded random ones."""
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    picks = [order[-1], order[0]]
    g = torch.Generator().manual_seed(977 + seed)
    for i in torch.randperm(len(lens), generator=g).tolist():
        if i not in picks and len(picks) < min(4, len(lens)):
            picks.append(i)
    return picks


def _oracle_error(case, shape, lens, page, out, picks):
    """max |err| and max relative err of the requests `picks` against the CPU oracle (checker only, outside every
    timed region)."""
    from oracle import directkv_oracle as orc

    k_cpu = case["k_pool"].cpu() if case["k_pool"].is_cuda else case["k_pool"]
    v_cpu = case["v_pool"].cpu() if case["v_pool"].is_cuda else case["v_pool"]
    worst_abs, worst_rel = 0.0, 0.0
    for pick in picks:
        sub = [pick]
        ref = orc.decode_layer(case["x"][sub].cpu(), case["wk"].cpu(), case["wv"].cpu(), case["q"][sub].cpu(), k_cpu, v_cpu,
                               case["page_table"][sub].cpu(), [lens[pick]], page,
                               None if case["cos_sin"] is None else case["cos_sin"].cpu(), shape.scale, save_kv_cache=False)
        got = out[pick].float().cpu().view_as(ref[0])
        err = (got - ref[0]).abs()
        worst_abs = max(worst_abs, float(err.max()))
        worst_rel = max(worst_rel, float((err / ref[0].abs().clamp_min(1e-2)).max()))
    return worst_abs, worst_rel


def measure_extend(dev, steps, warmup):
    """Chunked-prefill path (projection + RoPE + write-back + tensor-core attention) of one Llama-3-8B layer:
    4096 new tokens, no past, KV pool in HBM.  Returns the per-call time and attention TFLOP/s (causal flops only)."""
    from directkv_b200 import kernel
    from directkv_b200._lib import get_context

    shape, s_new = workloads.LLAMA3_8B, 4096
    g = torch.Generator(device=dev).manual_seed(1234)
    x = torch.randn(1, s_new, shape.hidden, generator=g, device=dev).to(torch.bfloat16)
    wk = (torch.randn(shape.nh_kv, 128, shape.hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    wv = (torch.randn(shape.nh_kv, 128, shape.hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    q = torch.randn(1, s_new, shape.nh_q, 128, generator=g, device=dev).to(torch.bfloat16)
    k = torch.zeros(1, s_new, shape.nh_kv, 128, dtype=torch.bfloat16, device=dev)
    v = torch.zeros_like(k)
    cs = workloads.build_cos_sin(s_new, shape.rope_theta, device=dev)

    def fn():
        kernel.smpv2_fwd(x, wk, wv, q, k, v, cs, shape.scale, True, 0, -1)

    med, best = _median_ms(fn, steps, warmup, torch.cuda.synchronize)
    get_context(dev.index).raise_on_status()
    attn_flops = 4 * 128 * shape.nh_q * s_new * (s_new + 1) / 2
    proj_flops = 2 * s_new * (2 * shape.nh_kv * 128) * shape.hidden
    return {"workload": "llama3-8b layer, 4096 new tokens, causal, KV in HBM", "ms_per_call": med,
            "attention_tflops": attn_flops / med / 1e9, "attention_plus_projection_tflops": (attn_flops + proj_flops) / med / 1e9}


def measure_request_pool(dev, lens, steps=5, warmup=2):
    """The same batch in the request pool's layout (one contiguous pinned row per request,
    directkv/directkv_request_pool.py:66-76): past rows streamed by the SMs against brought in by the copy
    engines (directkv_b200/staging.py).  GB/s of KV per step, host->device copies inside the timed region."""
    from directkv_b200 import kernel
    from directkv_b200._lib import get_context
    from directkv_b200.staging import DmaStagedDecode

    shape = workloads.OPT_6_7B
    B, s_pad = len(lens), (max(lens) + 63) // 64 * 64
    g = torch.Generator().manual_seed(4321)
    k = torch.empty(B, s_pad, shape.nh_kv, 128, dtype=torch.bfloat16).normal_(0, 0.5, generator=g).pin_memory()
    v = torch.empty_like(k).normal_(0, 0.5, generator=g).pin_memory()
    wk = (torch.randn(shape.nh_kv, 128, shape.hidden, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    wv = (torch.randn(shape.nh_kv, 128, shape.hidden, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    q = torch.randn(B, shape.nh_q * 128, generator=g).to(torch.bfloat16).to(dev)
    x = torch.randn(B, shape.hidden, generator=g).to(torch.bfloat16).to(dev)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    rm = torch.arange(B, dtype=torch.int32, device=dev)
    out = torch.empty_like(q)
    layer = 77
    kernel.register_layer(layer, k, v, wk, wv, None, row_stride=s_pad, device=dev.index)
    stager = DmaStagedDecode(dev, shape.nh_kv)
    kvb = workloads.kv_bytes(shape, lens)
    res = {"layout": "request pool: one contiguous pinned row per request", "kv_bytes_per_step": kvb}
    for name, fn in (("streamed_by_sms", lambda: kernel.decode(layer, q, sl, shape.scale, row_map=rm, x=x, out=out)),
                     ("staged_by_copy_engines", lambda: stager.decode(layer, k, v, list(range(B)), lens, q, sl, shape.scale, rm, x=x, out=out))):
        med, _ = _median_ms(fn, steps, warmup, torch.cuda.synchronize)
        res[name] = {"ms_per_step": med, "gbs": kvb / med / 1e6}
    get_context(dev.index).raise_on_status()
    kernel.unregister_layer(layer)
    return res


SHORT_CASES = {
    "llama1k": ("llama3-8b layer, one request of 1024 stored tokens", workloads.LLAMA3_8B, [1025]),
    "llama4k": ("llama3-8b layer, one request of 4096 stored tokens", workloads.LLAMA3_8B, [4097]),
    "opt4k": ("opt-6.7b layer, one request of 4096 stored tokens", workloads.OPT_6_7B, [4097]),
    "llama16k": ("llama3-8b layer, one request of 16384 stored tokens", workloads.LLAMA3_8B, [16385]),
    "llama128k": ("llama3-8b layer, one request of 131072 stored tokens", workloads.LLAMA3_8B, [131073]),
    "llama4x4k": ("llama3-8b layer, four requests of 4096 stored tokens", workloads.LLAMA3_8B, [4097] * 4),
}


def run_short_probe(args, dev):
    """--only short-<case>: a short decode step with the pool in HBM, where the step is launch structure and latency
    rather than bandwidth.  Twelve eager steps (what a profiler capture of this command sees), then the step time
    from a CUDA graph of 20 steps (median of 7 replays), with and without the projection of the new token."""
    from directkv_b200 import kernel
    from directkv_b200._lib import get_context

    label, shape, lens = SHORT_CASES[args.only[len("short-"):]]
    case = workloads.make_decode_case(shape, lens, PAGE, 0, dev, kv_on_host=False)
    kernel.register_layer(3, case["k_pool"], case["v_pool"], case["wk"], case["wv"], case["cos_sin"], page_size=PAGE,
                          device=dev.index)
    out = torch.empty_like(case["q"])

    def full():
        kernel.decode(3, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"], x=case["x"], out=out)

    def attention_only():
        kernel.decode(3, case["q"], case["seq_lens"], shape.scale, page_table=case["page_table"], out=out)

    for _ in range(12):
        full()
    torch.cuda.synchronize()
    get_context(dev.index).raise_on_status()
    res = {}
    for name, fn in (("step_us", full), ("attention_only_us", attention_only)):
        replay = _graphed(fn, 20)
        med, _ = _median_ms(replay, 7, 2, torch.cuda.synchronize)
        res[name] = med / 20 * 1e3
    get_context(dev.index).raise_on_status()
    kvb = workloads.kv_bytes(shape, lens)
    print(json.dumps({"metric": "short_decode_step_us", "unit": "us", "value": res["step_us"], "config": {"workload": label},
                      "attention_only_us": res["attention_only_us"], "kv_gbs": kvb / res["step_us"] / 1e3,
                      "frac_of_8TBs": kvb / res["step_us"] / 1e3 / 8000.0, "partial": "short decode step, pool in HBM"}))


def run_extend_probe(args, dev):
    r = measure_extend(dev, max(3, min(args.steps, 20)), args.warmup)
    print(json.dumps({"metric": "extend_attention_tflops", "value": r["attention_tflops"], "unit": "TFLOP/s",
                      "ms_per_step": r["ms_per_call"], "config": {"workload": r["workload"]},
                      "partial": "extend path only"}))


def run_sweep(args, rank, world, local_rank, dev, dist):
    from directkv_b200 import kernel, sharding
    from directkv_b200._lib import get_context

    ctx = get_context(local_rank)
    names = args.sweep.split(",")
    rows = []
    longctx_rows = []

    def sync():
        torch.cuda.synchronize()

    def allmax(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def link_gbs():
        nb = 1 << 30
        h = torch.empty(nb, dtype=torch.uint8, pin_memory=True)
        d = torch.empty(nb, dtype=torch.uint8, device=dev)
        best = 1e30
        for _ in range(4):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            d.copy_(h, non_blocking=True)
            b.record()
            sync()
            best = min(best, a.elapsed_time(b))
        return nb / best / 1e6

    link = link_gbs()
    link_all = None
    if world > 1:                     # all ranks copying at once: what the host can feed concurrently
        dist.barrier(device_ids=[local_rank])
        link_all = link_gbs()

    def one_layer(name, shape, lens, cfg, modes=("host", "hbm"), iters=50, layers=1, note="", shard=True):
        """Head-sharded over the ranks: every rank runs the same lengths on its own heads and pool."""
        sh = shape.shard(world) if (world > 1 and shard) else shape
        for mode in modes:
            case = workloads.make_decode_case(sh, lens, PAGE, cfg + 1000 * rank, dev, kv_on_host=(mode == "host"))
            kernel.register_layer(7, case["k_pool"], case["v_pool"], case["wk"], case["wv"], case["cos_sin"],
                                  page_size=PAGE, device=local_rank)
            out = torch.empty_like(case["q"])

            def fn():
                for _ in range(layers):
                    kernel.decode(7, case["q"], case["seq_lens"], sh.scale, page_table=case["page_table"], x=case["x"],
                                  out=out)

            fn()
            sync()
            ctx.raise_on_status()
            err = _oracle_error(case, sh, lens, PAGE, out, _oracle_picks(lens, cfg)) if rank == 0 else None
            replay = _graphed(fn) if layers == 1 else fn
            n_it = iters if mode == "hbm" else max(5, min(iters, int(2000 / max(1.0, workloads.kv_bytes(sh, lens) * layers / 50e6))))
            med, best = _median_ms(replay, n_it, 3 if mode == "host" else 20, sync)
            med = allmax(med)
            kvb = workloads.kv_bytes(sh, lens) * layers
            row = {"config": name, "mode": mode, "n_gpus": world, "layers": layers, "tokens": int(sum(lens)),
                   "kv_bytes_per_gpu": kvb, "latency_us": med * 1e3, "latency_us_per_layer": med * 1e3 / layers,
                   "kv_gbs_per_gpu": kvb / med / 1e6, "kv_gbs_aggregate": world * kvb / med / 1e6,
                   "host_link_gbs": link, "host_link_gbs_all_ranks_busy": link_all, "note": note}
            if mode == "host":
                row["frac_of_host_link"] = kvb / med / 1e6 / link
            else:
                row["frac_of_8TBs"] = kvb / med / 1e6 / 8000.0
                row["frac_of_measured_hbm"] = kvb / med / 1e6 / measured_peaks()[0]
            if err is not None:
                row["max_abs_err"], row["max_rel_err"] = err
            rows.append(row)
            kernel.unregister_layer(7)
            del case, out
            torch.cuda.empty_cache()

    def seq_split(name, ctx_len, cfg, layers=32):
        """One request split by sequence over the ranks; partial (O, m, l) all-gathered with NCCL and merged."""
        shape = workloads.LLAMA3_8B
        plan = sharding.plan_sequence_split(ctx_len + 1, world, PAGE)
        owner = sharding.owner_of_new_token(plan)
        s0, e0 = plan[rank]
        n_loc = e0 - s0
        case = workloads.make_decode_case(shape, [max(n_loc, 1)], PAGE, cfg + rank, dev, kv_on_host=True)
        cs = workloads.build_cos_sin(ctx_len + 2, shape.rope_theta, device=dev)
        kernel.register_layer(8, case["k_pool"], case["v_pool"], case["wk"], case["wv"], cs, page_size=PAGE, device=local_rank)
        lens_dev = torch.tensor([n_loc], dtype=torch.int32, device=dev)
        off = torch.tensor([s0], dtype=torch.int32, device=dev)
        is_owner = rank == owner

        out1 = torch.empty_like(case["q"])

        def fn():
            for _ in range(layers):
                if world == 1:
                    kernel.decode(8, case["q"], lens_dev, shape.scale, page_table=case["page_table"], x=case["x"], out=out1)
                else:
                    sharding.sequence_split_decode(8, case["q"], lens_dev, shape.scale, case["page_table"],
                                                   x=case["x"] if is_owner else None,
                                                   pos_offset=off if is_owner else None)

        fn()
        sync()
        ctx.raise_on_status()
        med, best = _median_ms(fn, 3 if not args.longctx_csv else 7, 1, sync)
        per_token_s = [t / 1e3 for t in _median_ms.last]
        med = allmax(med)
        if rank == 0 and args.longctx_csv:
            # Without offloading this layer stack would keep ctx_len x 32 layers x 4 KB of KV in HBM.
            kv_all_layers_mb = workloads.kv_bytes(shape, [ctx_len + 1]) * layers / 2**20
            peak_mb = torch.cuda.max_memory_allocated(dev) / 2**20
            longctx_rows.append({
                "system": f"directkv-b200 (attention layers only, {world} GPU)", "model": "llama3-8b, synthetic weights",
                "seq_length": ctx_len, "mean_latency_s": statistics.mean(per_token_s), "p50_latency_s": _pct(per_token_s, 0.5),
                "p90_latency_s": _pct(per_token_s, 0.9), "p99_latency_s": _pct(per_token_s, 0.99),
                "gpu_memory_peak_mb": peak_mb, "memory_saving_pct": 100.0 * (1.0 - peak_mb / (peak_mb + kv_all_layers_mb)),
                "throughput_tps": 1.0 / statistics.mean(per_token_s)})
        kvb_total = workloads.kv_bytes(shape, [ctx_len + 1]) * layers
        rows.append({"config": name, "mode": "host, sequence-split" if world > 1 else "host", "n_gpus": world, "layers": layers,
                     "tokens": ctx_len + 1, "kv_bytes_total": kvb_total, "latency_us": med * 1e3,
                     "latency_us_per_layer": med * 1e3 / layers, "kv_gbs_aggregate": kvb_total / med / 1e6,
                     "kv_gbs_per_gpu": kvb_total / med / 1e6 / world, "host_link_gbs": link,
                     "host_link_gbs_all_ranks_busy": link_all, "frac_of_host_link": kvb_total / med / 1e6 / world / link,
                     "note": "one layer's pool re-used for all 32 layers (32 x 4.3 GB of pinned memory per 1M tokens would not fit)"})
        kernel.unregister_layer(8)

    for name in names:
        if name == "C1":
            one_layer("C1 llama3-8b B=1 ctx 4096", workloads.LLAMA3_8B, [4097], 0, iters=100)
        elif name == "C2":
            one_layer("C2 opt-6.7b 16 ragged U[512,8192]", workloads.OPT_6_7B, c2_lengths(), CFG_ID, iters=100)
        elif name.startswith("C3"):
            for n in (32768, 131072, 524288, 1048576):
                if world > 1 and n < 1048576:
                    continue
                seq_split(f"C3 llama3-8b x32 layers ctx {n}", n, 2)
        elif name == "L128K":      # GQA streaming kernel at HBM speed: one Llama-3-8B request of 128K tokens
            one_layer("llama3-8b B=1 ctx 131072", workloads.LLAMA3_8B, [131073], 2, modes=("hbm",), iters=50)
        elif name == "C4":
            base = workloads.ragged_lengths_lognormal(64, 8192, 1.0, 256, 131072, seed=4234 + 3)
            g = torch.Generator().manual_seed(99)
            for step in range(3):                                  # 10 % of the requests replaced per step
                if step:
                    fresh = workloads.ragged_lengths_lognormal(6, 8192, 1.0, 256, 131072, seed=4234 + 3 + 17 * step)
                    for j, i in enumerate(torch.randperm(64, generator=g)[:6].tolist()):
                        base[i] = fresh[j]
                one_layer(f"C4 llama3-8b 64 ragged lognormal, step {step}", workloads.LLAMA3_8B, [n + 1 for n in base], 3 + step,
                          modes=("host",), iters=5, note="10% of requests replaced with fresh seeded lengths before this step")
        elif name == "C5":
            one_layer("C5 opt-30b B=32 ctx 16K (7 KV heads per GPU)", workloads.OPT_30B.shard(8), [16385] * 32, 5, iters=30,
                      note="one 7-head shard per GPU; with fewer than 8 GPUs each GPU still runs a 7-head shard",
                      shard=False)
    if rank == 0:
        with open(args.sweep_out, "a") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
                print(json.dumps(r), flush=True)
        if args.longctx_csv and longctx_rows:
            write_longctx_csv(args.longctx_csv, longctx_rows)


# ---------------------------------------------------------------------------------------------------
# Serving-level simulation (the reference's benchmarks/bench_offload_serving.py and bench_offload_longctx.py
# measure a served model over HTTP; here the attention backend is driven directly, see directkv_b200/serve_sim.py).
# ---------------------------------------------------------------------------------------------------
def serve_sim_configs():
    """(name, layer shape, prompt lengths, churn, lengths of the requests that join) per benchmark configuration,
    sized to what one request pool can hold: a pool row has the maximum context length, and the backend keeps at
    most 64 rows, like the reference."""
    c2 = workloads.ragged_lengths_uniform(16, 512, 8192, seed=4234 + CFG_ID)
    c4 = workloads.ragged_lengths_lognormal(58, 8192, 1.0, 256, 16384, seed=4234 + 3)
    c4_new = workloads.ragged_lengths_lognormal(48, 8192, 1.0, 256, 16384, seed=4234 + 20)
    return [
        ("C1 llama3-8b, 1 request, 4K prompt", workloads.LLAMA3_8B, [4096], 0.0, None),
        ("C2 opt-6.7b, 16 requests, prompts U[512,8192]", workloads.OPT_6_7B, c2, 0.0, None),
        ("C3 llama3-8b, 1 request, 32K prompt", workloads.LLAMA3_8B, [32768], 0.0, None),
        ("C3 llama3-8b, 1 request, 128K prompt", workloads.LLAMA3_8B, [131072], 0.0, None),
        ("C4 llama3-8b, 58 requests lognormal (median 8K, clipped to 16K), 10% replaced per step", workloads.LLAMA3_8B,
         c4, 0.1, c4_new),
        ("C5 opt-30b shard (7 of 56 heads), 32 requests, 16K prompts", workloads.OPT_30B.shard(8), [16384] * 32, 0.0, None),
    ]


def run_serve_sim(args, dev):
    """bench.py --serve-sim [--serve-sim-out PATH]: one row per configuration and launch mode (eager steps, which
    bring the rows in with the copy engines, and CUDA-graph replays, which stream them with the SMs) in the columns
    of the reference's serving benchmark; prints the rows as JSON lines and appends them to the CSV."""
    import csv

    from directkv_b200 import serve_sim

    only = set(args.serve_sim.split(",")) if args.serve_sim != "all" else None
    rows = []
    for name, shape, lens, churn, fresh in serve_sim_configs():
        if only is not None and name.split()[0] not in only:
            continue
        for use_graph in (False, True):
            r = serve_sim.run_config(name, shape, lens, dev, decode_steps=args.serve_sim_steps, churn=churn, fresh_lens=fresh,
                                     use_graph=use_graph, check_each_step=os.environ.get("DIRECTKV_B200_SIM_CHECK") == "1")
            rows.append(r)
            print(json.dumps(r), flush=True)
    if args.serve_sim_out:
        os.makedirs(os.path.dirname(args.serve_sim_out) or ".", exist_ok=True)
        exists = os.path.exists(args.serve_sim_out)
        with open(args.serve_sim_out, "a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=serve_sim.SERVING_CSV_HEADER, extrasaction="ignore")
            if not exists:
                w.writeheader()
            for r in rows:
                w.writerow({k: r.get(k, "") for k in serve_sim.SERVING_CSV_HEADER})


# ---------------------------------------------------------------------------------------------------
# Multi-GPU parts of the default run: parity on a small case, and the 1M-token sequence split.
# ---------------------------------------------------------------------------------------------------
def multi_gpu_check(rank, world, dev, dist):
    """Head shard, sequence split with the NCCL all-gather and with the fused peer-memory exchange, each against the
    CPU oracle on a small seeded case (the case of tests/test_sharding_gpu.py; outside every timed region).
    Returns the worst absolute errors; raises when one misses the parity bar or the device status word is set."""
    from directkv_b200 import kernel, sharding
    from directkv_b200._lib import get_context
    from oracle import directkv_oracle as orc

    ctx = get_context(dev.index)
    atol, rtol = 2e-2, 1e-2

    def worst(out, ref, what):
        err = (out.float().cpu() - ref).abs()
        if not bool((err <= atol + rtol * ref.abs()).all()):
            raise RuntimeError(f"multi_gpu_check: {what} outside the parity bar on rank {rank}: max abs err {float(err.max()):.3e}")
        return float(err.max())

    def allmax(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    shape = workloads.LayerShape("check", 256, 8 * world, 2 * world, 10000.0)     # 2 KV heads per rank
    lens = [5, 130, 1000, 64]
    full = workloads.make_decode_case(shape, lens, PAGE, 11, "cpu", kv_on_host=True)
    ref = orc.decode_layer(full["x"], full["wk"], full["wv"], full["q"], full["k_pool"].clone(), full["v_pool"].clone(),
                           full["page_table"], lens, PAGE, full["cos_sin"], shape.scale)
    sh = sharding.HeadShard(rank, world, shape.nh_q, shape.nh_kv)
    wk, wv = sh.weights(full["wk"], full["wv"])
    k_loc, v_loc = sh.pool(full["k_pool"]).pin_memory(), sh.pool(full["v_pool"]).pin_memory()
    kernel.register_layer(40, k_loc, v_loc, wk.to(dev), wv.to(dev), full["cos_sin"].to(dev), page_size=PAGE, device=dev.index)
    out = kernel.decode(40, sh.queries(full["q"]).to(dev), full["seq_lens"].to(dev), shape.scale,
                        page_table=full["page_table"].to(dev), x=full["x"].to(dev))
    ctx.raise_on_status()
    e_head = worst(out, ref[:, sh.q_heads.start:sh.q_heads.stop], "head-sharded output")
    kernel.unregister_layer(40)

    one_shape = workloads.LayerShape("check1", 256, 8, 2, 10000.0)
    n = 3000
    one = workloads.make_decode_case(one_shape, [n + 1], PAGE, 12, "cpu", kv_on_host=True)
    plan = sharding.plan_sequence_split(n + 1, world, PAGE)
    owner = sharding.owner_of_new_token(plan)
    s0, e0 = plan[rank]
    pages = one["page_table"][:, s0 // PAGE: -(-e0 // PAGE)].contiguous().to(dev)
    if pages.size(1) == 0:
        pages = torch.zeros(1, 1, dtype=torch.int32, device=dev)
    kp, vp = one["k_pool"].pin_memory(), one["v_pool"].pin_memory()
    kernel.register_layer(41, kp, vp, one["wk"].to(dev), one["wv"].to(dev), one["cos_sin"].to(dev), page_size=PAGE, device=dev.index)
    is_owner = rank == owner
    lens_dev = torch.tensor([e0 - s0], dtype=torch.int32, device=dev)
    off_dev = torch.tensor([s0], dtype=torch.int32, device=dev)
    x_dev = one["x"].to(dev) if is_owner else None
    ref1 = orc.decode_layer(one["x"], one["wk"], one["wv"], one["q"], one["k_pool"].clone(), one["v_pool"].clone(),
                            one["page_table"], [n + 1], PAGE, one["cos_sin"], one_shape.scale)
    o = sharding.sequence_split_decode(41, one["q"].to(dev), lens_dev, one_shape.scale, pages, x=x_dev,
                                       pos_offset=off_dev if is_owner else None)
    ctx.raise_on_status()
    e_nccl = worst(o, ref1, "sequence split (NCCL) output")
    # Fused exchange: steps back to back without host synchronisation, a different query in each.
    steps = 200
    g = torch.Generator().manual_seed(77)
    q_steps = torch.randn(steps, 1, one_shape.nh_q, 128, generator=g).to(torch.bfloat16)
    q_dev = q_steps.to(dev)
    outs = torch.empty(steps, 1, one_shape.nh_q, 128, dtype=torch.bfloat16, device=dev)
    ex = sharding.PartialExchange(max_rows=64, device=dev.index)
    for it in range(steps):
        kernel.decode(41, q_dev[it], lens_dev, one_shape.scale, page_table=pages, x=x_dev,
                      pos_offset=off_dev if is_owner else None, out=outs[it], exchange=ex.handle)
    torch.cuda.synchronize()
    ctx.raise_on_status()
    e_fused = 0.0
    k_ref, v_ref = one["k_pool"].clone(), one["v_pool"].clone()
    for it in range(steps):
        r_it = orc.decode_layer(one["x"], one["wk"], one["wv"], q_steps[it], k_ref, v_ref, one["page_table"], [n + 1], PAGE,
                                one["cos_sin"], one_shape.scale)
        e_fused = max(e_fused, worst(outs[it], r_it, f"sequence split (fused exchange) output of step {it}"))
    ex.close()
    kernel.unregister_layer(41)
    return {"head_shard_max_err": allmax(e_head), "seq_split_nccl_max_err": allmax(e_nccl),
            "seq_split_fused_max_err": allmax(e_fused), "steps": steps, "bar": "2e-2 abs + 1e-2 rel", "status": 0}


def measure_seq_split(rank, world, dev, dist, ctx_len=1 << 20, layers=8, iters=3):
    """One Llama-3-8B request of `ctx_len` tokens split by sequence over the ranks, pool in pinned host memory:
    `layers` layer steps per timed call (one layer's pool is used for all of them), partial (O, m, l) merged with
    an NCCL all-gather or by the fused peer-memory exchange.  Device-timed, maximum over ranks."""
    from directkv_b200 import kernel, sharding
    from directkv_b200._lib import get_context

    ctx = get_context(dev.index)
    shape = workloads.LLAMA3_8B
    plan = sharding.plan_sequence_split(ctx_len + 1, world, PAGE)
    owner = sharding.owner_of_new_token(plan)
    s0, e0 = plan[rank]
    n_loc = e0 - s0
    case = workloads.make_decode_case(shape, [max(n_loc, 1)], PAGE, 2 + rank, dev, kv_on_host=True)
    cs = workloads.build_cos_sin(ctx_len + 2, shape.rope_theta, device=dev)
    kernel.register_layer(42, case["k_pool"], case["v_pool"], case["wk"], case["wv"], cs, page_size=PAGE, device=dev.index)
    lens_dev = torch.tensor([n_loc], dtype=torch.int32, device=dev)
    off = torch.tensor([s0], dtype=torch.int32, device=dev)
    is_owner = rank == owner
    # every rank attends the same query (rank 0's)
    q = case["q"].clone()
    dist.broadcast(q, src=0)
    x = case["x"] if is_owner else None
    ex = sharding.PartialExchange(max_rows=shape.nh_q, device=dev.index)
    out_f = torch.empty_like(q)

    def run_nccl():
        o = None
        for _ in range(layers):
            o = sharding.sequence_split_decode(42, q, lens_dev, shape.scale, case["page_table"], x=x,
                                               pos_offset=off if is_owner else None)
        return o

    def run_fused():
        for _ in range(layers):
            kernel.decode(42, q, lens_dev, shape.scale, page_table=case["page_table"], x=x,
                          pos_offset=off if is_owner else None, out=out_f, exchange=ex.handle)
        return out_f

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            dist.barrier(device_ids=[dev.index])
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t.item()))
        return statistics.median(ts)

    ms_nccl = timed(run_nccl)
    o_nccl = run_nccl().float().clone()
    ms_fused = timed(run_fused)
    o_fused = run_fused().float().view_as(o_nccl)
    torch.cuda.synchronize()
    ctx.raise_on_status()
    diff = torch.tensor([float((o_nccl - o_fused).abs().max())], dtype=torch.float64, device=dev)
    dist.all_reduce(diff, op=dist.ReduceOp.MAX)
    ex.close()
    kernel.unregister_layer(42)
    kvb = workloads.kv_bytes(shape, [ctx_len + 1]) * layers
    best = min(ms_nccl, ms_fused)
    return {"workload": "llama3-8b layer, one request, KV in pinned host memory, split by sequence over the ranks",
            "ctx": ctx_len, "layers": layers, "ms_per_layer_nccl": ms_nccl / layers, "ms_per_layer_fused": ms_fused / layers,
            "kv_gbs_aggregate": kvb / best / 1e6, "kv_gbs_aggregate_nccl": kvb / ms_nccl / 1e6,
            "kv_gbs_aggregate_fused": kvb / ms_fused / 1e6, "nccl_vs_fused_max_diff": float(diff.item()),
            "note": "one layer's pool re-used for all layers of a call; time = maximum over ranks, median of "
                    f"{iters} calls of {layers} layers"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--variant", type=int, default=None, help="override the streaming-kernel variant")
    ap.add_argument("--only", default="all", choices=["all", "hbm", "host", "extend"] + ["short-" + k for k in SHORT_CASES],
                    help="hbm / host: time only that mode of the decode step; extend: time the chunked-prefill path "
                         "(Llama-3-8B layer, 4096 new tokens); short-<case>: a short decode step with the pool in HBM - "
                         "short runs for profiler captures")
    ap.add_argument("--sweep", default=None, help="comma list of C1,C2,C3,C4,C5: run those configurations instead")
    ap.add_argument("--sweep-out", default="sweep.jsonl")
    ap.add_argument("--longctx-csv", default=None,
                    help="with --sweep C3: also append rows in the column layout of the reference's long-context benchmark")
    ap.add_argument("--seq-split-ctx", type=int, default=1 << 20, help="context of the sequence-split arm (N > 1)")
    ap.add_argument("--serve-sim", default=None,
                    help="'all' or a comma list of C1..C5: run the serving-level simulation of those configurations instead")
    ap.add_argument("--serve-sim-steps", type=int, default=12, help="decoded tokens per request in the simulation")
    ap.add_argument("--serve-sim-out", default=None, help="CSV (columns of the reference's serving benchmark) to append to")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    from directkv_b200 import kernel
    from directkv_b200._lib import get_context

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    if args.sweep:
        os.makedirs(os.path.dirname(args.sweep_out) or ".", exist_ok=True)
        run_sweep(args, rank, world, local_rank, dev, dist)
        if world > 1:
            dist.destroy_process_group()
        return

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])

    def reduce_ranks(x: float, op) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=op)
        return float(t.item())

    def sum_over_ranks(x):
        return reduce_ranks(x, dist.ReduceOp.SUM)

    def max_over_ranks(x):
        return reduce_ranks(x, dist.ReduceOp.MAX)

    def per_rank(x: float):
        """min / mean / max of one figure over the ranks."""
        if world == 1:
            return {"min": x, "mean": x, "max": x}
        t = torch.zeros(world, dtype=torch.float64, device=dev)
        t[rank] = x
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        v = t.tolist()
        return {"min": min(v), "mean": sum(v) / len(v), "max": max(v)}

    if args.only == "extend":
        run_extend_probe(args, dev)
        return
    if args.only.startswith("short-"):
        run_short_probe(args, dev)
        return
    if args.serve_sim:
        run_serve_sim(args, dev)
        return

    full = workloads.OPT_6_7B
    if full.nh_kv % world != 0:
        raise SystemExit(f"--gpus {world}: the layer's {full.nh_kv} KV heads do not divide over {world} ranks")
    shape = full.shard(world) if world > 1 else full        # this rank's KV heads and their query heads
    lens = c2_lengths()
    ctx = get_context(local_rank)
    if args.variant is not None:
        ctx.set("attn_variant", args.variant)

    # ---- inputs: this rank's host-resident pool, and an HBM-resident copy of it ---------------------
    case = workloads.make_decode_case(shape, lens, PAGE, CFG_ID + 100 * rank, dev, kv_on_host=True)
    k_host, v_host = case["k_pool"], case["v_pool"]
    k_hbm, v_hbm = k_host.to(dev), v_host.to(dev)
    kernel.register_layer(0, k_host, v_host, case["wk"], case["wv"], None, page_size=PAGE, device=local_rank)
    kernel.register_layer(1, k_hbm, v_hbm, case["wk"], case["wv"], None, page_size=PAGE, device=local_rank)
    B = len(lens)
    x_pin, q_pin = case["x"].cpu().pin_memory(), case["q"].cpu().pin_memory()
    len_pin = case["seq_lens"].cpu().pin_memory()
    x_dev, q_dev, len_dev = torch.empty_like(case["x"]), torch.empty_like(case["q"]), torch.empty_like(case["seq_lens"])
    out_dev = torch.empty_like(case["q"])
    out_pin = torch.empty(out_dev.shape, dtype=out_dev.dtype, pin_memory=True)
    table = case["page_table"]
    kv_total = workloads.kv_bytes(shape, lens)                       # this rank: every attended token, incl. the new one
    kv_streamed = workloads.kv_bytes(shape, [n - 1 for n in lens])   # this rank: what the streaming kernel reads
    kv_all_ranks = sum_over_ranks(float(kv_total))

    def step_host():
        kernel.decode(0, case["q"], case["seq_lens"], shape.scale, page_table=table, x=case["x"], out=out_dev)

    def step_hbm():
        kernel.decode(1, case["q"], case["seq_lens"], shape.scale, page_table=table, x=case["x"], out=out_dev)

    def step_e2e():
        x_dev.copy_(x_pin, non_blocking=True)
        q_dev.copy_(q_pin, non_blocking=True)
        len_dev.copy_(len_pin, non_blocking=True)
        kernel.decode(0, q_dev, len_dev, shape.scale, page_table=table, x=x_dev, out=out_dev)
        out_pin.copy_(out_dev, non_blocking=True)

    def timed(fn, steps, warmup):
        """ms per step of `steps` calls after `warmup` untimed ones: (maximum over ranks, this rank's own)."""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        own = e0.elapsed_time(e1) / steps
        return max_over_ranks(own), own

    def link_rate(n_copies=6):
        """Pinned host->device cudaMemcpyAsync of 1 GiB, GB/s: the median of the middle copies of a back-to-back run
        (with several ranks the first and last copy may run while other ranks are still idle)."""
        nb = 1 << 30
        hbuf = torch.empty(nb, dtype=torch.uint8, pin_memory=True)
        dbuf = torch.empty(nb, dtype=torch.uint8, device=dev)
        dbuf.copy_(hbuf, non_blocking=True)
        torch.cuda.synchronize()
        barrier()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_copies + 1)]
        evs[0].record()
        for i in range(n_copies):
            dbuf.copy_(hbuf, non_blocking=True)
            evs[i + 1].record()
        torch.cuda.synchronize()
        ts = [evs[i].elapsed_time(evs[i + 1]) for i in range(n_copies)]
        barrier()
        del hbuf, dbuf
        mid = ts[1:-1] if world > 1 else ts
        return nb / statistics.median(mid) / 1e6, nb / min(ts) / 1e6

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- host link: every rank copying at once, behind a barrier -----------------------------------------
    link_gbs, link_best = link_rate()
    link_ranks = per_rank(link_gbs)

    # ---- host-KV mode: `value` -------------------------------------------------------------------------------
    # X, Q and the lengths are on the device; the KV pool is page-locked host memory that the streaming kernel reads
    # over the host link inside the timed region.  Every launch of that kernel is bracketed by CUDA events on the
    # launching stream (the roofline figure comes from the same timed steps).
    for _ in range(args.warmup):
        step_host()
    ctx.profile_read(reset=True)
    ctx.set("profile_attn", 1)
    ms_host, ms_host_own = timed(step_host, args.steps, 0)
    attn_ms, attn_n, launches_host = ctx.profile_read(reset=True)
    ctx.set("profile_attn", 0)
    ctx.raise_on_status()
    attn_avg_ms = attn_ms / max(attn_n, 1)
    host_rank_gbs = per_rank(kv_total / ms_host_own / 1e6)
    attn_rank_gbs = per_rank(kv_streamed / attn_avg_ms / 1e6 if attn_avg_ms > 0 else 0.0)

    if args.only == "host":
        if rank == 0:
            sampler.stop()
            print(json.dumps({"metric": METRIC, "value": kv_all_ranks / ms_host / 1e6, "unit": UNIT, "ms_per_step": ms_host,
                              "attn_avg_ms": attn_avg_ms, "partial": "host-KV mode only"}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- the same through the public API with per-step host copies: `e2e` -----------------------------------
    ms_e2e, _ = timed(step_e2e, args.steps, 3)
    ctx.raise_on_status()

    # ---- HBM-resident mode (secondary object) ------------------------------------------------------------------
    # (a) roofline of the streaming kernel: eager steps with every launch of it bracketed by CUDA events; (b) the
    #     step time: K steps captured in one CUDA graph (a model runs its layers that way), the graph replayed R
    #     times so that the timed work exceeds 0.2 s; median and spread over the R replays.
    for _ in range(args.warmup):
        step_hbm()
    ctx.profile_read(reset=True)
    ctx.set("profile_attn", 1)
    ms_hbm_eager, _ = timed(step_hbm, args.steps, 0)
    hattn_ms, hattn_n, _ = ctx.profile_read(reset=True)
    ctx.set("profile_attn", 0)
    ctx.raise_on_status()
    replay_hbm = _graphed(step_hbm, args.steps)
    for _ in range(3):
        replay_hbm()
    torch.cuda.synchronize()
    est = max(ms_hbm_eager * args.steps, 1e-3)
    n_rep = int(min(400, max(10, 250.0 / est)))
    barrier()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_rep + 1)]
    evs[0].record()
    for i in range(n_rep):
        replay_hbm()
        evs[i + 1].record()
    torch.cuda.synchronize()
    barrier()
    reps = sorted(evs[i].elapsed_time(evs[i + 1]) / args.steps for i in range(n_rep))
    ms_hbm_own = statistics.median(reps)
    ms_hbm = max_over_ranks(ms_hbm_own)
    hbm_total_s = max_over_ranks(evs[0].elapsed_time(evs[n_rep]) / 1e3)
    ctx.raise_on_status()
    hattn_avg_ms = hattn_ms / max(hattn_n, 1)

    if args.only == "hbm":
        if rank == 0:
            sampler.stop()
            print(json.dumps({"metric": "decode_attention_hbm_kv_gbps", "value": kv_all_ranks / ms_hbm / 1e6, "unit": UNIT,
                              "ms_per_step": ms_hbm, "attn_avg_ms": hattn_avg_ms, "partial": "hbm only"}))
        if world > 1:
            dist.destroy_process_group()
        return

    clocks = sampler.stop() if rank == 0 else None

    # ---- N > 1: parity of the partitionings, and the sequence split at 1M tokens (outside the timed regions above) ----
    mg_check = seq_split = None
    if world > 1:
        kernel.unregister_layer(0)
        kernel.unregister_layer(1)
        del k_hbm, v_hbm, k_host, v_host, case
        torch.cuda.empty_cache()
        mg_check = multi_gpu_check(rank, world, dev, dist)
        seq_split = measure_seq_split(rank, world, dev, dist, ctx_len=args.seq_split_ctx)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peaks()
    achieved_host = kv_streamed / attn_avg_ms / 1e6 if attn_avg_ms > 0 else 0.0
    achieved_hbm = kv_streamed / hattn_avg_ms / 1e6 if hattn_avg_ms > 0 else 0.0
    variant = "attn_partial_kernel<1,16,1>"
    cpu = cpu_reference_time(min(args.steps, 20), min(args.warmup, 3), lens, budget_s=40.0) if world == 1 else None
    # Secondary numbers, outside the timed regions of the headline.
    extend = measure_extend(dev, 10, 3) if world == 1 else None
    request_pool = measure_request_pool(dev, lens) if world == 1 else None

    value = kv_all_ranks / ms_host / 1e6
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_host, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world, lens),
        "modes": {"value": "KV pool in pinned host memory, streamed over the host link by the kernel; X, Q, lengths on the "
                           f"device; eager calls of kernel.decode ({launches_host // max(args.steps, 1)} launches per step)",
                  "e2e": "the same plus per-step pinned host->device copies of X, Q and the lengths and the output back",
                  "hbm": f"KV pool resident in HBM; {args.steps} steps per CUDA graph, {n_rep} replays timed one by one"},
        "per_rank": {"kv_bytes_per_step": kv_total, "host_kv_gbs": host_rank_gbs, "streaming_kernel_gbs": attn_rank_gbs,
                     "host_link_gbs": link_ranks},
        "e2e": {"value": kv_all_ranks / ms_e2e / 1e6, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": kv_streamed + x_pin.numel() * 2 + q_pin.numel() * 2 + len_pin.numel() * 4,
                "d2h_bytes_per_step": out_pin.numel() * 2 + B * shape.nh_kv * 2 * 128 * 2,
                "steps": args.steps},
        "roofline": {"kernel": variant, "bound": "host_link", "achieved": achieved_host, "peak": link_gbs,
                     "peak_kind": "pinned host->device cudaMemcpyAsync of 1 GiB measured in this run, all ranks copying at "
                                  "once behind a barrier (rank 0's median; per_rank.host_link_gbs has the spread)",
                     "peak_best_copy": link_best, "unit": "GB/s", "frac": achieved_host / link_gbs,
                     "per_rank": {k: attn_rank_gbs[k] / link_ranks[k2] for k, k2 in (("min", "max"), ("mean", "mean"), ("max", "min"))},
                     "algorithmic_bytes": kv_streamed, "avg_launch_ms": attn_avg_ms, "launches_timed": attn_n,
                     "traffic": HOST_TRAFFIC_BYTES_PER_LAUNCH if world == 1 and args.variant is None else None,
                     "traffic_source": HOST_TRAFFIC_SOURCE if world == 1 and args.variant is None else
                                       "none: the ncu capture belongs to the 1-GPU workload and the default kernel variant"},
        "hbm": {"value": kv_all_ranks / ms_hbm / 1e6, "unit": UNIT, "ms_per_step": ms_hbm,
                "ms_per_step_spread": {"min": reps[0], "median": ms_hbm_own, "max": reps[-1], "replays": n_rep,
                                       "timed_region_s": hbm_total_s},
                "ms_per_step_eager": ms_hbm_eager, "frac_of_8TBs": kv_all_ranks / ms_hbm / 1e6 / (8000.0 * world),
                "roofline": {"kernel": variant, "bound": "hbm", "achieved": achieved_hbm, "peak": peak,
                             "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved_hbm / peak,
                             "algorithmic_bytes": kv_streamed, "avg_launch_ms": hattn_avg_ms, "launches_timed": hattn_n,
                             "traffic": HBM_TRAFFIC_BYTES_PER_LAUNCH if world == 1 and args.variant is None else None,
                             "traffic_source": HBM_TRAFFIC_SOURCE if world == 1 and args.variant is None else
                                               "none: the ncu capture belongs to the 1-GPU workload and the default kernel variant"}},
        "gpu_launches": launches_host,
        "clocks": clocks,
    }
    if mg_check is not None:
        line["multi_gpu_check"] = mg_check
    if seq_split is not None:
        line["seq_split"] = seq_split
    if extend is not None:
        line["extend"] = extend
    if request_pool is not None:
        line["e2e_request_pool"] = request_pool
    if cpu is not None:
        cpu_gbs, cpu_ms, cores, sample, _ = cpu
        line["cpu_baseline"] = {"value": cpu_gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                "ms_per_step": cpu_ms}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# Bytes per launch of the streaming kernel on the 1-GPU workload, from ncu captures of the default variant
# (attn_partial_kernel<1,16,1>): with the pool in pinned host memory the traffic that matters crosses PCIe
# (pcie__read_bytes.sum; DRAM sees 0.2-2 MB), with the pool in HBM it is dram__bytes_read.sum + dram__bytes_write.sum.
HOST_TRAFFIC_BYTES_PER_LAUNCH = 1_071_759_872
HOST_TRAFFIC_SOURCE = ("ncu pcie__read_bytes.sum of one launch (payload 977.6 MB + completion headers), "
                       "`bench.py --steps 3 --warmup 3 --only host`, -k regex:attn_partial -s 3 -c 2, --clock-control none")
HBM_TRAFFIC_BYTES_PER_LAUNCH = 980_479_744
HBM_TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum (980.14 MB) + dram__bytes_write.sum (0.34 MB) of one launch, "
                      "`bench.py --steps 3 --warmup 3 --only hbm`, -k regex:attn_partial -s 15 -c 3, --clock-control none")

if __name__ == "__main__":
    main()
