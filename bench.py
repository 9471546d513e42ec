#!/usr/bin/env python
"""Benchmark of the paged-decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c1|c4|c5|prefill]

One step = one paged decode call over one batch of seeded synthetic input.  At N=1 the workload is
batch-64 GQA4 32/8-head decode at context 4096 with pages scattered in a 20000-page pool, direct
(non-split) path -- the configuration the headline target is quoted on.  With N GPUs every rank
owns its own shard of requests and of the paged KV cache (same per-GPU shape, weak scaling); the
decode path has no exchange step, so the timed region contains no collective.  The optional
all-gather of output rows is timed separately and reported under "allgather".  `--workload c5`
is the strong-scaling case instead: one ragged 512-request MQA + GQA4 batch split over the ranks.
`--workload prefill` measures the step before decode (paged causal prefill of one 8192-token
prompt per GPU) in TFLOP/s against the measured BF16 GEMM throughput.

`value` is aggregate algorithmic bytes per second with inputs resident in HBM; `e2e` is the same
metric through the public API with host buffers (pinned host -> device copy of the step's Q and
page table, device -> host read of O and LSE inside the timed region; the KV cache is device
state, as in serving).  `--impl reference` times the CPU reference (the C restatement of the
reference's own CPU path) on the host cores for the same workload and metric, on a bounded sample
per step (the first 16 requests of a decode workload; the last 8 query tokens of the prefill
prompt).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "paged_decode_achieved_hbm_bandwidth"
UNIT = "GB/s"
# DRAM traffic per launch / algorithmic bytes, from the ncu capture summarised in
# profiles/paged_decode_kernel_gqa4_ctx4096.md (dram__bytes_read.sum + dram__bytes_write.sum of a
# batch-16 launch, which scales with the units processed).
TRAFFIC_RATIO = 1.017


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        clocks, max_clock, reasons = [], None, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                    "sw_power_cap"), parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c in clocks if max_clock and c > 0.5 * max_clock] or clocks
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max_clock,
                "samples": len(clocks), "reasons": sorted(reasons)}


def build_workload(name: str, rank: int, batch: int = 64):
    from loom_kernels_b200 import workloads
    if name == "c3":
        return workloads.c3(batch=batch, seed=0xC3 + rank)
    if name == "c1":
        return workloads.c1()
    if name == "c4":
        return workloads.c4()
    raise SystemExit(f"unknown workload {name}")


def reference_arm(args):
    """CPU reference on the host cores: same workload, metric and unit."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    oracle.build()
    threads = os.cpu_count() or 1
    if args.workload == "prefill":
        return reference_arm_prefill(args, oracle, threads)
    w = build_workload(args.workload, 0, args.batch)
    # bounded sample: the first `sample` requests of the workload (whole requests, all heads)
    sample = min(w.batch, args.reference_requests)
    spec = oracle.paged_spec(sample, w.max_pages, w.qh, w.kvh)
    indptr, last = w.indptr[:sample + 1], w.last[:sample]
    indices = w.indices[:indptr[-1]]
    q = w.query[:sample * w.qh * 128]
    kv_bytes = int(w.kv_lens[:sample].sum()) * w.kvh * 128 * 2 * 2
    sample_bytes = kv_bytes + 2 * q.size * 2 + sample * w.qh * 4 + (len(indices) + 2 * sample + 1) * 4
    times = []
    for step in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        oracle.paged_decode(spec, q, w.key_pages, w.value_pages, indptr, indices, last,
                            threads=threads)
        if step >= args.warmup:
            times.append(time.perf_counter() - t0)
    seconds = float(np.mean(times))
    value = sample_bytes / seconds / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "impl": "reference",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w.name, "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"first {sample} of {w.batch} requests per step "
                                   f"({sample_bytes / 1e6:.1f} MB algorithmic)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "us_per_call": seconds * 1e6 * w.batch / sample,
        "tokens_per_s": sample / seconds,
    }
    print(json.dumps(line), flush=True)


def reference_arm_prefill(args, oracle, threads):
    """The prefill workload on the host cores: the oracle over the last `rows` query tokens of the
    8192-token prompt (all heads, the whole context they see), the same sample as the
    cpu_baseline of the device line.  Inputs are seeded synthetic data of the same shape."""
    tokens, qh, kvh, rows = 8192, 32, 8, 8
    pages = (tokens + 15) // 16
    pool = pages + 8
    rng = np.random.default_rng(0xF3)

    def normal_bf16(count):
        bits = rng.standard_normal(count, dtype=np.float32).view(np.uint32)
        return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)

    q = normal_bf16(rows * qh * 128)
    k = normal_bf16(pool * 16 * kvh * 128)
    v = normal_bf16(pool * 16 * kvh * 128)
    indices = rng.permutation(pool)[:pages].astype(np.int32)
    spec = oracle.prefill_spec(1, rows, pool, qh, kvh)
    flops = 4.0 * 128 * qh * sum(tokens - rows + i + 1 for i in range(rows))
    times = []
    for step in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        oracle.paged_prefill(spec, q, k, v, [0, rows], [0, pages], indices, [(tokens - 1) % 16 + 1],
                             threads=threads)
        if step >= args.warmup:
            times.append(time.perf_counter() - t0)
    seconds = float(np.mean(times))
    value = flops / seconds / 1e12
    line = {
        "metric": "paged_prefill_tflops", "value": value, "unit": "TFLOP/s", "impl": "reference",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "paged causal prefill, one 8192-token prompt per GPU, 32/8 heads, "
                               "page size 16, scattered pages", "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"last {rows} query tokens of the prompt per step, all heads "
                                   f"({flops / 1e9:.2f} GFLOP)"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_baseline(w, seconds_budget=20.0):
    from oracle import oracle
    oracle.build()
    threads = os.cpu_count() or 1
    sample = min(w.batch, 8)
    spec = oracle.paged_spec(sample, w.max_pages, w.qh, w.kvh)
    indptr, last = w.indptr[:sample + 1], w.last[:sample]
    indices = w.indices[:indptr[-1]]
    q = w.query[:sample * w.qh * 128]
    sample_bytes = (int(w.kv_lens[:sample].sum()) * w.kvh * 128 * 2 * 2 + 2 * q.size * 2
                    + sample * w.qh * 4 + (len(indices) + 2 * sample + 1) * 4)
    times, start = [], time.perf_counter()
    while len(times) < 3 and time.perf_counter() - start < seconds_budget:
        t0 = time.perf_counter()
        oracle.paged_decode(spec, q, w.key_pages, w.value_pages, indptr, indices, last,
                            threads=threads)
        times.append(time.perf_counter() - t0)
    seconds = min(times)
    return {"value": sample_bytes / seconds / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"first {sample} of {w.batch} requests, best of {len(times)} "
                      f"({sample_bytes / 1e6:.1f} MB algorithmic, {seconds * 1e3:.0f} ms)"}


def ours(args):
    import torch
    import torch.distributed as dist

    import loom_kernels_b200 as lk

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    w = build_workload(args.workload, rank, args.batch)
    spec = lk.Bf16PagedBatchDecodeSpec.new(w.batch, w.max_pages, w.qh, w.kvh)
    provider = lk.DecodeProvider.load(local_rank)
    plan = provider.plan_bf16_paged_batch(spec, partitions=w.partitions)
    info = plan.info()

    def dev_bf16(bits):
        return torch.from_numpy(bits.view(np.int16)).to(device).view(torch.bfloat16)

    k_pages, v_pages = dev_bf16(w.key_pages), dev_bf16(w.value_pages)
    # The per-step inputs (Q + page table) live in ONE device allocation and the per-step outputs
    # (O + LSE) in another, each mirrored by one pinned host buffer, so that the end-to-end step
    # is one host->device copy, the decode, one device->host copy.
    step_in = [("q", w.query.view(np.uint8)), ("indptr", w.indptr.view(np.uint8)),
               ("indices", w.indices.view(np.uint8)), ("last", w.last.view(np.uint8))]
    offsets, cursor = {}, 0
    for name, array in step_in:
        offsets[name] = (cursor, array.size)
        cursor += (array.size + 255) // 256 * 256
    host_in = torch.empty(cursor, dtype=torch.uint8).pin_memory()
    for name, array in step_in:
        start, size = offsets[name]
        host_in[start:start + size] = torch.from_numpy(np.ascontiguousarray(array).reshape(-1))
    dev_in = host_in.to(device)

    def in_view(name, dtype):
        start, size = offsets[name]
        return dev_in[start:start + size].view(dtype)

    q_dev = in_view("q", torch.bfloat16)
    indptr_dev, indices_dev, last_dev = (in_view(n, torch.int32)
                                         for n in ("indptr", "indices", "last"))
    out_bytes = spec.output_numel() * 2
    lse_offset = (out_bytes + 255) // 256 * 256
    dev_out = torch.zeros(lse_offset + spec.lse_numel() * 4, dtype=torch.uint8, device=device)
    out = dev_out[:out_bytes].view(torch.bfloat16)
    lse = dev_out[lse_offset:].view(torch.float32)
    workspace = (torch.zeros(plan.workspace_required_numel(), dtype=torch.float32, device=device)
                 if plan.workspace_required_numel() else None)
    stream = torch.cuda.Stream(device=device)
    queue = lk.CommandQueue(stream, max(4, 2 * args.steps))
    bindings = queue.bindings(9)
    reads = [bindings.bind_read(t) for t in (q_dev, k_pages, v_pages, indptr_dev, indices_dev,
                                             last_dev)]
    h_out, h_lse = bindings.bind_read_write(out), bindings.bind_read_write(lse)
    h_ws = bindings.bind_read_write(workspace) if workspace is not None else None
    decode_args = lk.Bf16PagedBatchDecodeArgs(*reads, h_out.write(), h_lse.write(), h_ws)
    launches_per_step = plan.commands()
    algorithmic = w.algorithmic_bytes(info.partitions)

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def one_scope(steps, bindings):
        scope = queue.begin(bindings)
        for _ in range(steps):
            plan.enqueue_into(scope, decode_args)
        return scope.finish().wait()

    # ---- device-resident timing: K steps, one launch list, CUDA events on the launching stream
    bindings = one_scope(args.warmup, bindings)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with torch.cuda.stream(stream):
        start.record(stream)
        scope = queue.begin(bindings)
        for _ in range(args.steps):
            plan.enqueue_into(scope, decode_args)
        end.record(stream)
        bindings = scope.finish().wait()
    barrier()
    elapsed_ms = start.elapsed_time(end)
    clocks = sampler.stop() if rank == 0 else None
    if provider.device_status() != 0:
        raise SystemExit("a decode kernel gave up on a bounded wait; the numbers are invalid")

    # ---- end to end through the public API with host buffers ------------------------------------
    host_out = torch.empty(dev_out.numel(), dtype=torch.uint8).pin_memory()
    h2d = sum(size for _, size in offsets.values())  # bytes of Q + page table (padding excluded)
    d2h = out_bytes + spec.lse_numel() * 4

    def e2e_step(bindings):
        with torch.cuda.stream(stream):
            dev_in.copy_(host_in, non_blocking=True)
            scope = queue.begin(bindings)
            plan.enqueue_into(scope, decode_args)
            bindings = scope.finish().wait()  # the completion fence hands O and LSE back
            host_out.copy_(dev_out, non_blocking=True)
            stream.synchronize()
        return bindings

    for _ in range(max(1, args.warmup)):
        bindings = e2e_step(bindings)
    barrier()
    e2e_start, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e2e_start.record(stream)
    for _ in range(args.steps):
        bindings = e2e_step(bindings)
    with torch.cuda.stream(stream):
        e2e_end.record(stream)
    barrier()
    e2e_ms = e2e_start.elapsed_time(e2e_end)

    # ---- optional all-gather of output rows (only when the caller wants one contiguous result)
    gather_us = None
    if world > 1:
        gathered = torch.empty(world * out.numel(), dtype=torch.bfloat16, device=device)
        for _ in range(3):
            dist.all_gather_into_tensor(gathered, out)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(20):
            dist.all_gather_into_tensor(gathered, out)
        g1.record()
        barrier()
        gather_us = g0.elapsed_time(g1) * 1e3 / 20

    times = torch.tensor([elapsed_ms, e2e_ms, gather_us or 0.0], dtype=torch.float64, device=device)
    total_bytes = torch.tensor([float(algorithmic)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
    elapsed_ms, e2e_ms, gather_us = (float(x) for x in times.tolist())
    job_bytes = float(total_bytes.item())

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        step_s = elapsed_ms / 1e3 / args.steps
        per_launch_s = step_s  # the timed region is back-to-back launches of this kernel
        achieved = algorithmic / per_launch_s / 1e9
        line = {
            "metric": METRIC, "value": job_bytes / step_s / 1e9, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w.name, "per_gpu_batch": w.batch, "global_batch": w.batch * world,
                       "partitioning": "by request, one KV shard per GPU, no collective",
                       "algorithm": {0: "direct", 1: f"split-K x{info.partitions}",
                                     2: "balanced"}.get(info.algorithm, str(info.algorithm)),
                       "heads_per_cta": info.heads_per_cta, "grid": info.grid,
                       "l2": f"inputs ({w.algorithmic_bytes() / 2**20:.0f} MiB per GPU per step) "
                             "exceed the 126 MB L2; no flush needed"},
            "us_per_call": step_s * 1e6,
            "tokens_per_s": w.batch * world / step_s,
            "frac_of_8TBs_per_gpu": achieved / 8000.0,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT,
                         "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         "traffic": algorithmic * TRAFFIC_RATIO,
                         "algorithmic_bytes_per_launch": algorithmic,
                         "kernel": "paged_decode_kernel"},
            "e2e": {"value": job_bytes / (e2e_ms / 1e3 / args.steps) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "us_per_call": e2e_ms * 1e3 / args.steps},
            "gpu_launches": args.steps * launches_per_step,
            "clocks": clocks,
        }
        if world > 1:
            line["allgather"] = {"us": gather_us, "bytes_per_rank": out.numel() * 2,
                                 "note": "NCCL all-gather of output rows, timed outside the step"}
        else:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


class RaggedJob:
    """One KV-head family of the ragged mixed batch on one rank: workload, plan and device buffers."""

    def __init__(self, lk, torch, provider, label, qh, kvh, kv_lens, seed, device):
        from loom_kernels_b200 import workloads
        self.label = label
        self.w = w = workloads.decode_workload(f"C5 {label}", len(kv_lens), qh, kvh, kv_lens, 65536,
                                               seed, with_values=False)
        w.query = workloads.normal_bf16(np.random.default_rng(seed + 1), w.batch * qh * 128)
        self.spec = lk.Bf16PagedBatchDecodeSpec.new(w.batch, w.max_pages, qh, kvh)
        self.plan = provider.plan_bf16_paged_batch(self.spec)
        self.info = self.plan.info()
        generator = torch.Generator(device=device).manual_seed(seed)
        pool = w.max_pages * 16 * kvh * 128
        self.k = torch.randn(pool, dtype=torch.bfloat16, device=device, generator=generator)
        self.v = torch.randn(pool, dtype=torch.bfloat16, device=device, generator=generator)
        self.host = {"q": torch.from_numpy(w.query.view(np.int16)).pin_memory(),
                     "indptr": torch.from_numpy(w.indptr).pin_memory(),
                     "indices": torch.from_numpy(w.indices).pin_memory(),
                     "last": torch.from_numpy(w.last).pin_memory()}
        self.dev = {name: t.to(device) for name, t in self.host.items()}
        self.out = torch.zeros(self.spec.output_numel(), dtype=torch.bfloat16, device=device)
        self.lse = torch.zeros(self.spec.lse_numel(), dtype=torch.float32, device=device)
        numel = self.plan.workspace_required_numel()
        self.workspace = torch.zeros(numel, dtype=torch.float32, device=device) if numel else None
        self.out_host = torch.empty(self.out.numel(), dtype=torch.bfloat16).pin_memory()
        self.lse_host = torch.empty(self.lse.numel(), dtype=torch.float32).pin_memory()
        self.args = None

    def bind(self, lk, torch, bindings):
        reads = [bindings.bind_read(t) for t in
                 (self.dev["q"].view(torch.bfloat16), self.k, self.v, self.dev["indptr"],
                  self.dev["indices"], self.dev["last"])]
        out, lse = bindings.bind_read_write(self.out), bindings.bind_read_write(self.lse)
        ws = bindings.bind_read_write(self.workspace) if self.workspace is not None else None
        self.args = lk.Bf16PagedBatchDecodeArgs(*reads, out.write(), lse.write(), ws)

    def algorithm(self):
        names = {0: "direct", 1: f"split-K x{self.info.partitions}", 2: "balanced"}
        return (f"{names.get(self.info.algorithm, self.info.algorithm)} hc{self.info.heads_per_cta} "
                f"grid{self.info.grid}")

    def h2d(self):
        for name, host in self.host.items():
            self.dev[name].copy_(host, non_blocking=True)

    def d2h(self):
        self.out_host.copy_(self.out, non_blocking=True)
        self.lse_host.copy_(self.lse, non_blocking=True)

    def io_bytes(self):
        h2d = sum(t.numel() * t.element_size() for t in self.host.values())
        return h2d, self.out_host.numel() * 2 + self.lse_host.numel() * 4


def ragged_c5(args):
    """Strong scaling on the ragged mixed batch: 512 requests with log-uniform contexts 128..16384,
    256 MQA (32/1) + 256 GQA4 (32/8), assigned to the ranks by KV bytes; every rank runs its MQA
    shard and its GQA4 shard as two decode calls on one stream.  No collective in the step."""
    import torch
    import torch.distributed as dist

    import loom_kernels_b200 as lk
    from loom_kernels_b200 import sharding, workloads

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    provider = lk.DecodeProvider.load(local_rank)
    lens = workloads.c5_lengths(512)
    jobs = []
    for index, (label, qh, kvh, family) in enumerate((("MQA 32/1", 32, 1, lens[:256]),
                                                      ("GQA4 32/8", 32, 8, lens[256:]))):
        if args.shard:  # one rank's share of an N-way split, on this GPU alone (no scaling claim)
            of, which = (int(x) for x in args.shard.split(":"))
            owned = sharding.balanced_assignment(family, of)[which]
        else:
            owned = sharding.balanced_assignment(family, world)[rank]
        jobs.append(RaggedJob(lk, torch, provider, label, qh, kvh, family[owned],
                              0xC5 + 64 * index + rank, device))
        jobs[-1].row_counts = [len(ids) for ids in sharding.balanced_assignment(family, world)]
    commands = sum(job.plan.commands() for job in jobs)
    stream = torch.cuda.Stream(device=device)
    queue = lk.CommandQueue(stream, max(8, commands * max(args.steps, args.warmup)))
    bindings = queue.bindings(9 * len(jobs))
    for job in jobs:
        job.bind(lk, torch, bindings)

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(selected, steps, bindings):
        """`steps` back-to-back steps of the selected jobs in one scope; ms on the device."""
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            start.record(stream)
            scope = queue.begin(bindings)
            for _ in range(steps):
                for job in selected:
                    job.plan.enqueue_into(scope, job.args)
            end.record(stream)
            bindings = scope.finish().wait()
        torch.cuda.synchronize(device)
        return start.elapsed_time(end), bindings

    _, bindings = timed(jobs, args.warmup, bindings)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    step_ms, bindings = timed(jobs, args.steps, bindings)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    family_ms = []
    for job in jobs:
        ms, bindings = timed([job], args.steps, bindings)
        family_ms.append(ms / args.steps)
    if provider.device_status() != 0:
        raise SystemExit("a decode kernel gave up on a bounded wait; the numbers are invalid")

    def e2e_step(bindings):
        with torch.cuda.stream(stream):
            for job in jobs:
                job.h2d()
            scope = queue.begin(bindings)
            for job in jobs:
                job.plan.enqueue_into(scope, job.args)
            bindings = scope.finish().wait()
            for job in jobs:
                job.d2h()
            stream.synchronize()
        return bindings

    for _ in range(3):
        bindings = e2e_step(bindings)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
    for _ in range(args.steps):
        bindings = e2e_step(bindings)
    with torch.cuda.stream(stream):
        e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    # ---- optional all-gather of the output rows of both families (host-checked: no rank enters
    #      the collective unless every rank enqueued its shard), timed outside the step
    gather_us = 0.0
    if world > 1 and not args.shard:
        def gather_all():
            for job in jobs:
                rows = job.out.view(job.w.batch, -1)
                sharding.gather_output_rows_checked(rows, True, job.row_counts)
        gather_all()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            gather_all()
        g1.record()
        barrier()
        gather_us = g0.elapsed_time(g1) * 1e3 / 5

    rank_bytes = [job.w.algorithmic_bytes() for job in jobs]
    times = torch.tensor([step_ms, e2e_ms] + family_ms, dtype=torch.float64, device=device)
    totals = torch.tensor([float(sum(rank_bytes))] + [float(b) for b in rank_bytes],
                          dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    times, totals = times.tolist(), totals.tolist()
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        step_s = times[0] / 1e3 / args.steps
        gqa = jobs[1]
        gqa_s = family_ms[1] / 1e3
        achieved = rank_bytes[1] / gqa_s / 1e9
        h2d, d2h = (sum(x) for x in zip(*(job.io_bytes() for job in jobs)))
        line = {
            "metric": METRIC, "value": totals[0] / step_s / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "C5 ragged mixed decode: 256 MQA 32/1 + 256 GQA4 32/8 requests, "
                                   "contexts log-uniform 128..16384, 65536-page pool per GPU and family",
                       "partitioning": "by request, longest-first by KV bytes; no collective",
                       "requests_on_rank0": [job.w.batch for job in jobs],
                       "algorithms_on_rank0": [job.algorithm() for job in jobs],
                       "family_us_max_over_ranks": [1e3 * t for t in times[2:]],
                       "family_GBs_whole_job": [totals[1 + i] / (times[2 + i] / 1e3) / 1e9
                                                for i in range(len(jobs))],
                       "l2": "each family's pages exceed the 126 MB L2 at every N measured; no flush"},
            "us_per_call": step_s * 1e6, "tokens_per_s": 512 / step_s,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT,
                         "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                         "algorithmic_bytes_per_launch": rank_bytes[1],
                         "kernel": f"rank 0 GQA4 shard, all commands of the call ({gqa.algorithm()})"},
            "e2e": {"value": totals[0] / (times[1] / 1e3 / args.steps) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "us_per_call": times[1] * 1e3 / args.steps},
            "gpu_launches": args.steps * commands, "clocks": clocks,
        }
        if gather_us:
            line["allgather"] = {"us": gather_us,
                                 "note": "NCCL all-gather of both families' output rows (padded "
                                         "to the widest rank) with the host-side all-ranks-"
                                         "enqueued check, timed outside the step"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def prefill_workload(args):
    """`--workload prefill`: the step before decode on the same pools (built after the decode
    rows).  One step = paged causal prefill of one seeded 8192-token prompt (32 query / 8 KV heads)
    per GPU; the metric is causal FLOPs (4 * 128 per visible (query, key) pair and query head) per
    second against the measured BF16 GEMM throughput.  Same line format as the decode workloads."""
    import torch
    import torch.distributed as dist

    import loom_kernels_b200 as lk
    from loom_kernels_b200.prefill_bench import PrefillCase, tensor_peak_tflops

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    tokens, qh, kvh = 8192, 32, 8
    provider = lk.PrefillProvider.load(local_rank)
    case = PrefillCase(provider, "prompt", [tokens], [tokens], qh, kvh, device, seed=0xF3 + rank)
    stream = torch.cuda.Stream(device=device)
    queue = lk.CommandQueue(stream, 1)
    host_q = case.q.cpu().pin_memory()
    host_meta = [m.cpu().pin_memory() for m in case.meta]
    host_out = torch.empty_like(case.out, device="cpu").pin_memory()

    def step(copies: bool):
        if copies:
            with torch.cuda.stream(stream):
                case.q.copy_(host_q, non_blocking=True)
                for dst, src in zip(case.meta, host_meta):
                    dst.copy_(src, non_blocking=True)
        b = queue.bindings(9)
        reads = [b.bind_read(t) for t in (case.q, case.k, case.v, *case.meta)]
        out, lse = b.bind_read_write(case.out), b.bind_read_write(case.lse)
        scope = queue.begin(b)
        case.plan.enqueue_into(scope, lk.Bf16PagedPrefillArgs(*reads, out.write(), lse.write()))
        scope.finish().wait()
        if copies:
            with torch.cuda.stream(stream):
                host_out.copy_(case.out, non_blocking=True)
            stream.synchronize()

    def timed(copies: bool):
        for _ in range(args.warmup):
            step(copies)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if copies:
            start.record(stream)
            for _ in range(args.steps):
                step(True)
            end.record(stream)
        else:
            # the reference's protocol: every step of the timed region enqueued in one scope
            batch_queue = lk.CommandQueue(stream, args.steps)
            b = batch_queue.bindings(9)
            reads = [b.bind_read(t) for t in (case.q, case.k, case.v, *case.meta)]
            out, lse = b.bind_read_write(case.out), b.bind_read_write(case.lse)
            call = lk.Bf16PagedPrefillArgs(*reads, out.write(), lse.write())
            scope = batch_queue.begin(b)
            start.record(stream)
            for _ in range(args.steps):
                case.plan.enqueue_into(scope, call)
            end.record(stream)
            scope.finish().wait()
        torch.cuda.synchronize()
        ms = torch.tensor([start.elapsed_time(end)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / args.steps

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(False)
    clocks = sampler.stop()
    ms_e2e = timed(True)
    status = provider.device_status()
    flops = case.flops()
    peak, peak_kind = tensor_peak_tflops()
    if rank == 0:
        # CPU leg: the oracle on the last 8 query tokens of the prompt (all heads, whole context)
        from oracle import oracle
        rows = 8
        pages = (tokens + 15) // 16
        q_bits = host_q.view(torch.int16).numpy().view(np.uint16)[-rows * qh * 128:]
        k_bits = case.k.cpu().view(torch.int16).numpy().view(np.uint16)
        v_bits = case.v.cpu().view(torch.int16).numpy().view(np.uint16)
        meta = [m.numpy() for m in host_meta]
        ospec = oracle.prefill_spec(1, rows, case.spec.max_num_pages(), qh, kvh)
        cores = os.cpu_count() or 1
        begin = time.perf_counter()
        oracle.paged_prefill(ospec, q_bits, k_bits, v_bits, [0, rows], meta[1], meta[2], meta[3],
                             threads=cores)
        cpu_s = time.perf_counter() - begin
        cpu_flops = 4.0 * 128 * qh * sum(tokens - rows + i + 1 for i in range(rows))
        tflops = flops * world / (ms * 1e-3) / 1e12
        line = {
            "metric": "paged_prefill_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"paged causal prefill, one {tokens}-token prompt per GPU, "
                                   f"{qh}/{kvh} heads, page size 16, scattered pages",
                       "algorithm": ["token_parallel", "tiled_tcgen05"][case.plan.algorithm()],
                       "l2": "K/V of a prompt (33 MB) stay in L2; the operator is tensor-bound"},
            "roofline": {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "peak": peak,
                         "unit": "TFLOP/s", "frac": flops / (ms * 1e-3) / 1e12 / peak,
                         "peak_kind": f"of {peak_kind}", "traffic": None,
                         "kernel": "paged_prefill_tiled_kernel"},
            "cpu_baseline": {"value": cpu_flops / cpu_s / 1e12, "unit": "TFLOP/s", "cores": cores,
                             "kind": "port",
                             "sample": f"last {rows} query tokens of the prompt, all heads "
                                       f"({cpu_flops / 1e9:.2f} GFLOP, {cpu_s * 1e3:.0f} ms)"},
            "e2e": {"value": flops * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": int(host_q.numel() * 2 + sum(m.numel() * 4 for m in host_meta)),
                    "d2h_bytes_per_step": int(host_out.numel() * 2)},
            "clocks": clocks, "gpu_launches": args.steps, "device_status": status,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="c3", choices=["c1", "c3", "c4", "c5", "prefill"])
    parser.add_argument("--reference-requests", type=int, default=16)
    parser.add_argument("--shard", default="",
                        help="c5 only, 'N:r': time rank r's share of an N-way split on one GPU")
    parser.add_argument("--batch", type=int, default=64,
                        help="requests per GPU for the c3 workload (64 = the headline shape; "
                             "smaller values are for profiler captures)")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        reference_arm(args)
    elif args.workload == "c5":
        ragged_c5(args)
    elif args.workload == "prefill":
        prefill_workload(args)
    else:
        ours(args)


if __name__ == "__main__":
    main()
