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
# profiles/paged_decode_kernel_gqa4_ctx4096.md: dram__bytes_read.sum + dram__bytes_write.sum =
# 268.63 + 3.69 MB of a batch-16 launch of the timed plan (direct, 4 KV heads per CTA, 16 KB
# boxes) over its 268.72 MB of algorithmic bytes; traffic scales with the pages read.
TRAFFIC_RATIO = 1.0134


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


def setup_ranks():
    """torch.distributed over NCCL with one process per GPU (RANK / LOCAL_RANK / WORLD_SIZE)."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    return rank, local_rank, world, device


def make_barrier(torch, dist, device, world):
    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)
    return barrier


def bits_of(t):
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def oracle_check_requests(w, requests, out_bits, lse, key_pages, value_pages):
    """O and LSE of whole requests against the CPU oracle at the decode tolerances (max-abs 2e-2,
    row-relative 1e-2, LSE 1e-3).  key_pages / value_pages: host BF16 bits of the pool, or device
    tensors (the pages of a request are then fetched from the device)."""
    import torch
    from oracle import oracle
    oracle.build()
    worst = 0.0
    for r in requests:
        pages = w.indices[w.indptr[r]:w.indptr[r + 1]].astype(np.int64)
        row = 16 * w.kvh * 128
        if isinstance(key_pages, torch.Tensor):
            ids = torch.from_numpy(pages).to(key_pages.device)
            k_sub = bits_of(key_pages.view(-1, row)[ids].reshape(-1))
            v_sub = bits_of(value_pages.view(-1, row)[ids].reshape(-1))
        else:
            k_sub = key_pages.reshape(-1, row)[pages].reshape(-1)
            v_sub = value_pages.reshape(-1, row)[pages].reshape(-1)
        spec = oracle.paged_spec(1, len(pages), w.qh, w.kvh)
        q = w.query[r * w.qh * 128:(r + 1) * w.qh * 128]
        eo, el = oracle.paged_decode(spec, q, k_sub, v_sub, np.array([0, len(pages)], np.int32),
                                     np.arange(len(pages), dtype=np.int32), w.last[r:r + 1],
                                     threads=os.cpu_count() or 1)
        a = (out_bits[r * w.qh * 128:(r + 1) * w.qh * 128].astype(np.uint32) << 16).view(np.float32)
        e = (eo.astype(np.uint32) << 16).view(np.float32)
        err = float(np.abs(a - e).max())
        rel = float((np.linalg.norm((a - e).reshape(-1, 128), axis=1)
                     / np.maximum(np.linalg.norm(e.reshape(-1, 128), axis=1), 1e-6)).max())
        lse_err = float(np.abs(lse[r * w.qh:(r + 1) * w.qh] - el).max())
        if not (err <= 2e-2 and rel <= 1e-2 and lse_err <= 1e-3):
            return False, err
        worst = max(worst, err)
    return True, worst


class DecodeJob:
    """One paged-decode call of one rank: plan, device state, and `sets` independent sets of
    per-step buffers (inputs mirrored by pinned host memory, outputs plain or gathered)."""

    def __init__(self, lk, torch, provider, w, device, k_pages, v_pages, sets=2, group=None,
                 dest_rows=None, total_requests=0, gathered_qh=0, head_offset=0,
                 heads_per_cta=0):
        self.lk, self.torch, self.w, self.device, self.group = lk, torch, w, device, group
        self.spec = lk.Bf16PagedBatchDecodeSpec.new(w.batch, w.max_pages, w.qh, w.kvh)
        self.plan = provider.plan_bf16_paged_batch(self.spec, partitions=w.partitions,
                                                   heads_per_cta=heads_per_cta)
        self.info = self.plan.info()
        self.k, self.v = k_pages, v_pages
        step_in = [("q", w.query.view(np.uint8)), ("indptr", w.indptr.view(np.uint8)),
                   ("indices", w.indices.view(np.uint8)), ("last", w.last.view(np.uint8))]
        self.offsets, cursor = {}, 0
        for name, array in step_in:
            self.offsets[name] = (cursor, array.size)
            cursor += (array.size + 255) // 256 * 256
        self.out_bytes = self.spec.output_numel() * 2
        self.lse_offset = (self.out_bytes + 255) // 256 * 256
        self.host_in, self.dev_in, self.dev_out = [], [], []
        for _ in range(sets):
            host = torch.empty(cursor, dtype=torch.uint8).pin_memory()
            for name, array in step_in:
                start, size = self.offsets[name]
                host[start:start + size] = torch.from_numpy(
                    np.ascontiguousarray(array).reshape(-1))
            self.host_in.append(host)
            self.dev_in.append(host.to(device))
            self.dev_out.append(torch.zeros(self.lse_offset + self.spec.lse_numel() * 4,
                                            dtype=torch.uint8, device=device))
        numel = self.plan.workspace_required_numel()
        self.workspace = [torch.zeros(numel, dtype=torch.float32, device=device) if numel else None
                          for _ in range(sets)]
        self.h2d_bytes = sum(size for _, size in self.offsets.values())
        self.d2h_bytes = self.out_bytes + self.spec.lse_numel() * 4
        # gathered result: two peer buffers per set (O and LSE), the same on every rank
        self.total_requests = total_requests
        self.gathered_qh = gathered_qh or w.qh
        self.head_offset = head_offset
        self.gathered_out, self.gathered_lse, self.dest_rows = [], [], None
        if group is not None:
            rows = total_requests * self.gathered_qh
            for _ in range(sets):
                self.gathered_out.append(group.buffer(rows * 128, lk.BF16))
                self.gathered_lse.append(group.buffer(rows, lk.F32))
            self.dest_rows = torch.from_numpy(np.asarray(dest_rows, dtype=np.int32)).to(device)
        # what a step hands back to the host: O and LSE of this rank's requests, or -- when the
        # result is gathered -- the whole gathered O and LSE, as every rank holds them
        self.result_dev, self.result_host = [], []
        for which in range(sets):
            tensors = (list(self.gathered_tensors(which)) if group is not None
                       else [self.dev_out[which]])
            self.result_dev.append(tensors)
            self.result_host.append([torch.empty(t.numel(), dtype=t.dtype).pin_memory()
                                     for t in tensors])
        if group is not None:
            self.d2h_bytes = sum(t.numel() * t.element_size() for t in self.result_dev[0])

    def in_view(self, which, name, dtype):
        start, size = self.offsets[name]
        return self.dev_in[which][start:start + size].view(dtype)

    def out_view(self, which):
        torch = self.torch
        return (self.dev_out[which][:self.out_bytes].view(torch.bfloat16),
                self.dev_out[which][self.lse_offset:].view(torch.float32))

    def bind(self, bindings, which):
        """Binds set `which`; returns (plain args, gathered args or None)."""
        lk, torch = self.lk, self.torch
        reads = [bindings.bind_read(t) for t in (
            self.in_view(which, "q", torch.bfloat16), self.k, self.v,
            self.in_view(which, "indptr", torch.int32), self.in_view(which, "indices", torch.int32),
            self.in_view(which, "last", torch.int32))]
        out, lse = self.out_view(which)
        h_out, h_lse = bindings.bind_read_write(out), bindings.bind_read_write(lse)
        h_ws = (bindings.bind_read_write(self.workspace[which])
                if self.workspace[which] is not None else None)
        plain = lk.Bf16PagedBatchDecodeArgs(*reads, h_out.write(), h_lse.write(), h_ws)
        gathered = None
        if self.group is not None:
            g_out = bindings.bind_read_write(self.gathered_out[which].span)
            g_lse = bindings.bind_read_write(self.gathered_lse[which].span)
            gathered = (lk.Bf16PagedBatchDecodeArgs(*reads, g_out.write(), g_lse.write(), h_ws),
                        bindings.bind_read(self.dest_rows), which)
        self.handles = {"out": h_out, "lse": h_lse}
        return plain, gathered

    BINDINGS = 12

    def enqueue_plain(self, scope, plain):
        self.plan.enqueue_into(scope, plain)

    def enqueue_gathered(self, scope, gathered, defer_wait=False):
        args, dest_rows, which = gathered
        self.plan.enqueue_gathered_into(scope, args, dest_rows, self.group, self.gathered_out[which],
                                        self.gathered_lse[which], self.total_requests,
                                        self.gathered_qh, self.head_offset, defer_wait)

    def gathered_tensors(self, which):
        return (self.gathered_out[which].tensor(self.device),
                self.gathered_lse[which].tensor(self.device))

    def algorithm(self):
        names = {0: "direct", 1: f"split-K x{self.info.partitions}", 2: "balanced"}
        return (f"{names.get(self.info.algorithm, self.info.algorithm)} hc{self.info.heads_per_cta} "
                f"grid{self.info.grid}")


def timed_scope(torch, queue, stream, bindings, steps, enqueue_step):
    """`steps` steps enqueued back to back in one command scope; device milliseconds between two
    CUDA events on the queue's stream."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        start.record(stream)
        scope = queue.begin(bindings)
        for step in range(steps):
            enqueue_step(scope, step)
        end.record(stream)
        bindings = scope.finish().wait()
    torch.cuda.synchronize()
    return start.elapsed_time(end), bindings


class PipelinedSteps:
    """The end-to-end step through the public API with host buffers, two steps in flight: step n
    runs on queue n % 2 (its own stream, bindings and buffer set): pinned host -> device copy of
    the step's Q and page table, the decode, device -> host copy of its O and LSE.  While step n
    decodes, step n + 1's inputs are already on their way and step n - 1's outputs are on their way
    back; every step's copies are inside the timed region."""

    def __init__(self, lk, torch, jobs, device, gathered, commands_per_step):
        self.torch, self.jobs, self.gathered = torch, jobs, gathered
        self.streams = [torch.cuda.Stream(device=device) for _ in range(2)]
        self.queues = [lk.CommandQueue(s, commands_per_step) for s in self.streams]
        self.bindings, self.args = [], []
        for which in range(2):
            b = self.queues[which].bindings(DecodeJob.BINDINGS * len(jobs))
            self.args.append([job.bind(b, which) for job in jobs])
            self.bindings.append(b)
        self.completion = [None, None]
        self.copied = [torch.cuda.Event(), torch.cuda.Event()]
        self.decoded = None

    def step(self, n):
        torch, which = self.torch, n % 2
        stream = self.streams[which]
        self.settle(which)
        with torch.cuda.stream(stream):
            for job in self.jobs:
                job.dev_in[which].copy_(job.host_in[which], non_blocking=True)
            # the decodes of successive steps keep their order across the two streams (gathering
            # commands of one peer group must run one after the other on a GPU)
            if self.decoded is not None:
                stream.wait_event(self.decoded)
            scope = self.queues[which].begin(self.bindings[which])
            for job, (plain, gathered) in zip(self.jobs, self.args[which]):
                if self.gathered:
                    job.enqueue_gathered(scope, gathered, defer_wait=job is not self.jobs[-1])
                else:
                    job.enqueue_plain(scope, plain)
            self.completion[which] = scope.finish()
            self.decoded = torch.cuda.Event()
            self.decoded.record(stream)
            for job in self.jobs:
                for host, dev in zip(job.result_host[which], job.result_dev[which]):
                    host.copy_(dev, non_blocking=True)
            self.copied[which].record(stream)

    def settle(self, which):
        if self.completion[which] is not None:
            self.bindings[which] = self.completion[which].wait()
            self.completion[which] = None
            self.copied[which].synchronize()

    def run(self, steps):
        """Milliseconds for `steps` steps, from the first copy to the last byte back on the host."""
        torch = self.torch
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(self.streams[0])
        if len(self.streams) > 1:
            self.streams[1].wait_event(start)
        for n in range(steps):
            self.step(n)
        last = (steps - 1) % 2
        self.streams[last].wait_event(self.copied[1 - last])
        end.record(self.streams[last])
        self.settle(0)
        self.settle(1)
        torch.cuda.synchronize()
        return start.elapsed_time(end)


def kv_head_slice(w, world, rank):
    """The share of a decode workload one rank owns when the batch is split by KV head: a block of
    KV heads (and their query heads) of every request, the same page table."""
    import copy
    from loom_kernels_b200 import sharding
    kv_lo, kv_hi, q_lo, q_hi = sharding.kv_head_range(w.kvh, w.qh, world, rank)
    local = copy.copy(w)
    local.kvh, local.qh = kv_hi - kv_lo, q_hi - q_lo
    local.query = np.ascontiguousarray(
        w.query.reshape(w.batch, w.qh, 128)[:, q_lo:q_hi]).reshape(-1)
    for name in ("key_pages", "value_pages"):
        pool = getattr(w, name).reshape(w.max_pages, 16, w.kvh, 128)
        setattr(local, name, np.ascontiguousarray(pool[:, :, kv_lo:kv_hi]).reshape(-1))
    local.name = f"{w.name}, KV heads {kv_lo}..{kv_hi - 1} of {w.kvh} on this rank"
    return local, q_lo


def verify_gathered(torch, dist, job, world, rank, plain_out, plain_lse, which=0):
    """Row for row: what every rank produced (its plain, ungathered run, exchanged here with
    torch.distributed) against this rank's copy of the gathered result."""
    g_out, g_lse = job.gathered_tensors(which)
    ok = True
    counts = [None] * world
    dist.all_gather_object(counts, (plain_out.numel(), job.dest_rows.cpu().numpy(), job.w.qh,
                                    job.head_offset))
    widest = max(c[0] for c in counts)
    padded = torch.zeros(widest, dtype=torch.bfloat16, device=job.device)
    padded[:plain_out.numel()] = plain_out
    padded_lse = torch.zeros(widest // 128, dtype=torch.float32, device=job.device)
    padded_lse[:plain_lse.numel()] = plain_lse
    everyone = torch.empty(world * widest, dtype=torch.bfloat16, device=job.device)
    everyone_lse = torch.empty(world * (widest // 128), dtype=torch.float32, device=job.device)
    dist.all_gather_into_tensor(everyone, padded)
    dist.all_gather_into_tensor(everyone_lse, padded_lse)
    rows = g_out.view(job.total_requests, job.gathered_qh, 128)
    lses = g_lse.view(job.total_requests, job.gathered_qh)
    covered = torch.zeros(job.total_requests, job.gathered_qh, dtype=torch.bool, device=job.device)
    for r, (numel, dest, qh, head_offset) in enumerate(counts):
        theirs = everyone[r * widest:r * widest + numel].view(-1, qh, 128)
        theirs_lse = everyone_lse[r * (widest // 128):r * (widest // 128) + numel // 128].view(-1, qh)
        index = torch.from_numpy(dest.astype(np.int64)).to(job.device)
        mine = rows[index, head_offset:head_offset + qh]
        ok &= bool(torch.equal(mine.view(torch.int16), theirs.view(torch.int16)))
        ok &= bool(torch.equal(lses[index, head_offset:head_offset + qh], theirs_lse))
        covered[index, head_offset:head_offset + qh] = True
    return ok and bool(covered.all())


def ours(args):
    import torch
    import torch.distributed as dist

    import loom_kernels_b200 as lk
    from loom_kernels_b200 import sharding

    rank, local_rank, world, device = setup_ranks()
    barrier = make_barrier(torch, dist, device, world)
    provider = lk.DecodeProvider.load(local_rank)
    group = lk.PeerGroup.from_torch_distributed(local_rank) if world > 1 else None

    # ---- this rank's share ---------------------------------------------------------------------
    head_offset, scaling = 0, "weak"
    if args.workload == "c1" and world > 1:
        # one request: split by KV head (sharding.choose_partition), strong scaling
        full = build_workload("c1", 0)
        if sharding.choose_partition(full.batch, full.kvh, world) != "kv_head":
            raise SystemExit(f"{world} GPUs do not divide {full.kvh} KV heads")
        w, head_offset = kv_head_slice(full, world, rank)
        dest_rows, total_requests, gathered_qh = np.arange(w.batch), w.batch, full.qh
        partitioning, scaling = "by KV head, same page table on every GPU", "strong"
    else:
        w = build_workload(args.workload, rank, args.batch)
        dest_rows = rank * w.batch + np.arange(w.batch)
        total_requests, gathered_qh = w.batch * world, w.qh
        partitioning = "by request, one KV shard per GPU"

    def dev_bf16(bits):
        return torch.from_numpy(bits.view(np.int16)).to(device).view(torch.bfloat16)

    k_pages, v_pages = dev_bf16(w.key_pages), dev_bf16(w.value_pages)
    job = DecodeJob(lk, torch, provider, w, device, k_pages, v_pages, sets=2, group=group,
                    dest_rows=dest_rows, total_requests=total_requests, gathered_qh=gathered_qh,
                    head_offset=head_offset, heads_per_cta=args.heads_per_cta)
    info, plan, spec = job.info, job.plan, job.spec
    commands = plan.commands()
    algorithmic = w.algorithmic_bytes(info.partitions)
    stream = torch.cuda.Stream(device=device)
    queue = lk.CommandQueue(stream, max(8, (commands + 1) * max(args.steps, args.warmup)))
    bindings = queue.bindings(2 * DecodeJob.BINDINGS + 4)
    sets = [job.bind(bindings, which) for which in range(2)]
    nccl_plan = nccl_args = nccl_gathered = None
    if group is not None:
        # the library all-gather as a command of the scope, for comparison
        nccl_plan = lk.OutputGatherPlan(group, lk.BF16, [w.batch] * world, w.qh * 128)
        nccl_gathered = torch.zeros(world * spec.output_numel(), dtype=torch.bfloat16, device=device)
        nccl_args = lk.OutputGatherArgs(job.handles["out"].read(),
                                        bindings.bind_read_write(nccl_gathered).write())

    def plain_step(scope, step):
        job.enqueue_plain(scope, sets[1][0])  # set 1: the last bound set owns job.handles

    def gathered_step(scope, step):
        job.enqueue_gathered(scope, sets[step % 2][1])

    def nccl_step(scope, step):
        job.enqueue_plain(scope, sets[1][0])
        nccl_plan.enqueue_into(scope, nccl_args)

    # ---- verify before timing ---------------------------------------------------------------------
    verified = None
    if world > 1:
        _, bindings = timed_scope(torch, queue, stream, bindings, 1, plain_step)
        plain_out, plain_lse = (t.clone() for t in job.out_view(1))
        sample = sorted({0, w.batch - 1})
        ok, worst = oracle_check_requests(w, sample, bits_of(plain_out), plain_lse.cpu().numpy(),
                                          w.key_pages, w.value_pages)
        _, bindings = timed_scope(torch, queue, stream, bindings, 2, gathered_step)
        # no barrier here: the command's own fence means the gathered result is whole on this GPU
        for which in range(2):
            ok &= verify_gathered(torch, dist, job, world, rank, plain_out, plain_lse, which)
        if args.workload != "c1":
            _, bindings = timed_scope(torch, queue, stream, bindings, 1, nccl_step)
            everyone = torch.empty_like(nccl_gathered)
            dist.all_gather_into_tensor(everyone, plain_out)
            ok &= bool(torch.equal(everyone.view(torch.int16), nccl_gathered.view(torch.int16)))
        flag = torch.tensor([1 if ok else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        verified = bool(flag.item())
        if not verified:
            raise SystemExit("sharded or gathered results differ from the oracle / the ranks' rows")

    # ---- device-resident timing: K steps, one launch list, CUDA events on the launching stream
    main_step = gathered_step if world > 1 else plain_step
    _, bindings = timed_scope(torch, queue, stream, bindings, args.warmup, main_step)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    elapsed_ms, bindings = timed_scope(torch, queue, stream, bindings, args.steps, main_step)
    barrier()
    plain_ms = nccl_ms = 0.0
    if world > 1:
        plain_ms, bindings = timed_scope(torch, queue, stream, bindings, args.steps, plain_step)
        barrier()
        if args.workload != "c1":
            _, bindings = timed_scope(torch, queue, stream, bindings, args.warmup, nccl_step)
            barrier()
            nccl_ms, bindings = timed_scope(torch, queue, stream, bindings, args.steps, nccl_step)
            barrier()

    # ---- end to end through the public API with host buffers ------------------------------------
    pipeline = PipelinedSteps(lk, torch, [job], device, world > 1, commands)
    pipeline.run(max(2, args.warmup))
    barrier()
    e2e_ms = pipeline.run(args.steps)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if provider.device_status() != 0:
        raise SystemExit("a decode kernel gave up on a bounded wait; the numbers are invalid")

    c5 = None
    if args.workload == "c3" and not args.no_c5:
        c5 = c5_measure(args, lk, torch, dist, provider, group, rank, world, device, barrier)

    times = torch.tensor([elapsed_ms, e2e_ms, plain_ms, nccl_ms], dtype=torch.float64, device=device)
    total_bytes = torch.tensor([float(algorithmic)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
    elapsed_ms, e2e_ms, plain_ms, nccl_ms = (float(x) for x in times.tolist())
    job_bytes = float(total_bytes.item())

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        step_s = elapsed_ms / 1e3 / args.steps
        achieved = algorithmic / step_s / 1e9
        line = {
            "metric": METRIC, "value": job_bytes / step_s / 1e9, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w.name, "per_gpu_batch": w.batch,
                       "global_batch": total_requests,
                       "partitioning": partitioning + (
                           "; every step leaves the gathered O and LSE on every GPU (rows stored "
                           "to the peers by the decode kernel itself, inside the timed step)"
                           if world > 1 else ""),
                       "algorithm": {0: "direct", 1: f"split-K x{info.partitions}",
                                     2: "balanced"}.get(info.algorithm, str(info.algorithm)),
                       "heads_per_cta": info.heads_per_cta, "grid": info.grid,
                       "l2": (f"inputs ({w.algorithmic_bytes() / 2**20:.0f} MiB per GPU per step) "
                              "exceed the 126 MB L2; no flush needed"
                              if w.algorithmic_bytes() > 2 * 126 * 2**20 else
                              f"inputs ({w.algorithmic_bytes() / 2**20:.1f} MiB) fit the L2 and stay "
                              "there between steps: a warm, latency-bound figure")},
            "us_per_call": step_s * 1e6,
            "tokens_per_s": total_requests / step_s,
            "frac_of_8TBs_per_gpu": achieved / 8000.0,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT,
                         "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         "peak_note": "the peak is a read+write copy; a read-dominated kernel can "
                                      "read a little above it",
                         "traffic": algorithmic * TRAFFIC_RATIO if args.workload == "c3" else None,
                         "algorithmic_bytes_per_launch": algorithmic,
                         "kernel": "paged_decode_kernel"},
            "e2e": {"value": job_bytes / (e2e_ms / 1e3 / args.steps) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": job.h2d_bytes, "d2h_bytes_per_step": job.d2h_bytes,
                    "us_per_call": e2e_ms * 1e3 / args.steps,
                    "note": "two steps in flight on two queues; every step's copies are timed"},
            "gpu_launches": args.steps * commands,
            "clocks": clocks,
        }
        if world > 1:
            line["verified"] = verified
            line["gather"] = {
                "in_step": "peer stores from the decode kernel + epoch wait, no collective kernel",
                "us_per_step_with_gather": step_s * 1e6,
                "us_per_step_without_gather": plain_ms * 1e3 / args.steps,
                "us_per_step_with_nccl_all_gather_command":
                    nccl_ms * 1e3 / args.steps if nccl_ms else None,
                "gathered_bytes_per_gpu": job.d2h_bytes}
        else:
            line["cpu_baseline"] = cpu_baseline(w)
        if c5 is not None:
            line["c5"] = c5
        print(json.dumps(line), flush=True)
    barrier()
    if group is not None:
        group.close()
    if world > 1:
        dist.destroy_process_group()


class RaggedFamily:
    """One KV-head family of the ragged mixed batch on one rank."""

    def __init__(self, lk, torch, provider, label, qh, kvh, kv_lens, owned, seed, device, group,
                 pools=None):
        from loom_kernels_b200 import workloads
        self.label, self.owned = label, np.asarray(owned)
        w = workloads.decode_workload(f"C5 {label}", len(owned), qh, kvh, kv_lens[owned], 65536,
                                      seed, with_values=False)
        w.query = workloads.normal_bf16(np.random.default_rng(seed + 1), w.batch * qh * 128)
        if pools is None:
            generator = torch.Generator(device=device).manual_seed(seed)
            pool = w.max_pages * 16 * kvh * 128
            pools = (torch.randn(pool, dtype=torch.bfloat16, device=device, generator=generator),
                     torch.randn(pool, dtype=torch.bfloat16, device=device, generator=generator))
        self.pools = pools
        self.job = DecodeJob(lk, torch, provider, w, device, pools[0], pools[1], sets=2,
                             group=group, dest_rows=self.owned, total_requests=len(kv_lens),
                             gathered_qh=qh)


def c5_measure(args, lk, torch, dist, provider, group, rank, world, device, barrier):
    """Strong scaling on the ragged mixed batch: 512 requests with log-uniform contexts 128..16384,
    256 MQA (32/1) + 256 GQA4 (32/8), assigned to the ranks longest-first by KV bytes; every rank
    runs its MQA share and its GQA4 share as two decode calls on one stream, and every step leaves
    both families' gathered O and LSE, in request order, on every GPU."""
    from loom_kernels_b200 import sharding, workloads

    lens = workloads.c5_lengths(512)
    families = (("MQA 32/1", 32, 1, lens[:256]), ("GQA4 32/8", 32, 8, lens[256:]))
    shard = None
    if args.shard:  # one rank's share of an N-way split, on this GPU alone (no scaling claim)
        shard = tuple(int(x) for x in args.shard.split(":"))

    def build(parts, which, group, pools=None):
        return [RaggedFamily(lk, torch, provider, label, qh, kvh, family,
                             sharding.balanced_assignment(family, parts)[which],
                             0xC5 + 64 * index + which, device, group,
                             pools[index] if pools else None)
                for index, (label, qh, kvh, family) in enumerate(families)]

    def measure(fams, gathered, steps, warmup):
        jobs = [f.job for f in fams]
        commands = sum(j.plan.commands() for j in jobs)
        stream = torch.cuda.Stream(device=device)
        queue = lk.CommandQueue(stream, max(8, commands * max(steps, warmup)))
        bindings = queue.bindings(2 * DecodeJob.BINDINGS * len(jobs))
        sets = [[job.bind(bindings, which) for job in jobs] for which in range(2)]

        def step_of(selected):
            selected = list(selected)

            def step(scope, n):
                for index in selected:
                    if gathered:  # only the step's last gathering command waits for the ranks
                        jobs[index].enqueue_gathered(scope, sets[n % 2][index][1],
                                                     defer_wait=index != selected[-1])
                    else:
                        jobs[index].enqueue_plain(scope, sets[n % 2][index][0])
            return step

        everything = step_of(range(len(jobs)))
        _, bindings = timed_scope(torch, queue, stream, bindings, warmup, everything)
        barrier()
        step_ms, bindings = timed_scope(torch, queue, stream, bindings, steps, everything)
        barrier()
        family_ms = []
        for index in range(len(jobs)):
            ms, bindings = timed_scope(torch, queue, stream, bindings, steps, step_of([index]))
            family_ms.append(ms / steps)
            barrier()
        return step_ms / steps, family_ms, queue, stream, bindings, sets

    steps, warmup = max(5, min(args.steps, 20)), 3
    if shard:
        fams = build(shard[0], shard[1], None)
        step_ms, family_ms, *_ = measure(fams, False, steps, warmup)
        return {"shard": args.shard, "us_per_step": step_ms * 1e3,
                "family_us": [1e3 * t for t in family_ms],
                "algorithms": [f.job.algorithm() for f in fams]}

    fams = build(world, rank, group)
    verified = None
    if world > 1:
        # verify before timing: two requests of every family against the oracle, then the gathered
        # result row for row against every rank's own rows
        ok = True
        jobs = [f.job for f in fams]
        stream = torch.cuda.Stream(device=device)
        queue = lk.CommandQueue(stream, 16)
        bindings = queue.bindings(2 * DecodeJob.BINDINGS * len(jobs))
        sets = [[job.bind(bindings, which) for job in jobs] for which in range(2)]
        _, bindings = timed_scope(torch, queue, stream, bindings, 1, lambda scope, n: [
            job.enqueue_plain(scope, sets[0][i][0]) for i, job in enumerate(jobs)])
        plain = [tuple(t.clone() for t in job.out_view(0)) for job in jobs]
        for job, (out, lse), fam in zip(jobs, plain, fams):
            longest = int(np.argmax(job.w.kv_lens))
            good, _ = oracle_check_requests(job.w, sorted({0, longest}), bits_of(out),
                                            lse.cpu().numpy(), fam.pools[0], fam.pools[1])
            ok &= good
        _, bindings = timed_scope(torch, queue, stream, bindings, 2, lambda scope, n: [
            job.enqueue_gathered(scope, sets[n % 2][i][1], defer_wait=i + 1 < len(jobs))
            for i, job in enumerate(jobs)])
        for job, (out, lse) in zip(jobs, plain):
            for which in range(2):
                ok &= verify_gathered(torch, dist, job, world, rank, out, lse, which)
        flag = torch.tensor([1 if ok else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        verified = bool(flag.item())
        if not verified:
            raise SystemExit("C5: sharded or gathered results differ from the oracle / the ranks' rows")
        del queue, bindings, sets

    step_ms, family_ms, *_ = measure(fams, world > 1, steps, warmup)
    plain_ms = step_ms
    if world > 1:
        plain_ms, _, *_ = measure(fams, False, steps, warmup)
    rank_bytes = [f.job.w.algorithmic_bytes() for f in fams]
    times = torch.tensor([step_ms, plain_ms] + family_ms, dtype=torch.float64, device=device)
    totals = torch.tensor([float(sum(rank_bytes))], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    times = times.tolist()
    result = {
        "workload": "C5 ragged mixed decode: 256 MQA 32/1 + 256 GQA4 32/8 requests, contexts "
                    "log-uniform 128..16384, 65536-page pool per GPU and family; strong scaling",
        "partitioning": "by request, longest-first by KV bytes" + (
            "; both families' gathered O and LSE on every GPU inside the step" if world > 1 else ""),
        "us_per_step": times[0] * 1e3, "us_per_step_without_gather": times[1] * 1e3,
        "family_us_max_over_ranks": [1e3 * t for t in times[2:]],
        "whole_job_GBs": float(totals.item()) / (times[0] / 1e3) / 1e9,
        "algorithms_on_rank0": [f.job.algorithm() for f in fams],
        "requests_on_rank0": [f.job.w.batch for f in fams], "steps": steps,
    }
    if world > 1:
        result["verified"] = verified
        # the same batch on one GPU (rank 0 alone, the others wait): the strong-scaling reference
        barrier()
        single = None
        if rank == 0:
            del fams
            torch.cuda.empty_cache()
            one = build(1, 0, None)
            single, single_family, *_ = measure_single(torch, lk, one, device, steps, warmup)
        barrier()
        if rank == 0:
            result["us_per_step_on_one_gpu"] = single * 1e3
            result["family_us_on_one_gpu"] = [1e3 * t for t in single_family]
            result["speedup_over_one_gpu"] = single / times[0]
    return result


def measure_single(torch, lk, fams, device, steps, warmup):
    """The C5 step on this GPU alone (no group, no barrier): ms per step and per family."""
    jobs = [f.job for f in fams]
    commands = sum(j.plan.commands() for j in jobs)
    stream = torch.cuda.Stream(device=device)
    queue = lk.CommandQueue(stream, max(8, commands * max(steps, warmup)))
    bindings = queue.bindings(2 * DecodeJob.BINDINGS * len(jobs))
    sets = [[job.bind(bindings, which) for job in jobs] for which in range(2)]

    def step_of(selected):
        def step(scope, n):
            for index in selected:
                jobs[index].enqueue_plain(scope, sets[n % 2][index][0])
        return step

    _, bindings = timed_scope(torch, queue, stream, bindings, warmup, step_of(range(len(jobs))))
    step_ms, bindings = timed_scope(torch, queue, stream, bindings, steps, step_of(range(len(jobs))))
    family_ms = []
    for index in range(len(jobs)):
        ms, bindings = timed_scope(torch, queue, stream, bindings, steps, step_of([index]))
        family_ms.append(ms / steps)
    return step_ms / steps, family_ms, queue


def ragged_c5(args):
    """`--workload c5`: the C5 strong-scaling case as a bench line of its own."""
    import torch
    import torch.distributed as dist

    import loom_kernels_b200 as lk

    rank, local_rank, world, device = setup_ranks()
    barrier = make_barrier(torch, dist, device, world)
    provider = lk.DecodeProvider.load(local_rank)
    group = lk.PeerGroup.from_torch_distributed(local_rank) if world > 1 and not args.shard else None
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    c5 = c5_measure(args, lk, torch, dist, provider, group, rank, world, device, barrier)
    clocks = sampler.stop() if rank == 0 else None
    if provider.device_status() != 0:
        raise SystemExit("a decode kernel gave up on a bounded wait; the numbers are invalid")
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        step_s = c5["us_per_step"] / 1e6
        value = c5.get("whole_job_GBs", 0.0)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": c5.get("steps", args.steps), "warmup": 3, "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": c5.get("workload", "C5 shard"),
                                            "l2": "each family's pages exceed the 126 MB L2; no flush"},
            "us_per_call": step_s * 1e6, "tokens_per_s": 512 / step_s,
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": UNIT,
                         "frac": value / world / peak, "peak_kind": f"of {peak_kind}",
                         "traffic": None, "kernel": "all commands of the step, per GPU"},
            "c5": c5, "gpu_launches": c5.get("steps", args.steps) * 4, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    barrier()
    if group is not None:
        group.close()
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
    parser.add_argument("--heads-per-cta", type=int, default=0,
                        help="pin the KV heads one CTA streams (0 = the plan's choice)")
    parser.add_argument("--no-c5", action="store_true",
                        help="leave the C5 strong-scaling sub-object out of the c3 line")
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
