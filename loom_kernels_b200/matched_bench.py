"""Per-configuration benchmark of the paged-decode path with the reference's timing protocol.

    python -m loom_kernels_b200.matched_bench [--cases c1,c2,c3,c4,c5,gates] [--samples 20]

Protocol = the reference's `eager_stream_batch_cuda_event`
(crates/loom-infer-validation/src/benchmarks/matched.rs:141-173): plan, allocation and upload
outside; warm-up; per sample one CUDA-event pair around N calls enqueued in ONE command scope on
one stream, divided by N; raw samples kept.  Added columns: algorithmic bytes, achieved GB/s,
fraction of the 8 TB/s nominal and of the measured copy peak, tokens/s, and the time of one
fixed-address Graph replay including its completion event (graph/mod.rs:301-323).

Working sets smaller than L2 (C1, C2, the gate shapes) are measured twice: "warm" re-runs one
copy, "cold" rotates over enough copies of the pools to exceed the 126 MB L2.
Prints one JSON object per case (JSONL), like crates/loom-infer-validation/src/support/benchmark.rs.

The reference harness is configured through the environment
(crates/loom-infer-validation/src/benchmarks/matched.rs:47-59,116-124,1245) and the same names
work here: LOOM_BENCH_WARMUP (warm-up launches), LOOM_BENCH_LAUNCHES (launches per sample),
LOOM_BENCH_SAMPLES, LOOM_BENCH_OPERATORS (comma-separated cases, as --cases), LOOM_BENCH_RUN_LABEL
and LOOM_SOURCE_COMMIT (a full 40-character commit SHA; when unset the commit of the working tree
is asked of git).  Every record carries provider_commit and run_label.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

import loom_kernels_b200 as lk
from loom_kernels_b200 import workloads

L2_BYTES = 126 * 2 ** 20
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    return float(json.load(open(path))["hbm_gbs"]) if os.path.exists(path) else 6650.0


def dev_bf16(bits, device):
    return torch.from_numpy(bits.view(np.int16)).to(device).view(torch.bfloat16)


class DecodeCase:
    def __init__(self, provider, w: workloads.DecodeWorkload, device, copies=1, heads_per_cta=0,
                 balanced=0, balanced_ctas=0):
        self.w, self.device = w, device
        self.spec = lk.Bf16PagedBatchDecodeSpec.new(w.batch, w.max_pages, w.qh, w.kvh)
        self.plan = provider.plan_bf16_paged_batch(self.spec, w.partitions, heads_per_cta,
                                                   balanced, balanced_ctas)
        self.copies = copies
        k, v = dev_bf16(w.key_pages, device), dev_bf16(w.value_pages, device)
        self.pools = [(k, v)] + [(k.clone(), v.clone()) for _ in range(copies - 1)]
        self.q = dev_bf16(w.query, device)
        self.meta = [torch.from_numpy(a).to(device) for a in (w.indptr, w.indices, w.last)]
        self.out = torch.zeros(self.spec.output_numel(), dtype=torch.bfloat16, device=device)
        self.lse = torch.zeros(self.spec.lse_numel(), dtype=torch.float32, device=device)
        n = self.plan.workspace_required_numel()
        self.ws = torch.zeros(n, dtype=torch.float32, device=device) if n else None

    def bytes(self):
        return self.w.algorithmic_bytes(self.plan.partitions())

    def units(self):
        return self.w.batch  # decode tokens per call

    def commands(self):
        return self.plan.commands()

    def bind(self, bindings):
        q = bindings.bind_read(self.q)
        meta = [bindings.bind_read(t) for t in self.meta]
        out, lse = bindings.bind_read_write(self.out), bindings.bind_read_write(self.lse)
        ws = bindings.bind_read_write(self.ws) if self.ws is not None else None
        self.args = []
        for k, v in self.pools:
            self.args.append(lk.Bf16PagedBatchDecodeArgs(q, bindings.bind_read(k),
                                                         bindings.bind_read(v), *meta,
                                                         out.write(), lse.write(), ws))

    def slots(self):
        return 7 + 2 * self.copies

    def enqueue(self, scope, call):
        self.plan.enqueue_into(scope, self.args[call % self.copies])


class AppendCase:
    def __init__(self, provider, w: workloads.AppendWorkload, device, chunked=False, copies=1):
        self.w, self.device, self.chunked, self.copies = w, device, chunked, copies
        self.q, self.k, self.v = (dev_bf16(a, device) for a in (w.query, w.key, w.value))
        self.q_out = torch.zeros_like(self.q)
        kp, vp = dev_bf16(w.key_pages, device), dev_bf16(w.value_pages, device)
        self.pools = [(kp, vp)] + [(kp.clone(), vp.clone()) for _ in range(copies - 1)]
        self.meta = [torch.from_numpy(a).to(device) for a in (w.indptr, w.indices, w.last)]
        self.chunks = []
        step = 64 if chunked else w.tokens
        for start in range(0, w.tokens, step):
            stop = min(w.tokens, start + step)
            make = (lk.Bf16RopePagedKvAppendTokensSpec.new if chunked
                    else lk.Bf16RopePagedKvAppendTokensSpec.new_extended)
            spec = make(stop - start, w.batch, w.max_pages, w.qh, w.kvh)
            self.chunks.append((start, stop, provider.plan_bf16_paged_append_tokens(spec)))
        self.batch_indices = torch.from_numpy(w.batch_indices).to(device)
        self.positions = torch.from_numpy(w.positions).to(device)

    def bytes(self):
        return self.w.algorithmic_bytes()

    def units(self):
        return self.w.tokens

    def commands(self):
        return sum(plan.commands() for _, _, plan in self.chunks)

    def slots(self):
        return 3 + 7 * len(self.chunks) + 2 * self.copies

    def bind(self, bindings):
        w = self.w
        meta = [bindings.bind_read(t) for t in self.meta]
        pools = [(bindings.bind_read_write(k), bindings.bind_read_write(v)) for k, v in self.pools]
        self.args = []
        for start, stop, plan in self.chunks:
            views = (self.q[start * w.qh * 128:stop * w.qh * 128],
                     self.k[start * w.kvh * 128:stop * w.kvh * 128],
                     self.v[start * w.kvh * 128:stop * w.kvh * 128],
                     self.batch_indices[start:stop], self.positions[start:stop])
            reads = [bindings.bind_read(t) for t in views]
            q_out = bindings.bind_read_write(self.q_out[start * w.qh * 128:stop * w.qh * 128])
            ws = None
            if plan.workspace_required_numel():  # extended plans validate into a workspace
                ws = bindings.bind_read_write(torch.zeros(plan.workspace_required_numel(),
                                                          dtype=torch.int32, device=self.device))
            per_pool = [lk.Bf16RopePagedKvAppendTokensArgs(*reads, *meta, q_out.write(), kp.write(),
                                                           vp.write(), ws) for kp, vp in pools]
            self.args.append((plan, per_pool))

    def enqueue(self, scope, call):
        for plan, per_pool in self.args:
            plan.enqueue_into(scope, per_pool[call % self.copies])


def env_int(name):
    value = os.environ.get(name)
    return int(value) if value else None


def run_identity():
    """provider_commit and run_label of BenchmarkRecord (support/benchmark.rs:5-32)."""
    commit = os.environ.get("LOOM_SOURCE_COMMIT", "")
    if commit and (len(commit) != 40 or any(c not in "0123456789abcdefABCDEF" for c in commit)):
        raise SystemExit("LOOM_SOURCE_COMMIT must be a full 40-character Git commit SHA")
    if not commit:
        import subprocess
        try:
            commit = subprocess.run(["git", "rev-parse", "HEAD"], cwd=ROOT, capture_output=True,
                                    text=True, timeout=10).stdout.strip() or "unknown"
        except OSError:
            commit = "unknown"
    return commit, os.environ.get("LOOM_BENCH_RUN_LABEL", "unlabeled")


def measure(case, name, calls, samples, warmup, device, extra=None):
    # the reference's environment overrides, when set, apply to every case
    calls = env_int("LOOM_BENCH_LAUNCHES") or calls
    samples = env_int("LOOM_BENCH_SAMPLES") or samples
    warmup = env_int("LOOM_BENCH_WARMUP") if env_int("LOOM_BENCH_WARMUP") is not None else warmup
    stream = torch.cuda.Stream(device=device)
    queue = lk.CommandQueue(stream, calls * case.commands() + 1)
    bindings = queue.bindings(case.slots())
    case.bind(bindings)
    torch.cuda.synchronize(device)

    def scope_of(n, bindings):
        scope = queue.begin(bindings)
        for call in range(n):
            case.enqueue(scope, call)
        return scope.finish().wait()

    for _ in range(max(1, warmup // calls)):
        bindings = scope_of(calls, bindings)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    samples_us = []
    for _ in range(samples):
        with torch.cuda.stream(stream):
            start.record(stream)
            scope = queue.begin(bindings)
            for call in range(calls):
                case.enqueue(scope, call)
            end.record(stream)
            bindings = scope.finish().wait()
        samples_us.append(start.elapsed_time(end) * 1e3 / calls)

    # one fixed-address Graph replay + its completion event
    graph_us = None
    try:
        gq = lk.GraphQueue(device.index or 0, case.commands() + 1)
        gb = gq.bindings(case.slots())
        case.bind(gb)
        exec_ = gq.capture(gb, lambda scope: case.enqueue(scope, 0)).instantiate()
        for _ in range(5):
            exec_.launch().wait()
        graph_us = float(np.median([exec_.measure_launch_ms() * 1e3 for _ in range(samples)]))
        exec_.into_bindings()
    except lk.LoomError as error:  # pragma: no cover - reported, not fatal
        graph_us = f"unavailable: {error.variant}"

    # the same `calls` calls captured as ONE Graph: device time per call with no host launch cost
    graph_batch_us = None
    try:
        gq = lk.GraphQueue(device.index or 0, calls * case.commands() + 1)
        gb = gq.bindings(case.slots())
        case.bind(gb)

        def record_all(scope):
            for call in range(calls):
                case.enqueue(scope, call)
        exec_ = gq.capture(gb, record_all).instantiate()
        for _ in range(3):
            exec_.launch().wait()
        graph_batch_us = float(np.median([exec_.measure_launch_ms() * 1e3 / calls
                                          for _ in range(samples)]))
        exec_.into_bindings()
        case.bind(queue.bindings(case.slots()))  # restore eager handles (not used again)
    except lk.LoomError as error:  # pragma: no cover - reported, not fatal
        graph_batch_us = f"unavailable: {error.variant}"

    us = float(np.median(samples_us))
    commit, label = run_identity()
    record = {
        "schema_version": 1, "provider": "loom_b200", "provider_commit": commit,
        "run_label": label, "measurement": "eager_stream_batch_cuda_event", "case": name,
        "dtype": "bf16", "layout": "NHD",
        "warmup_launches": warmup, "launches_per_sample": calls, "commands_per_call": case.commands(),
        "us_per_call": round(us, 3), "p10_us": round(float(np.percentile(samples_us, 10)), 3),
        "p90_us": round(float(np.percentile(samples_us, 90)), 3), "graph_us": graph_us,
        "graph_batch_us_per_call": graph_batch_us,
        "bytes_algorithmic": case.bytes(), "achieved_GBs": round(case.bytes() / us / 1e3, 1),
        "roofline_frac_8TB": round(case.bytes() / us / 1e3 / 8000, 4),
        "roofline_frac_measured": round(case.bytes() / us / 1e3 / peak_gbs(), 4),
        "tokens_per_s": round(case.units() / us * 1e6, 1),
        "samples_us": [round(s, 3) for s in samples_us],
    }
    if extra:
        record.update(extra)
    print(json.dumps(record), flush=True)
    return record


def gate_workload(name, batch, pages, qh, kvh, indptr, indices, last, seed):
    rng = np.random.default_rng(seed)
    indptr, indices, last = (np.asarray(a, dtype=np.int32) for a in (indptr, indices, last))
    kv_lens = (indptr[1:] - indptr[:-1] - 1) * 16 + last
    w = workloads.DecodeWorkload(name, batch, pages, qh, kvh, kv_lens.astype(np.int64), indptr,
                                 indices, last, partitions=1)
    pool = pages * 16 * kvh * 128
    w.query = workloads.normal_bf16(rng, batch * qh * 128)
    w.key_pages = workloads.normal_bf16(rng, pool)
    w.value_pages = workloads.normal_bf16(rng, pool)
    return w


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--cases", default="gates,c1,c2,c3,c4,c5")
    parser.add_argument("--samples", type=int, default=20)
    parser.add_argument("--device", type=int, default=0)
    args = parser.parse_args()
    device = torch.device("cuda", args.device)
    torch.cuda.set_device(device)
    decode = lk.DecodeProvider.load(args.device)
    rope = lk.RopeProvider.load(args.device)
    cases = set((os.environ.get("LOOM_BENCH_OPERATORS") or args.cases).split(","))

    if "gates" in cases:
        # the three shapes the reference published H20 numbers for (3.100 / 5.798 / 5.854 us)
        for name, shape in [("mha_b1_l1", (1, 2, 8, 8, [0, 1], [1], [1])),
                            ("mqa_b3_mixed", (3, 7, 8, 1, [0, 1, 3, 6], [4, 6, 1, 5, 0, 3],
                                              [16, 7, 16])),
                            ("gqa4_b4_reuse", (4, 8, 16, 4, [0, 1, 3, 5, 8],
                                               [7, 2, 6, 5, 1, 7, 0, 4], [3, 16, 1, 9]))]:
            w = gate_workload("gate " + name, *shape, seed=1)
            measure(DecodeCase(decode, w, device), w.name, 100, args.samples, 200, device)
        # the append shapes the reference published H20 numbers for (3.989 us for one token per
        # request at batch 4; 5.510 us eager / 8.288 us Graph for 6 explicit tokens at batch 3)
        for name, new_tokens, prior in (("append b4 16/4 one token per request", [1, 1, 1, 1],
                                         [0, 15, 16, 40]),
                                        ("append b3 16/4 six explicit tokens", [1, 2, 3],
                                         [3, 16, 30])):
            w = workloads.append_small("gate " + name, new_tokens, prior, 16, 4, 16)
            measure(AppendCase(rope, w, device, chunked=True), w.name, 100, args.samples, 200,
                    device)
    if "c1" in cases:
        w = workloads.c1()
        measure(DecodeCase(decode, w, device), w.name + " warm", 100, args.samples, 200, device)
        copies = L2_BYTES // (2 * w.key_pages.nbytes) + 2
        measure(DecodeCase(decode, w, device, copies=copies), w.name + " cold", 100, args.samples,
                200, device, {"pool_copies": copies})
    if "c2" in cases:
        w = workloads.c2()
        copies = 6  # the page rows a call writes differ per copy (Q stays warm)
        measure(AppendCase(rope, w, device), w.name + " extended warm", 50, args.samples, 100,
                device)
        measure(AppendCase(rope, w, device, copies=copies), w.name + " extended cold", 50,
                args.samples, 100, device, {"pool_copies": copies})
        measure(AppendCase(rope, w, device, chunked=True), w.name + " contract chunks of 64", 20,
                args.samples, 40, device)
    if "c3" in cases:
        w = workloads.c3()
        measure(DecodeCase(decode, w, device), w.name, 10, args.samples, 30, device)
        w.partitions = 0
        measure(DecodeCase(decode, w, device), w.name.replace("direct", "plan-chosen (balanced)"),
                10, args.samples, 30, device)
    if "c4" in cases:
        w = workloads.c4()
        measure(DecodeCase(decode, w, device), w.name, 10, args.samples, 30, device)
        w.partitions = 0
        measure(DecodeCase(decode, w, device), w.name + " (plan-chosen split)", 10, args.samples,
                30, device)
    if "c5" in cases:
        lens = workloads.c5_lengths()
        for tag, qh, kvh, ids in (("MQA 32/1", 32, 1, slice(0, 256)),
                                  ("GQA4 32/8", 32, 8, slice(256, 512))):
            w = workloads.decode_workload(f"C5 ragged {tag} b256 ctx128-16384 pool65536", 256, qh,
                                          kvh, lens[ids], 65536, 0xC5 + kvh)
            measure(DecodeCase(decode, w, device), w.name, 10, args.samples, 30, device)


if __name__ == "__main__":
    sys.exit(main())
