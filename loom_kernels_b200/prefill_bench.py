"""Benchmark of paged causal prefill.

    python -m loom_kernels_b200.prefill_bench [--cases gates,long,chunked] [--samples 10]
                                              [--q-tiles N] [--only NAME] [--plans ...]

Three groups of cases:
  gates  the shapes the reference publishes prefill latencies for (H20, matched against FlashInfer,
         docs/results/h20-flashinfer-v0.6.16.post1-paged-prefill-{,long-}eager-performance-
         20260807.json), with its protocol (crates/loom-infer-validation/src/benchmarks/matched.rs:
         141-173): one CUDA-event pair around N calls enqueued in one command scope, divided by N.
  long   prompts at serving sizes, where the operator is bound by the tensor pipe: causal FLOPs
         (4 * 128 per visible (query, key) pair and query head) over the CUDA-event time, against
         the measured BF16 GEMM throughput of this machine.
  chunked  a chunk of new tokens behind cached ones (chunked prefill at serving shapes): per-call
         device time of calls enqueued back to back over rotating copies of the pools, for the
         plan's own choice, the token-parallel kernel and the tiled kernel with one CTA per tile.
Prints one JSON object per case (JSONL).  Inputs are seeded synthetic data of the named shapes.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

import loom_kernels_b200 as lk

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# name -> (qo_lens, kv_lens, query heads, KV heads, published Loom us, published FlashInfer us)
GATE_SHAPES = {
    "mha_b1_q4_kv4_qh8_kvh8": ([4], [4], 8, 8, 4.816, 15.718),
    "mqa_b3_q2_3_1_kv4_22_35_qh8_kvh1": ([2, 3, 1], [4, 22, 35], 8, 1, 16.902, 15.630),
    "gqa4_b2_q4_2_kv23_18_qh16_kvh4": ([4, 2], [23, 18], 16, 4, 12.171, 15.677),
    "mqa_b3_q1_4_16_kv128_256_512_qh8_kvh1": ([1, 4, 16], [128, 256, 512], 8, 1, 27.917, 19.524),
    "gqa4_b2_q32_64_kv256_1024_qh16_kvh4": ([32, 64], [256, 1024], 16, 4, 260.709, 23.210),
}
# name -> (qo_lens, kv_lens, query heads, KV heads)
LONG_SHAPES = {
    "prompt_8192_gqa4_32_8": ([8192], [8192], 32, 8),
    "prompts_4x4096_gqa4_32_8": ([4096] * 4, [4096] * 4, 32, 8),
    "prompts_16x2048_gqa8_64_8": ([2048] * 16, [2048] * 16, 64, 8),
    "chunk_2048_after_14336_gqa4_32_8": ([2048], [16384], 32, 8),
    "ragged_prompts_gqa4_32_8": ([512, 3000, 64, 7000, 1500, 900, 4096, 33], None, 32, 8),
}


# Chunked prefill: a chunk of new tokens behind cached ones.  name -> (qo_lens, kv_lens, query
# heads, KV heads).  Timed back to back over rotating copies of the pools (chunked_times).
CHUNK_SHAPES = {
    "chunk_128_of_16384": ([128], [16384], 32, 8),
    "chunk_512_of_16384": ([512], [16384], 32, 8),
    "chunk_1024_of_16384": ([1024], [16384], 32, 8),
    "chunk_128_of_4096": ([128], [4096], 32, 8),
    "chunk_32_of_8192": ([32], [8192], 32, 8),
    "chunk_256_of_2048": ([256], [2048], 32, 8),
    "chunk_64_of_2048": ([64], [2048], 32, 8),
    "chunks_8x64_of_1024": ([64] * 8, [1024] * 8, 32, 8),
    "chunks_32x16_of_2048": ([16] * 32, [2048] * 32, 32, 8),
    "prompt_512": ([512], [512], 32, 8),
    "chunk_128_of_512": ([128], [512], 32, 8),
    "chunk_64_of_512": ([64], [512], 32, 8),
    # a few query tokens per request over a large batch (multi-token verification, the 1-64-token
    # append followed by attention): HBM-bound like decode
    "verify_8_b64_ctx4096": ([8] * 64, [4096] * 64, 32, 8),
    "verify_4_b256_ctx1024": ([4] * 256, [1024] * 256, 32, 8),
    "verify_8_b16_ctx8192": ([8] * 16, [8192] * 16, 32, 8),
    "verify_8_b8_ctx32768_gqa8": ([8] * 8, [32768] * 8, 64, 8),
}
# plan variants of the chunked table: label -> (algorithm, partitions) options
CHUNK_PLANS = {"plan": (0, 0), "token_parallel": (1, 0), "tiled_unsplit": (2, 1)}


def tensor_peak_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peaks = json.load(open(path))
        return float(peaks.get("bf16_tflops", 1590.0)), "measured"
    return 1590.0, "fallback"


def normal_bf16(generator, numel, device):
    return torch.randn(numel, generator=generator, device=device, dtype=torch.float32).to(
        torch.bfloat16)


class PrefillCase:
    def __init__(self, provider, name, qo_lens, kv_lens, qh, kvh, device, q_tiles=0, seed=1):
        kv_lens = list(kv_lens) if kv_lens is not None else list(qo_lens)
        self.name, self.qo_lens, self.kv_lens, self.qh, self.kvh = name, qo_lens, kv_lens, qh, kvh
        pages = [(n + 15) // 16 for n in kv_lens]
        pool = sum(pages) + 8
        rng = np.random.default_rng(seed)
        self.spec = lk.Bf16PagedPrefillSpec.new(len(qo_lens), sum(qo_lens), pool, qh, kvh)
        self.device = device
        self.use_plan(provider.plan_bf16_paged(self.spec, q_tiles=q_tiles))
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        self.q = normal_bf16(g, self.spec.query_numel(), device)
        self.k = normal_bf16(g, self.spec.kv_pages_numel(), device)
        self.v = normal_bf16(g, self.spec.kv_pages_numel(), device)
        meta = (np.concatenate([[0], np.cumsum(qo_lens)]), np.concatenate([[0], np.cumsum(pages)]),
                rng.permutation(pool)[:sum(pages)], [(n - 1) % 16 + 1 for n in kv_lens])
        self.meta = [torch.tensor(np.asarray(a, dtype=np.int32), device=device) for a in meta]
        self.out = torch.zeros(self.spec.output_numel(), dtype=torch.bfloat16, device=device)
        self.lse = torch.zeros(self.spec.lse_numel(), dtype=torch.float32, device=device)

    def use_plan(self, plan):
        """The plan to time, with the workspace a split plan needs."""
        self.plan = plan
        numel = plan.workspace_required_numel()
        self.workspace = torch.zeros(numel, dtype=torch.float32, device=self.device) if numel else None

    def flops(self):
        """4 * 128 per visible (query, key) pair and query head: Q K^T and P V, 2 FLOPs per MAC."""
        pairs = sum(q * (kv - q) + q * (q + 1) // 2 for q, kv in zip(self.qo_lens, self.kv_lens))
        return 4.0 * 128 * pairs * self.qh

    def bytes(self):
        """Q read + O written + every request's K/V read once per KV head (the ideal)."""
        qo = 2 * self.spec.query_numel() * 2
        kv = sum(self.kv_lens) * self.kvh * 128 * 2 * 2
        return qo + kv

    def time_us(self, queue, calls, samples, warmup=3):
        stream = queue.stream()
        times = []
        for sample in range(warmup + samples):
            b = queue.bindings(10)
            reads = [b.bind_read(t) for t in (self.q, self.k, self.v, *self.meta)]
            out, lse = b.bind_read_write(self.out), b.bind_read_write(self.lse)
            ws = b.bind_read_write(self.workspace) if self.workspace is not None else None
            args = lk.Bf16PagedPrefillArgs(*reads, out.write(), lse.write(), ws)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            scope = queue.begin(b)
            start.record(stream)
            for _ in range(calls):
                self.plan.enqueue_into(scope, args)
            end.record(stream)
            scope.finish().wait()
            if sample >= warmup:
                times.append(start.elapsed_time(end) * 1000.0 / calls)
        return times


def chunked_times(provider, shape, device, options, samples):
    """Per-call device time (us) of calls enqueued back to back in one scope, rotating over
    enough copies of the operands (2..8, at least 300 MB of K/V) that the pools do not stay in
    L2 from one call to the next.  Returns (times, plan info of the first copy)."""
    qo_lens, kv_lens, qh, kvh = shape
    kv_bytes = sum(kv_lens) * kvh * 256 * 2
    copies = max(2, min(8, int(300e6 / kv_bytes) + 1))
    rounds = max(1, 24 // copies)
    cases = [PrefillCase(provider, "copy", qo_lens, kv_lens, qh, kvh, device, seed=seed + 1)
             for seed in range(copies)]
    for case in cases:
        case.use_plan(provider.plan_bf16_paged(case.spec, algorithm=options[0],
                                               partitions=options[1]))
    queue = lk.CommandQueue(torch.cuda.Stream(), 2 * copies * rounds)
    stream = queue.stream()
    times = []
    for sample in range(2 + samples):
        b = queue.bindings(10 * copies)
        calls = []
        for case in cases:
            reads = [b.bind_read(t) for t in (case.q, case.k, case.v, *case.meta)]
            out, lse = b.bind_read_write(case.out), b.bind_read_write(case.lse)
            ws = b.bind_read_write(case.workspace) if case.workspace is not None else None
            calls.append((case.plan, lk.Bf16PagedPrefillArgs(*reads, out.write(), lse.write(), ws)))
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        scope = queue.begin(b)
        start.record(stream)
        for _ in range(rounds):
            for plan, call in calls:
                plan.enqueue_into(scope, call)
        end.record(stream)
        scope.finish().wait()
        if sample >= 2:
            times.append(start.elapsed_time(end) * 1000.0 / (rounds * copies))
    return times, cases[0].plan.info(), cases[0].flops()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--cases", default="gates,long",
                        help="comma list of gates, long, chunked")
    parser.add_argument("--plans", default="plan,token_parallel,tiled_unsplit",
                        help="chunked only: comma list of " + ", ".join(CHUNK_PLANS))
    parser.add_argument("--samples", type=int, default=10)
    parser.add_argument("--q-tiles", type=int, default=0)
    parser.add_argument("--only", default="", help="substring filter on case names")
    args = parser.parse_args()
    if not torch.cuda.is_available():
        sys.exit("prefill_bench needs a CUDA device; the library has no CPU path")
    device = torch.device("cuda:0")
    provider = lk.PrefillProvider.load(0)
    peak, peak_kind = tensor_peak_tflops()
    groups = args.cases.split(",")
    if "chunked" in groups:
        for name, shape in CHUNK_SHAPES.items():
            if args.only and args.only not in name:
                continue
            line = {"case": name, "protocol": "back to back, rotating copies", "us_per_call": {}}
            for label in args.plans.split(","):
                times, info, flops = chunked_times(provider, shape, device, CHUNK_PLANS[label],
                                                   args.samples)
                median = float(np.median(times))
                kv_bytes = sum(shape[1]) * shape[3] * 128 * 2 * 2  # K and V of every request once
                line["us_per_call"][label] = {
                    "median": round(median, 1), "algorithm": info.algorithm,
                    "partitions": info.partitions, "grid": info.grid,
                    "tflops": round(flops / median / 1e6, 1),
                    "kv_gbs": round(kv_bytes / median / 1e3, 0)}
            line["status"] = provider.device_status()
            print(json.dumps(line), flush=True)
    cases = []
    if "gates" in groups:
        cases += [(name, shape[:4], 100, shape[4:]) for name, shape in GATE_SHAPES.items()]
    if "long" in groups:
        cases += [(name, shape, 1, None) for name, shape in LONG_SHAPES.items()]
    for name, (qo_lens, kv_lens, qh, kvh), calls, published in cases:
        if args.only and args.only not in name:
            continue
        case = PrefillCase(provider, name, qo_lens, kv_lens, qh, kvh, device, q_tiles=args.q_tiles)
        queue = lk.CommandQueue(torch.cuda.Stream(), calls * case.plan.commands())
        times = case.time_us(queue, calls, args.samples)
        median = float(np.median(times))
        info = case.plan.info()
        line = {
            "case": name, "median_us": round(median, 3), "min_us": round(min(times), 3),
            "calls_per_sample": calls, "samples": len(times),
            "plan": {"q_tiles": info.q_tiles, "pages_per_stage": info.pages_per_stage,
                     "stages": info.stages, "grid": info.grid},
            "tflops": round(case.flops() / median / 1e6, 2),
            "tensor_frac": round(case.flops() / median / 1e6 / peak, 4),
            "tensor_peak_tflops": peak, "tensor_peak_kind": peak_kind,
            "ideal_gbs": round(case.bytes() / median / 1e3, 1),
            "status": provider.device_status(),
        }
        if published:
            line["reference_h20_us"] = {"loom": published[0], "flashinfer": published[1]}
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
