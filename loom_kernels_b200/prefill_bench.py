"""Benchmark of paged causal prefill.

    python -m loom_kernels_b200.prefill_bench [--cases gates,long] [--samples 10] [--q-tiles N]

Two groups of cases:
  gates  the shapes the reference publishes prefill latencies for (H20, matched against FlashInfer,
         docs/results/h20-flashinfer-v0.6.16.post1-paged-prefill-{,long-}eager-performance-
         20260807.json), with its protocol (crates/loom-infer-validation/src/benchmarks/matched.rs:
         141-173): one CUDA-event pair around N calls enqueued in one command scope, divided by N.
  long   prompts at serving sizes, where the operator is bound by the tensor pipe: causal FLOPs
         (4 * 128 per visible (query, key) pair and query head) over the CUDA-event time, against
         the measured BF16 GEMM throughput of this machine.
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


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--cases", default="gates,long")
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
