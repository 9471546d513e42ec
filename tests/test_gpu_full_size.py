"""Paged decode at the full sizes of the benchmark configurations, through the C ABI.

Each case checks
  * EVERY request against the CPU oracle on all host cores (a request's pages are gathered into a
    compact pool for the oracle; O max-abs 2e-2, row-relative 1e-2, LSE 1e-3 as in the small
    cases), and
  * size-independent properties over every row: the direct, split-K and page-balanced algorithms
    agree within the same tolerances, and moving every page to another physical slot of the pool
    (with the page table updated) leaves the direct output bit-identical (page indexing is exact).
K/V pools are generated on the device (seeded); Q and the page table come from the host.
"""
import os

import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from loom_kernels_b200 import workloads
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def provider():
    return lk.DecodeProvider.load(0)


def device_pool(pool_pages, kvh, seed, outliers=None):
    generator = torch.Generator(device="cuda:0").manual_seed(seed)
    numel = pool_pages * 16 * kvh * 128
    k = torch.randn(numel, dtype=torch.bfloat16, device="cuda:0", generator=generator)
    v = torch.randn(numel, dtype=torch.bfloat16, device="cuda:0", generator=generator)
    for page, offset in outliers or []:  # one x8 token per request stresses the softmax maximum
        row = (page * 16 + offset) * kvh * 128
        k[row:row + kvh * 128] *= 8.0
        v[row:row + kvh * 128] *= 8.0
    return k, v


def oracle_rows(oracle, w, k, v, requests):
    """Oracle O/LSE of whole requests: their pages are gathered into a compact pool."""
    outs, lses = [], []
    k4 = k.view(w.max_pages, 16 * w.kvh * 128)
    v4 = v.view(w.max_pages, 16 * w.kvh * 128)
    for r in requests:
        pages = w.indices[w.indptr[r]:w.indptr[r + 1]].astype(np.int64)
        ids = torch.from_numpy(pages).to("cuda:0")
        k_sub = H.host_bits(k4[ids].reshape(-1))
        v_sub = H.host_bits(v4[ids].reshape(-1))
        spec = oracle.paged_spec(1, len(pages), w.qh, w.kvh)
        q = w.query[r * w.qh * 128:(r + 1) * w.qh * 128]
        out, lse = oracle.paged_decode(spec, q, k_sub, v_sub, np.array([0, len(pages)], np.int32),
                                       np.arange(len(pages), dtype=np.int32),
                                       w.last[r:r + 1], threads=os.cpu_count() or 1)
        outs.append(out)
        lses.append(lse)
    return np.concatenate(outs), np.concatenate(lses)


def rows_of(bits, lse, w, requests):
    out = np.concatenate([bits[r * w.qh * 128:(r + 1) * w.qh * 128] for r in requests])
    return out, np.concatenate([lse[r * w.qh:(r + 1) * w.qh] for r in requests])


def run(provider, w, k, v, indices=None, **plan_options):
    spec = lk.Bf16PagedBatchDecodeSpec.new(w.batch, w.max_pages, w.qh, w.kvh)
    runner = H.DecodeRun(spec, w.query, k, v, w.indptr, w.indices if indices is None else indices,
                         w.last, provider=provider, **plan_options)
    return runner.run()


def check_algorithms_agree(results, large_outputs=False):
    (base_bits, base_lse), others = results[0], results[1:]
    for bits, lse in others:
        H.check_decode(bits, lse, base_bits, base_lse, lse_limit=1e-3, large_outputs=large_outputs)


def moved_pool(w, k, v, seed):
    """Every page moves to another physical slot; returns the new pools and page ids."""
    rng = np.random.default_rng(seed)
    destination = rng.permutation(w.max_pages).astype(np.int64)  # old page id -> new page id
    dest = torch.from_numpy(destination).to("cuda:0")
    row = 16 * w.kvh * 128
    k2, v2 = torch.empty_like(k), torch.empty_like(v)
    k2.view(w.max_pages, row)[dest] = k.view(w.max_pages, row)
    v2.view(w.max_pages, row)[dest] = v.view(w.max_pages, row)
    return k2, v2, destination[w.indices].astype(np.int32)


def test_c1_mha_batch1_context1024(provider, oracle):
    """MHA 32/32, one request of 1024 tokens on 64 of 256 pages: small enough for the oracle to
    check every one of the 32 x 128 outputs and 32 LSEs, on the plan the heuristic picks for it and
    on the direct, split-K and page-balanced plans a caller can pin."""
    w = workloads.c1()
    k, v = H.dev_bf16(w.key_pages), H.dev_bf16(w.value_pages)
    ospec = oracle.paged_spec(w.batch, w.max_pages, w.qh, w.kvh)
    expected = oracle.paged_decode(ospec, w.query, w.key_pages, w.value_pages, w.indptr, w.indices,
                                   w.last, threads=os.cpu_count() or 1)
    spec = lk.Bf16PagedBatchDecodeSpec.new(w.batch, w.max_pages, w.qh, w.kvh)
    chosen = provider.plan_bf16_paged_batch(spec).info()
    assert chosen.heads_per_cta * (w.kvh // chosen.heads_per_cta) == w.kvh
    assert w.kvh // chosen.heads_per_cta > 1  # several head blocks: more KV heads than a CTA takes
    results = []
    assert chosen.algorithm == lk.Bf16PagedBatchDecodeAlgorithm.ClusterSplit and chosen.commands == 1
    for options in ({}, {"partitions": 1}, {"partitions": 9, "heads_per_cta": 4},
                    {"partitions": 4, "heads_per_cta": 8}, {"balanced": 1}):
        bits, lse = run(provider, w, k, v, **options)
        H.check_decode(bits, lse, *expected, lse_limit=1e-3)
        results.append((bits, lse))
    moved_k, moved_v, moved_indices = moved_pool(w, k, v, 11)
    moved = run(provider, w, moved_k, moved_v, indices=moved_indices, partitions=1)
    assert np.array_equal(moved[0], results[1][0]) and np.array_equal(moved[1], results[1][1])


def test_c3_batch64_gqa4_context4096(provider, oracle):
    w = workloads.c3(with_values=False)
    w.query = workloads.normal_bf16(np.random.default_rng(3), w.batch * w.qh * 128)
    k, v = device_pool(w.max_pages, w.kvh, 0xC3)
    direct = run(provider, w, k, v, partitions=1)
    everyone = list(range(w.batch))
    expected = oracle_rows(oracle, w, k, v, everyone)
    H.check_decode(*rows_of(*direct, w, everyone), *expected, lse_limit=1e-3)
    check_algorithms_agree([direct, run(provider, w, k, v, partitions=4),
                            run(provider, w, k, v, balanced=1)])
    k2, v2, indices2 = moved_pool(w, k, v, 33)
    moved = run(provider, w, k2, v2, indices=indices2, partitions=1)
    assert np.array_equal(moved[0], direct[0]) and np.array_equal(moved[1], direct[1])


def test_c4_batch8_gqa8_context32768_with_outliers(provider, oracle):
    w = workloads.c4(with_values=False)
    rng = np.random.default_rng(4)
    w.query = workloads.normal_bf16(rng, w.batch * w.qh * 128)
    outliers = []
    for r in range(w.batch):
        token = int(rng.integers(0, w.kv_lens[r]))
        outliers.append((int(w.indices[w.indptr[r] + token // 16]), token % 16))
    k, v = device_pool(w.max_pages, w.kvh, 0xC4, outliers)
    split = run(provider, w, k, v, partitions=16)
    everyone = list(range(w.batch))
    expected = oracle_rows(oracle, w, k, v, everyone)
    H.check_decode(*rows_of(*split, w, everyone), *expected, lse_limit=1e-3, large_outputs=True)
    check_algorithms_agree([split, run(provider, w, k, v, partitions=1),
                            run(provider, w, k, v, balanced=1)], large_outputs=True)


@pytest.mark.parametrize("label,qh,kvh,first", [("mqa", 32, 1, 0), ("gqa4", 32, 8, 256)])
def test_c5_ragged_256_requests(provider, oracle, label, qh, kvh, first):
    lens = workloads.c5_lengths(512)[first:first + 256]
    w = workloads.decode_workload(f"C5 {label}", 256, qh, kvh, lens, 65536, 0xC5 + kvh,
                                  with_values=False)
    w.query = workloads.normal_bf16(np.random.default_rng(5), w.batch * w.qh * 128)
    k, v = device_pool(w.max_pages, w.kvh, 0xC5 + kvh)
    balanced = run(provider, w, k, v)  # what the plan chooses for this shape
    everyone = list(range(w.batch))
    expected = oracle_rows(oracle, w, k, v, everyone)
    H.check_decode(*rows_of(*balanced, w, everyone), *expected, lse_limit=1e-3)
    check_algorithms_agree([balanced, run(provider, w, k, v, partitions=1)])


def test_serving_step_graph_at_c3_size(provider, oracle):
    """One serving step as a fixed-address Graph: append the newest token of all 64 requests
    (RoPE on Q and K, scatter K/V into position 4095's slot), then decode over the pool.  The
    decode must see what the append wrote (the two commands are linked by programmatic
    dependent launch inside the Graph); a second replay with new token contents at the same
    addresses must change exactly the outputs."""
    w = workloads.c3(with_values=False)
    rng = np.random.default_rng(6)
    k, v = device_pool(w.max_pages, w.kvh, 0xC3)
    rope = lk.RopeProvider.load(0)
    spec = lk.Bf16PagedBatchDecodeSpec.new(w.batch, w.max_pages, w.qh, w.kvh)
    append_plan = rope.plan_bf16_paged_append(
        lk.Bf16RopePagedKvAppendSpec.new(w.batch, w.max_pages, w.qh, w.kvh))
    decode_plan = provider.plan_bf16_paged_batch(spec, partitions=1)
    new = {name: H.dev_bf16(workloads.normal_bf16(rng, w.batch * heads * 128))
           for name, heads in (("q", w.qh), ("k", w.kvh), ("v", w.kvh))}
    meta = [H.dev_i32(x) for x in (w.indptr, w.indices, w.last)]
    q_rot = torch.zeros(w.batch * w.qh * 128, dtype=torch.bfloat16, device="cuda:0")
    out = torch.full((spec.output_numel(),), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    lse = torch.full((spec.lse_numel(),), float("nan"), dtype=torch.float32, device="cuda:0")
    torch.cuda.synchronize()

    graph_queue = lk.GraphQueue(0, 2)
    b = graph_queue.bindings(11)
    r = {name: b.bind_read(t) for name, t in new.items()}
    m = [b.bind_read(t) for t in meta]
    h_qrot, h_k, h_v = b.bind_read_write(q_rot), b.bind_read_write(k), b.bind_read_write(v)
    h_out, h_lse = b.bind_read_write(out), b.bind_read_write(lse)

    def record(scope):
        append_plan.enqueue_into(scope, lk.Bf16RopePagedKvAppendArgs(
            r["q"], r["k"], r["v"], *m, h_qrot.write(), h_k.write(), h_v.write()))
        decode_plan.enqueue_into(scope, lk.Bf16PagedBatchDecodeArgs(
            h_qrot.read(), h_k.read(), h_v.read(), *m, h_out.write(), h_lse.write()))

    exec_ = graph_queue.capture(b, record).instantiate()
    exec_.launch().wait()
    first_out, first_lse = H.host_bits(out), lse.cpu().numpy().copy()
    assert provider.device_status() == 0
    # the oracle decodes from the pools as the device left them and the rotated query
    w.query = H.host_bits(q_rot)
    sample = [0, 40, 63]
    expected = oracle_rows(oracle, w, k, v, sample)
    H.check_decode(*rows_of(first_out, first_lse, w, sample), *expected, lse_limit=1e-3)
    # appended V rows are bit-exact copies at slot (last page, offset 15) of every request
    v_rows = v.view(w.max_pages * 16, w.kvh * 128)
    for request in sample:
        slot = int(w.indices[w.indptr[request + 1] - 1]) * 16 + 15
        assert torch.equal(v_rows[slot], new["v"].view(w.batch, -1)[request])

    for name, heads in (("q", w.qh), ("k", w.kvh), ("v", w.kvh)):
        new[name].copy_(H.dev_bf16(workloads.normal_bf16(rng, w.batch * heads * 128)))
    torch.cuda.synchronize()
    exec_.launch().wait()
    second_out = H.host_bits(out)
    assert not np.array_equal(second_out, first_out)
    w.query = H.host_bits(q_rot)
    H.check_decode(*rows_of(second_out, lse.cpu().numpy(), w, sample),
                   *oracle_rows(oracle, w, k, v, sample), lse_limit=1e-3)
    step_us = float(np.median([exec_.measure_launch_ms() * 1e3 for _ in range(10)]))
    print(f"C3 serving step (append + decode) as one Graph replay: {step_us:.1f} us")
    exec_.into_bindings()
