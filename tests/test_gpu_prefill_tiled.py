"""GPU parity of the tcgen05 (tiled) paged-prefill kernel against the CPU oracle and against the
token-parallel kernel, through the C ABI.  Same cases and limits as tests/test_gpu_prefill.py
(the reference's gates/paged_prefill.rs shapes, guards and Graph replay), with the plan forced to
the tiled algorithm, plus shapes that exercise what is particular to it: several 128-token
blocks per tile, the lazy exponent base, partly filled tiles and blocks."""
import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from tests import helpers as H
from tests.test_gpu_prefill import GATE_CASES, K_SALT, V_SALT, PrefillRun, check, ragged_case

pytestmark = pytest.mark.gpu
TILED = 2


@pytest.fixture(scope="module")
def provider():
    return lk.PrefillProvider.load(0)


@pytest.mark.parametrize("name", list(GATE_CASES))
def test_reference_gate_cases(provider, oracle, name):
    dims, qo_indptr, indptr, indices, last, salt = GATE_CASES[name]
    spec = lk.Bf16PagedPrefillSpec.new(*dims)
    q = oracle.fixture_bf16(spec.query_numel(), salt)
    k = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ K_SALT)
    v = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ V_SALT)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), q, k, v, qo_indptr,
                                                  indptr, indices, last)
    run = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last, algorithm=TILED)
    assert run.plan.algorithm() == lk.Bf16PagedPrefillAlgorithm.Tiled
    actual, actual_lse = run.run()
    check(actual, actual_lse, expected, expected_lse)


@pytest.mark.parametrize("qh,kvh", [(8, 8), (16, 4), (32, 8), (8, 1), (32, 1), (12, 4), (40, 8)])
def test_ragged_requests(provider, oracle, qh, kvh):
    rng = np.random.default_rng(qh * 100 + kvh)
    qo_lens = [70, 3, 1, 32, 17, 129]
    kv_lens = [70, 300, 45, 64, 17, 257]
    pool = 80
    case = ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool)
    dims = (len(qo_lens), sum(qo_lens), pool, qh, kvh)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=8)
    actual, actual_lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case,
                                    algorithm=TILED).run()
    check(actual, actual_lse, expected, expected_lse, gate=False)


def test_long_rows_with_a_rising_maximum(provider, oracle):
    """Keys whose scores grow along the sequence (a x4 scale on later pages) force the exponent
    base to move several times over many blocks; a x0.1 prefix keeps early rows flat."""
    rng = np.random.default_rng(31)
    qh, kvh, pool = 8, 2, 130
    qo_lens, kv_lens = [200, 40], [1500, 520]
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool)
    kf = H.bits_to_f32(k).reshape(pool, 16, kvh, 128)
    for logical, page in enumerate(indices[:int(indptr[1])]):
        kf[page] *= 0.1 if logical < 20 else (1.0 if logical < 60 else 4.0)
    k = H.bf16_bits(kf.reshape(-1))
    dims = (2, sum(qo_lens), pool, qh, kvh)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), q, k, v, qo_indptr,
                                                  indptr, indices, last, threads=8)
    actual, actual_lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), q, k, v,
                                    qo_indptr, indptr, indices, last, algorithm=TILED).run()
    check(actual, actual_lse, expected, expected_lse, gate=False)


def test_matches_the_token_parallel_kernel_on_a_long_prompt(provider, oracle):
    """A 3000-token prompt (too long for the CPU oracle in a test): both device kernels agree, and
    sampled rows agree with the oracle."""
    rng = np.random.default_rng(41)
    total, qh, kvh, pool = 3000, 16, 4, 200
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, [total], [total], qh, kvh, pool)
    spec = lk.Bf16PagedPrefillSpec.new(1, total, pool, qh, kvh)
    tiled, tiled_lse = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last,
                                  algorithm=TILED).run()
    other, other_lse = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last,
                                  algorithm=1).run()
    check(tiled, tiled_lse, other, other_lse, gate=False)
    rows = [0, 1, 127, 128, 1000, 2047, 2048, 2999]
    spec_rows = oracle.prefill_spec(len(rows), len(rows), pool, qh, kvh)
    q_rows = np.concatenate([q[r * qh * 128:(r + 1) * qh * 128] for r in rows])
    row_pages = [(r + 16) // 16 for r in rows]
    expected, expected_lse = oracle.paged_prefill(
        spec_rows, q_rows, k, v, np.arange(len(rows) + 1),
        np.concatenate([[0], np.cumsum(row_pages)]).astype(np.int32),
        np.concatenate([indices[:n] for n in row_pages]), [r % 16 + 1 for r in rows], threads=8)
    sample = np.concatenate([tiled[r * qh * 128:(r + 1) * qh * 128] for r in rows])
    sample_lse = np.concatenate([tiled_lse[r * qh:(r + 1) * qh] for r in rows])
    check(sample, sample_lse, expected, expected_lse, gate=False)


def test_guards(provider):
    """The invalid-page guard of gates/paged_prefill.rs:238-314, an out-of-range id past the causal
    limit, malformed query ranges and a query longer than its KV: rejected rows keep sentinels."""
    spec = lk.Bf16PagedPrefillSpec.new(2, 2, 8, 1, 1)
    zeros = np.zeros(spec.kv_pages_numel(), np.uint16)
    out, lse = PrefillRun(provider, spec, np.zeros(spec.query_numel(), np.uint16), zeros, zeros,
                          [0, 1, 2], [0, 1, 2], [0, 8], [1, 1], algorithm=TILED).run()
    assert np.all(out[:128] == 0) and lse[0] == 0.0
    assert np.all(np.isnan(H.bits_to_f32(out[128:]))) and np.isnan(lse[1])

    rng = np.random.default_rng(4)
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, [10, 30, 8], [64, 40, 24], 8, 2, 16)
    spec = lk.Bf16PagedPrefillSpec.new(3, 48, 16, 8, 2)

    def written(**override):
        meta = dict(qo_indptr=qo_indptr, indptr=indptr, indices=indices, last=last)
        meta.update({name: np.asarray(value, np.int32) for name, value in override.items()})
        out, lse = PrefillRun(provider, spec, q, k, v, meta["qo_indptr"], meta["indptr"],
                              meta["indices"], meta["last"], algorithm=TILED).run()
        rows = np.isfinite(lse.reshape(48, 8)).all(axis=1)
        assert np.array_equal(np.isfinite(H.bits_to_f32(out)).reshape(48, -1).all(axis=1), rows)
        return [bool(rows[a:b].all()) for a, b in ((0, 10), (10, 40), (40, 48))], bool(rows.any())

    assert written() == ([True, True, True], True)
    bad = indices.copy()
    bad[3] = 99  # the last page of request 0: no row of it is written, the others are
    assert written(indices=bad)[0] == [False, True, True]
    assert written(qo_indptr=[0, 10, 10, 48])[0] == [True, False, False]
    assert written(qo_indptr=[1, 10, 40, 48])[1] is False
    assert written(indptr=[0, 4, 7, 8])[1] is False
    assert written(last=[16, 0, 8])[0] == [True, False, True]
    assert written(indptr=[0, 4, 5, 7], indices=indices[:7], last=[16, 8, 8])[0] == \
        [True, False, True]  # request 1: 30 queries over 8 tokens


def test_fixed_address_graph_replays(provider, oracle):
    dims, qo_indptr, indptr, indices, last, salt = GATE_CASES["gqa4_token_parallel"]
    spec = lk.Bf16PagedPrefillSpec.new(*dims)
    q = oracle.fixture_bf16(spec.query_numel(), salt)
    k = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ K_SALT)
    v = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ V_SALT)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), q, k, v, qo_indptr,
                                                  indptr, indices, last)
    plan = provider.plan_bf16_paged(spec, algorithm=TILED)
    tensors = [H.dev_bf16(t) for t in (q, k, v)] + [H.dev_i32(a) for a in
                                                    (qo_indptr, indptr, indices, last)]
    out = torch.full((spec.output_numel(),), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    lse = torch.full((spec.lse_numel(),), float("nan"), dtype=torch.float32, device="cuda:0")
    torch.cuda.synchronize()
    graph_queue = lk.GraphQueue(0, 1)
    b = graph_queue.bindings(9)
    reads = [b.bind_read(t) for t in tensors]
    h_out, h_lse = b.bind_read_write(out), b.bind_read_write(lse)
    exec_ = graph_queue.capture(b, lambda scope: plan.enqueue_into(
        scope, lk.Bf16PagedPrefillArgs(*reads, h_out.write(), h_lse.write()))).instantiate()
    for replay in range(3):
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        exec_.launch().wait()
        check(H.host_bits(out), lse.cpu().numpy(), expected, expected_lse)
    assert provider.device_status() == 0
    exec_.into_bindings()


def test_chunk_after_a_long_cache(provider, oracle):
    """Chunked prefill at serving shape: a few hundred new queries over thousands of cached tokens
    (many blocks per tile, page-id windows refilled several times, no block crosses the causal
    limit until the last ones), against the oracle."""
    rng = np.random.default_rng(51)
    qo_lens, kv_lens = [130, 40], [5000, 2177]
    qh, kvh, pool = 16, 4, 460
    case = ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool)
    dims = (2, sum(qo_lens), pool, qh, kvh)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=16)
    for algorithm in (TILED, 1):
        actual, actual_lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case,
                                        algorithm=algorithm).run()
        check(actual, actual_lse, expected, expected_lse, gate=False)


def test_full_size_prompt_properties(provider, oracle):
    """An 8192-token prompt at serving head counts (32 query / 8 KV heads), the size of the prefill
    bench line, through size-independent properties over EVERY row: prefilling the prompt in two
    chunks gives, bit for bit, the rows of the one-shot call (the mask is bottom-right aligned and
    a row's arithmetic does not depend on its tile); a second run of the same plan repeats the
    first bit for bit; the plan with the KV range shared out agrees within the parity limits; and
    sampled rows agree with the CPU oracle."""
    rng = np.random.default_rng(61)
    total, first, qh, kvh, pool = 8192, 5000, 32, 8, 520
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, [total], [total], qh, kvh, pool)
    kd, vd = H.dev_bf16(k), H.dev_bf16(v)
    whole = lk.Bf16PagedPrefillSpec.new(1, total, pool, qh, kvh)
    run = PrefillRun(provider, whole, q, kd, vd, qo_indptr, indptr, indices, last, algorithm=TILED)
    one_shot, one_lse = run.run()
    again, again_lse = run.run()
    assert np.array_equal(again, one_shot)
    assert np.array_equal(again_lse.view(np.uint32), one_lse.view(np.uint32))
    pages1 = (first + 15) // 16
    out1, lse1 = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(1, first, pool, qh, kvh),
                            q[:first * qh * 128], kd, vd, [0, first], [0, pages1],
                            indices[:pages1], [(first - 1) % 16 + 1], algorithm=TILED).run()
    out2, lse2 = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(1, total - first, pool, qh, kvh),
                            q[first * qh * 128:], kd, vd, [0, total - first], indptr, indices,
                            last, algorithm=TILED).run()
    assert np.array_equal(np.concatenate([out1, out2]), one_shot)
    assert np.array_equal(np.concatenate([lse1, lse2]).view(np.uint32), one_lse.view(np.uint32))
    shared, shared_lse = PrefillRun(provider, whole, q, kd, vd, qo_indptr, indptr, indices, last,
                                    algorithm=TILED, partitions=3).run()
    check(shared, shared_lse, one_shot, one_lse, gate=False)
    rows = [0, 63, 64, 4999, 5000, 8191]
    spec_rows = oracle.prefill_spec(len(rows), len(rows), pool, qh, kvh)
    q_rows = np.concatenate([q[r * qh * 128:(r + 1) * qh * 128] for r in rows])
    row_pages = [(r + 16) // 16 for r in rows]
    expected, expected_lse = oracle.paged_prefill(
        spec_rows, q_rows, k, v, np.arange(len(rows) + 1),
        np.concatenate([[0], np.cumsum(row_pages)]).astype(np.int32),
        np.concatenate([indices[:n] for n in row_pages]), [r % 16 + 1 for r in rows], threads=16)
    sample = np.concatenate([one_shot[r * qh * 128:(r + 1) * qh * 128] for r in rows])
    sample_lse = np.concatenate([one_lse[r * qh:(r + 1) * qh] for r in rows])
    check(sample, sample_lse, expected, expected_lse, gate=False)
