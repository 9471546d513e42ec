"""GPU parity of paged causal prefill against the CPU oracle, through the C ABI.

Cases follow crates/loom-infer-validation/src/gates/paged_prefill.rs of the reference: its five
correctness shapes (:528-610) with its limits (:16-17, O max-abs 0.015625, log2 LSE 0.01), the
invalid-page guard (:238-314) and the fixed-address Graph case (:382-526); then seeded ragged
cases over every tile shape, and the two properties that tie the operator to the decode path.
"""
import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from tests import helpers as H

pytestmark = pytest.mark.gpu
K_SALT, V_SALT = 0x4B455900, 0x56414C554500
GATE_CASES = {
    "mha_equal_lengths": ((1, 4, 2, 8, 8), [0, 4], [0, 1], [1], [4], 0x1001),
    "mqa_append_mixed": ((3, 6, 7, 8, 1), [0, 2, 5, 6], [0, 1, 3, 6], [4, 6, 1, 5, 0, 3],
                         [4, 6, 3], 0x2001),
    "gqa4_reordered_reuse": ((2, 6, 6, 16, 4), [0, 4, 6], [0, 2, 4], [5, 1, 5, 3], [7, 2], 0x4001),
    "mqa_token_parallel": ((3, 21, 64, 8, 1), [0, 1, 5, 21], [0, 8, 24, 56],
                           [7, 2, 11, 5, 13, 3, 17, 19, 23, 29, 31, 37, 41, 43, 47, 53, 59, 61, 1,
                            4, 8, 14, 22, 28, 32, 34, 36, 38, 40, 42, 44, 46, 48, 50, 52, 54, 56,
                            58, 60, 62, 0, 6, 9, 10, 12, 15, 16, 18, 20, 21, 24, 25, 26, 27, 30,
                            33], [16, 16, 16], 0x6001),
    "gqa4_token_parallel": ((2, 96, 96, 16, 4), [0, 32, 96], [0, 16, 80],
                            [15, 3, 27, 9, 31, 1, 35, 5, 39, 7, 43, 11, 47, 13, 51, 17, 19, 21, 23,
                             25, 29, 33, 37, 41, 45, 49, 53, 55, 57, 59, 61, 63, 65, 67, 69, 71,
                             73, 75, 77, 79, 81, 83, 85, 87, 89, 91, 93, 95, 0, 2, 4, 6, 8, 10, 12,
                             14, 16, 18, 20, 22, 24, 26, 28, 30, 32, 34, 36, 38, 40, 42, 44, 46,
                             48, 50, 52, 54, 56, 58, 60, 62], [16, 16], 0x8001),
}


@pytest.fixture(scope="module")
def provider():
    return lk.PrefillProvider.load(0)


class PrefillRun:
    """One paged prefill through the public API: spec -> plan -> bindings -> scope -> fence."""

    def __init__(self, provider, spec, q, k, v, qo_indptr, indptr, indices, last, q_tiles=0,
                 sentinel=float("nan"), indices_capacity=False, algorithm=1, partitions=1):
        self.provider, self.spec = provider, spec
        self.plan = provider.plan_bf16_paged(spec, q_tiles=q_tiles, algorithm=algorithm,
                                             indices_capacity=indices_capacity,
                                             partitions=partitions)
        self.queue = lk.CommandQueue(torch.cuda.Stream(), 2)
        # a split plan's chunk states; NaN so that a state the merge reads unwritten shows
        self.workspace = None
        if self.plan.workspace_required_numel():
            self.workspace = torch.full((self.plan.workspace_required_numel(),), float("nan"),
                                        dtype=torch.float32, device="cuda:0")
        self.tensors = [t if isinstance(t, torch.Tensor) else H.dev_bf16(t) for t in (q, k, v)]
        self.tensors += [H.dev_i32(a) for a in (qo_indptr, indptr, indices, last)]
        self.out = torch.full((spec.output_numel(),), sentinel, dtype=torch.bfloat16, device="cuda:0")
        self.lse = torch.full((spec.lse_numel(),), sentinel, dtype=torch.float32, device="cuda:0")
        torch.cuda.synchronize()

    def run(self):
        b = self.queue.bindings(10)
        reads = [b.bind_read(t) for t in self.tensors]
        h_out, h_lse = b.bind_read_write(self.out), b.bind_read_write(self.lse)
        h_ws = b.bind_read_write(self.workspace) if self.workspace is not None else None
        scope = self.queue.begin(b)
        self.plan.enqueue_into(scope, lk.Bf16PagedPrefillArgs(*reads, h_out.write(), h_lse.write(),
                                                              h_ws))
        completion = scope.finish()
        assert completion.submitted() == self.plan.commands()
        b = completion.wait()
        out, lse = b.take_read_write(h_out), b.take_read_write(h_lse)
        assert self.provider.device_status() == 0, "a kernel gave up on a bounded wait"
        return H.host_bits(out), lse.cpu().numpy().copy()


def check(actual, actual_lse, expected, expected_lse, gate=True):
    """Gate cases: the reference's limits.  Seeded normal data: rows that see one or two tokens
    have |O| up to ~4, where a BF16 ulp exceeds 2e-2, so the bound there is 2e-2 + 1e-2 |e|."""
    return H.check_decode(actual, actual_lse, expected, expected_lse, lse_limit=1e-3, gate=gate,
                          large_outputs=not gate)


@pytest.mark.parametrize("name", list(GATE_CASES))
@pytest.mark.parametrize("q_tiles", [0, 1, 2, 4, 8])
def test_reference_gate_cases(provider, oracle, name, q_tiles):
    dims, qo_indptr, indptr, indices, last, salt = GATE_CASES[name]
    batch, nnz, pages, qh, kvh = dims
    spec = lk.Bf16PagedPrefillSpec.new(*dims)
    spec.validate_metadata(qo_indptr, indptr, indices, last)
    q = oracle.fixture_bf16(spec.query_numel(), salt)
    k = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ K_SALT)
    v = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ V_SALT)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), q, k, v, qo_indptr,
                                                  indptr, indices, last)
    actual, actual_lse = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last,
                                    q_tiles=q_tiles).run()
    check(actual, actual_lse, expected, expected_lse)


def ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool, reuse=False):
    qo_indptr = np.concatenate([[0], np.cumsum(qo_lens)]).astype(np.int32)
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool, allow_reuse=reuse)
    q = H.normal_bf16(rng, int(qo_indptr[-1]) * qh * 128)
    k = H.normal_bf16(rng, pool * 16 * kvh * 128)
    v = H.normal_bf16(rng, pool * 16 * kvh * 128)
    return q, k, v, qo_indptr, indptr, indices, last


@pytest.mark.parametrize("qh,kvh", [(8, 8), (16, 4), (32, 8), (8, 1), (32, 1), (12, 4), (40, 8)])
@pytest.mark.parametrize("q_tiles", [0, 1, 4, 8])
def test_ragged_requests(provider, oracle, qh, kvh, q_tiles):
    """Mixed chunk shapes: a whole prompt, an append of a few tokens to a long KV, one token, a
    chunk that ends on a page boundary, query as long as the KV."""
    rng = np.random.default_rng(qh * 100 + kvh + q_tiles)
    qo_lens = [70, 3, 1, 32, 17, 129]
    kv_lens = [70, 300, 45, 64, 17, 257]
    pool = 80
    case = ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool)
    dims = (len(qo_lens), sum(qo_lens), pool, qh, kvh)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=8)
    actual, actual_lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case,
                                    q_tiles=q_tiles).run()
    check(actual, actual_lse, expected, expected_lse, gate=False)


def test_many_requests_span_several_scan_windows(provider, oracle):
    """More than 32 requests: the owner of a row tile is found across prefix-scan windows."""
    rng = np.random.default_rng(77)
    qo_lens = [int(n) for n in rng.integers(1, 9, size=75)]
    kv_lens = [q + int(n) for q, n in zip(qo_lens, rng.integers(0, 40, size=75))]
    pool = 300
    case = ragged_case(rng, qo_lens, kv_lens, 16, 4, pool)
    dims = (75, sum(qo_lens), pool, 16, 4)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=8)
    for q_tiles in (1, 2):
        actual, actual_lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case,
                                        q_tiles=q_tiles).run()
        check(actual, actual_lse, expected, expected_lse, gate=False)


def test_one_token_per_request_matches_paged_decode(provider, oracle):
    """qo_len == 1: the operator is paged decode; both device paths are checked against the same
    oracle output and against each other."""
    rng = np.random.default_rng(9)
    kv_lens = [500, 16, 33, 1, 1000]
    case = ragged_case(rng, [1] * 5, kv_lens, 32, 8, 140)
    q, k, v, qo_indptr, indptr, indices, last = case
    dims = (5, 5, 140, 32, 8)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=8)
    actual, actual_lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case).run()
    check(actual, actual_lse, expected, expected_lse, gate=False)
    decoded, decoded_lse = H.DecodeRun(lk.Bf16PagedBatchDecodeSpec.new(5, 140, 32, 8), q, k, v,
                                       indptr, indices, last, partitions=1).run()
    check(decoded, decoded_lse, expected, expected_lse, gate=False)
    assert np.abs(H.bits_to_f32(actual) - H.bits_to_f32(decoded)).max() <= 2.0 ** -6


def test_chunked_prefill_equals_one_shot(provider, oracle):
    """Size-independent property: prefilling a prompt in two chunks over the same pages gives,
    row for row, the one-shot result (the second chunk's mask is bottom-right aligned)."""
    rng = np.random.default_rng(21)
    total, first = 1500, 900
    qh, kvh, pool = 16, 4, 100
    indptr, indices, last = H.make_page_table(rng, [total], pool)
    q = H.normal_bf16(rng, total * qh * 128)
    k = H.normal_bf16(rng, pool * 16 * kvh * 128)
    v = H.normal_bf16(rng, pool * 16 * kvh * 128)
    whole = lk.Bf16PagedPrefillSpec.new(1, total, pool, qh, kvh)
    # the same tile shape for all three calls: the page-to-warp assignment, and with it the
    # order in which a row's partial states are merged, depends on it
    one_shot, one_lse = PrefillRun(provider, whole, q, k, v, [0, total], indptr, indices, last,
                                   q_tiles=4).run()
    # chunk 1: the first 900 tokens over the first 900 KV tokens
    pages1 = (first + 15) // 16
    out1, lse1 = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(1, first, pool, qh, kvh),
                            q[:first * qh * 128], k, v, [0, first], [0, pages1],
                            indices[:pages1], [(first - 1) % 16 + 1], q_tiles=4).run()
    # chunk 2: the remaining 600 queries over all 1500 KV tokens
    out2, lse2 = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(1, total - first, pool, qh, kvh),
                            q[first * qh * 128:], k, v, [0, total - first], indptr, indices,
                            last, q_tiles=4).run()
    assert np.array_equal(np.concatenate([out1, out2]), one_shot)
    assert np.array_equal(np.concatenate([lse1, lse2]).view(np.uint32), one_lse.view(np.uint32))
    # and a sample of rows against the oracle (the whole prompt would take the CPU minutes)
    rows = [0, 1, 15, 16, 899, 900, 1499]
    spec_rows = oracle.prefill_spec(len(rows), len(rows), pool, qh, kvh)
    q_rows = np.concatenate([q[r * qh * 128:(r + 1) * qh * 128] for r in rows])
    row_pages = [(r + 16) // 16 for r in rows]
    row_indptr = np.concatenate([[0], np.cumsum(row_pages)]).astype(np.int32)
    row_indices = np.concatenate([indices[:n] for n in row_pages])
    row_last = [r % 16 + 1 for r in rows]
    expected, expected_lse = oracle.paged_prefill(spec_rows, q_rows, k, v, np.arange(len(rows) + 1),
                                                  row_indptr, row_indices, row_last, threads=8)
    sample = np.concatenate([one_shot[r * qh * 128:(r + 1) * qh * 128] for r in rows])
    sample_lse = np.concatenate([one_lse[r * qh:(r + 1) * qh] for r in rows])
    check(sample, sample_lse, expected, expected_lse, gate=False)


def test_invalid_page_keeps_that_requests_sentinels(provider):
    """gates/paged_prefill.rs:238-314: request 0 completes, request 1 (page index 8 of 8) keeps
    its NaN sentinels."""
    spec = lk.Bf16PagedPrefillSpec.new(2, 2, 8, 1, 1)
    zeros = np.zeros(spec.kv_pages_numel(), np.uint16)
    out, lse = PrefillRun(provider, spec, np.zeros(spec.query_numel(), np.uint16), zeros, zeros,
                          [0, 1, 2], [0, 1, 2], [0, 8], [1, 1]).run()
    assert np.all(out[:128] == 0) and lse[0] == 0.0
    assert np.all(np.isnan(H.bits_to_f32(out[128:]))) and np.isnan(lse[1])


def test_invalid_page_past_the_causal_limit_still_guards_the_request(provider):
    """The reference validates every page of a request before any row of it is computed
    (prefill.rs:333-340): an out-of-range id in the last page silences the early rows too."""
    rng = np.random.default_rng(4)
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, [40, 8], [64, 24], 8, 2, 16)
    indices = indices.copy()
    indices[3] = 99  # the last page of request 0; rows 0..23 never reach it
    out, lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(2, 48, 16, 8, 2), q, k, v,
                          qo_indptr, indptr, indices, last, q_tiles=1).run()
    assert np.all(np.isnan(H.bits_to_f32(out[:40 * 8 * 128]))) and np.all(np.isnan(lse[:40 * 8]))
    assert np.all(np.isfinite(H.bits_to_f32(out[40 * 8 * 128:]))) and np.all(np.isfinite(lse[40 * 8:]))


@pytest.mark.parametrize("field,values,written_requests", [
    ("qo_indptr", [0, 10, 10, 48], [0]),      # request 1 is empty: rows of requests 1.. are guarded
    ("qo_indptr", [1, 10, 40, 48], []),       # the global checks fail for every row
    ("qo_indptr", [0, 10, 40, 47], []),
    ("page_indptr", [0, 4, 7, 8], []),        # page_indptr[batch] != len(page_indices)
    ("last", [16, 0, 8], [0, 2]),             # only request 1 is rejected
    ("last", [16, 17, 8], [0, 2])])
def test_device_guard_on_dynamic_metadata(provider, field, values, written_requests):
    """prefill.rs:289-347: malformed device-resident metadata is not an error; rows the guard
    rejects keep their sentinels and nothing is read out of bounds."""
    rng = np.random.default_rng(6)
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, [10, 30, 8], [64, 40, 24], 8, 2,
                                                            16)
    meta = dict(qo_indptr=qo_indptr, page_indptr=indptr, last=last)
    meta[field] = np.asarray(values, np.int32)
    out, lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(3, 48, 16, 8, 2), q, k, v,
                          meta["qo_indptr"], meta["page_indptr"], indices, meta["last"]).run()
    written = np.isfinite(lse.reshape(48, 8)).all(axis=1)
    expected = np.zeros(48, bool)
    for request in written_requests:
        expected[qo_indptr[request]:qo_indptr[request + 1]] = True
    assert np.array_equal(written, expected)
    assert np.array_equal(np.isfinite(H.bits_to_f32(out)).reshape(48, -1).all(axis=1), expected)


def test_query_longer_than_kv_is_guarded(provider):
    rng = np.random.default_rng(8)
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, [40, 8], [64, 24], 8, 2, 16)
    out, lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(2, 48, 16, 8, 2), q, k, v,
                          qo_indptr, [0, 4, 5], indices[:5], [16, 7]).run()
    written = np.isfinite(lse.reshape(48, 8)).all(axis=1)
    assert written[:40].all() and not written[40:].any()  # request 1: 8 queries over 7 tokens


def test_fixed_address_graph_replays(provider, oracle):
    """gates/paged_prefill.rs:382-526: one checked command captured on a private stream and
    replayed twice after the plan and provider references are dropped."""
    dims, qo_indptr, indptr, indices, last, salt = GATE_CASES["gqa4_reordered_reuse"]
    spec = lk.Bf16PagedPrefillSpec.new(*dims)
    q = oracle.fixture_bf16(spec.query_numel(), salt)
    k = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ K_SALT)
    v = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ V_SALT)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), q, k, v, qo_indptr,
                                                  indptr, indices, last)
    plan = lk.PrefillProvider.load(0).plan_bf16_paged(spec)
    tensors = [H.dev_bf16(t) for t in (q, k, v)] + [H.dev_i32(a) for a in
                                                    (qo_indptr, indptr, indices, last)]
    out = torch.full((spec.output_numel(),), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    lse = torch.full((spec.lse_numel(),), float("nan"), dtype=torch.float32, device="cuda:0")
    torch.cuda.synchronize()
    graph_queue = lk.GraphQueue(0, 1)
    b = graph_queue.bindings(9)
    reads = [b.bind_read(t) for t in tensors]
    h_out, h_lse = b.bind_read_write(out), b.bind_read_write(lse)
    captured = graph_queue.capture(b, lambda scope: plan.enqueue_into(
        scope, lk.Bf16PagedPrefillArgs(*reads, h_out.write(), h_lse.write())))
    assert captured.commands() == 1
    exec_ = captured.instantiate()
    del plan
    for replay in range(2):
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        exec_.launch().wait()
        check(H.host_bits(out), lse.cpu().numpy(), expected, expected_lse)
    assert exec_.launches() == 2
    exec_.into_bindings()
