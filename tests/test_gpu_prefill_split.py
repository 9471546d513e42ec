"""GPU parity of the tiled paged-prefill kernel with the KV range of every tile shared out to
several CTAs (plans with partitions > 1: chunk states in a workspace, then the LSE merge of the
split-K contract), against the CPU oracle, through the C ABI.  The cases are those of
tests/test_gpu_prefill_tiled.py -- gate shapes, ragged batches, a moving exponent base, chunks
after a long cache, the device guards, Graph replay -- plus chunk counts that leave CTAs without
a block."""
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
@pytest.mark.parametrize("partitions", [2, 5])
def test_reference_gate_cases(provider, oracle, name, partitions):
    """Short KV ranges: most chunks get no block and publish an empty state."""
    dims, qo_indptr, indptr, indices, last, salt = GATE_CASES[name]
    spec = lk.Bf16PagedPrefillSpec.new(*dims)
    q = oracle.fixture_bf16(spec.query_numel(), salt)
    k = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ K_SALT)
    v = oracle.fixture_bf16(spec.kv_pages_numel(), salt ^ V_SALT)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), q, k, v, qo_indptr,
                                                  indptr, indices, last)
    run = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last, algorithm=TILED,
                     partitions=partitions)
    assert run.plan.algorithm() == lk.Bf16PagedPrefillAlgorithm.Tiled
    assert (run.plan.partitions(), run.plan.commands()) == (partitions, 2)
    actual, actual_lse = run.run()
    check(actual, actual_lse, expected, expected_lse)


@pytest.mark.parametrize("qh,kvh", [(8, 8), (32, 8), (8, 1), (12, 4)])
@pytest.mark.parametrize("partitions", [2, 3, 7])
def test_ragged_requests(provider, oracle, qh, kvh, partitions):
    rng = np.random.default_rng(qh * 100 + kvh + partitions)
    qo_lens = [70, 3, 1, 32, 17, 129, 60]
    kv_lens = [70, 300, 45, 64, 17, 257, 700]
    pool = 130
    case = ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool)
    dims = (len(qo_lens), sum(qo_lens), pool, qh, kvh)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=8)
    actual, actual_lse = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case,
                                    algorithm=TILED, partitions=partitions).run()
    check(actual, actual_lse, expected, expected_lse, gate=False)


def test_chunk_states_follow_the_split_k_contract(provider, oracle):
    """The workspace holds, per (query row, head, chunk), [max_log2, normaliser, weighted V] of the
    chunk's 64-token blocks (the balanced rule over blocks): merging them on the host with the
    oracle's split-K merge reproduces O and LSE, and rows that see nothing of a chunk hold the
    empty state."""
    rng = np.random.default_rng(77)
    qh, kvh, pool, partitions = 8, 2, 70, 3
    qo_lens, kv_lens = [40], [1000]
    case = ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool)
    dims = (1, 40, pool, qh, kvh)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=8)
    run = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case, algorithm=TILED,
                     partitions=partitions)
    actual, actual_lse = run.run()
    check(actual, actual_lse, expected, expected_lse, gate=False)
    states = run.workspace.cpu().numpy().reshape(40 * qh, partitions, 130)
    assert np.isfinite(states).all()
    # 40 rows x group 4 = 160 packed rows per KV head: tile 0 holds tokens 0..31, which see
    # 961..992 tokens = 16 blocks (6 + 5 + 5); tile 1 holds tokens 32..39 (1000 tokens, 16 blocks)
    assert (states[:, :, 1] > 0).all()
    merged, merged_lse = oracle.split_k_merge(40 * qh, partitions, states.reshape(-1))
    check(merged, merged_lse, expected, expected_lse, gate=False)


def test_rows_before_a_chunk_publish_empty_states(provider, oracle):
    """A whole prompt: early rows of a tile end before later chunks begin, and a tile with fewer
    blocks than the plan has chunks uses as many chunks as it has blocks (the other CTAs leave
    the workspace alone)."""
    rng = np.random.default_rng(78)
    qh, kvh, pool, partitions = 4, 4, 40, 4
    case = ragged_case(rng, [600], [600], qh, kvh, pool)
    dims = (1, 600, pool, qh, kvh)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=8)
    run = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case, algorithm=TILED,
                     partitions=partitions)
    actual, actual_lse = run.run()
    check(actual, actual_lse, expected, expected_lse, gate=False)
    states = run.workspace.cpu().numpy().reshape(600, qh, partitions, 130)
    # tile 0 (tokens 0..127, one head per KV head) sees at most 128 keys = 2 blocks = 2 chunks
    assert np.isfinite(states[:128, :, :2]).all() and np.isnan(states[:128, :, 2:]).all()
    # token 0 sees one key: only the first chunk has a state, the second is empty
    assert (states[0, :, 0, 1] > 0).all() and (states[0, :, 1, :2] == 0).all()
    # the last token of the tile sees 128 keys: chunks 0 and 1 hold one block each
    assert (states[127, :, :2, 1] > 0).all()
    # the last tile (tokens 512..599) sees 600 keys = 10 blocks: all four chunks
    assert np.isfinite(states[512:]).all() and (states[599, :, :, 1] > 0).all()


def test_long_rows_with_a_rising_maximum(provider, oracle):
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
    for partitions in (4, 2):
        run = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), q, k, v, qo_indptr, indptr,
                         indices, last, algorithm=TILED, partitions=partitions)
        assert run.plan.partitions() == partitions
        actual, actual_lse = run.run()
        check(actual, actual_lse, expected, expected_lse, gate=False)


@pytest.mark.parametrize("partitions", [0, 5, 16, 64])
def test_chunk_after_a_long_cache(provider, oracle, partitions):
    """Chunked prefill at serving shape -- the case the split exists for: the plan-time heuristic
    picks several chunks, and any count gives the oracle's result."""
    rng = np.random.default_rng(51)
    qo_lens, kv_lens = [130, 40], [5000, 2177]
    qh, kvh, pool = 16, 4, 460
    case = ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool)
    dims = (2, sum(qo_lens), pool, qh, kvh)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=16)
    run = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case, algorithm=TILED,
                     partitions=partitions)
    assert run.plan.partitions() == (partitions or 3) and run.plan.commands() == 2
    actual, actual_lse = run.run()
    check(actual, actual_lse, expected, expected_lse, gate=False)


def test_guards(provider):
    """As for the unsplit kernel: rejected rows keep their sentinels, whichever chunk meets the
    defect; a bad page id poisons the chunk that streams it and the merge publishes nothing."""
    spec = lk.Bf16PagedPrefillSpec.new(2, 2, 8, 1, 1)
    zeros = np.zeros(spec.kv_pages_numel(), np.uint16)
    out, lse = PrefillRun(provider, spec, np.zeros(spec.query_numel(), np.uint16), zeros, zeros,
                          [0, 1, 2], [0, 1, 2], [0, 8], [1, 1], algorithm=TILED,
                          partitions=2).run()
    assert np.all(out[:128] == 0) and lse[0] == 0.0
    assert np.all(np.isnan(H.bits_to_f32(out[128:]))) and np.isnan(lse[1])

    rng = np.random.default_rng(4)
    kv_lens = [640, 400, 240]
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, [10, 30, 8], kv_lens, 8, 2, 90)
    spec = lk.Bf16PagedPrefillSpec.new(3, 48, 90, 8, 2)

    def written(**override):
        meta = dict(qo_indptr=qo_indptr, indptr=indptr, indices=indices, last=last)
        meta.update({name: np.asarray(value, np.int32) for name, value in override.items()})
        out, lse = PrefillRun(provider, spec, q, k, v, meta["qo_indptr"], meta["indptr"],
                              meta["indices"], meta["last"], algorithm=TILED, partitions=3).run()
        rows = np.isfinite(lse.reshape(48, 8)).all(axis=1)
        assert np.array_equal(np.isfinite(H.bits_to_f32(out)).reshape(48, -1).all(axis=1), rows)
        return [bool(rows[a:b].all()) for a, b in ((0, 10), (10, 40), (40, 48))], bool(rows.any())

    assert written() == ([True, True, True], True)
    for position in (0, 17, 39):  # a page of request 0 in the first, second and third chunk
        bad = indices.copy()
        bad[position] = 99
        assert written(indices=bad)[0] == [False, True, True]
    bad = indices.copy()
    bad[int(indptr[2]) - 1] = -1  # the last page of request 1
    assert written(indices=bad)[0] == [True, False, True]
    assert written(qo_indptr=[0, 10, 10, 48])[0] == [True, False, False]
    assert written(qo_indptr=[1, 10, 40, 48])[1] is False
    assert written(indptr=[0, 40, 65, 79])[1] is False
    assert written(last=[16, 0, 16])[0] == [True, False, True]
    short = np.asarray(indptr).copy()
    short[2:] -= 24  # request 1: 30 queries over one page with 8 tokens
    assert written(indptr=short, indices=np.concatenate([indices[:41], indices[65:]]),
                   last=[16, 8, 16])[0] == [True, False, True]


def test_fixed_address_graph_replays(provider, oracle):
    rng = np.random.default_rng(52)
    qh, kvh, pool = 8, 2, 70
    case = ragged_case(rng, [33, 5], [700, 300], qh, kvh, pool)
    dims = (2, 38, pool, qh, kvh)
    spec = lk.Bf16PagedPrefillSpec.new(*dims)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=8)
    plan = provider.plan_bf16_paged(spec, algorithm=TILED, partitions=4)
    tensors = [H.dev_bf16(t) for t in case[:3]] + [H.dev_i32(a) for a in case[3:]]
    out = torch.full((spec.output_numel(),), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    lse = torch.full((spec.lse_numel(),), float("nan"), dtype=torch.float32, device="cuda:0")
    workspace = torch.full((plan.workspace_required_numel(),), float("nan"), dtype=torch.float32,
                           device="cuda:0")
    torch.cuda.synchronize()
    graph_queue = lk.GraphQueue(0, 2)
    b = graph_queue.bindings(10)
    reads = [b.bind_read(t) for t in tensors]
    h_out, h_lse, h_ws = (b.bind_read_write(x) for x in (out, lse, workspace))
    exec_ = graph_queue.capture(b, lambda scope: plan.enqueue_into(
        scope, lk.Bf16PagedPrefillArgs(*reads, h_out.write(), h_lse.write(), h_ws))).instantiate()
    for replay in range(3):
        out.fill_(float("nan"))
        workspace.fill_(float("nan"))
        torch.cuda.synchronize()
        exec_.launch().wait()
        check(H.host_bits(out), lse.cpu().numpy(), expected, expected_lse, gate=False)
    assert provider.device_status() == 0
    exec_.into_bindings()


def test_many_requests_span_several_scan_windows(provider, oracle):
    """More than 32 requests: the main kernel finds the owner of a tile and the merge kernel the
    owner of a row across prefix-scan windows; a malformed query range in the third window stops
    every request from there on, and only those."""
    rng = np.random.default_rng(79)
    qo_lens = [int(n) for n in rng.integers(1, 40, size=75)]
    kv_lens = [q + int(n) for q, n in zip(qo_lens, rng.integers(0, 300, size=75))]
    pool = 900
    case = ragged_case(rng, qo_lens, kv_lens, 16, 4, pool)
    q, k, v, qo_indptr, indptr, indices, last = case
    nnz = sum(qo_lens)
    dims = (75, nnz, pool, 16, 4)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=8)
    spec = lk.Bf16PagedPrefillSpec.new(*dims)
    for partitions in (2, 3):
        actual, actual_lse = PrefillRun(provider, spec, *case, algorithm=TILED,
                                        partitions=partitions).run()
        check(actual, actual_lse, expected, expected_lse, gate=False)
    broken = np.asarray(qo_indptr).copy()
    broken[70] = broken[69]  # request 69 is empty: it and every later request are rejected
    out, lse = PrefillRun(provider, spec, q, k, v, broken, indptr, indices, last, algorithm=TILED,
                          partitions=2).run()
    written = np.isfinite(lse.reshape(nnz, 16)).all(axis=1)
    assert written[:broken[69]].all() and not written[broken[69]:].any()
    check(out[:broken[69] * 16 * 128], lse[:broken[69] * 16], expected[:broken[69] * 16 * 128],
          expected_lse[:broken[69] * 16], gate=False)


def test_split_and_unsplit_plans_agree_on_a_long_chunk(provider, oracle):
    """Size-independent property at a serving size the CPU oracle cannot cover in a test: 256 new
    tokens behind 12 000 cached ones give the same rows whether a tile has one CTA or nine, and
    sampled rows agree with the oracle."""
    rng = np.random.default_rng(83)
    chunk, total, qh, kvh, pool = 256, 12256, 16, 4, 800
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, [chunk], [total], qh, kvh, pool)
    spec = lk.Bf16PagedPrefillSpec.new(1, chunk, pool, qh, kvh)
    whole, whole_lse = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last,
                                  algorithm=TILED, partitions=1).run()
    auto = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last, algorithm=0,
                      partitions=0)
    assert auto.plan.algorithm() == lk.Bf16PagedPrefillAlgorithm.Tiled
    assert auto.plan.partitions() == 9  # 32 whole tiles for 296 slots
    shared, shared_lse = auto.run()
    check(shared, shared_lse, whole, whole_lse, gate=False)
    rows = [0, 1, 100, 255]
    spec_rows = oracle.prefill_spec(len(rows), len(rows), pool, qh, kvh)
    q_rows = np.concatenate([q[r * qh * 128:(r + 1) * qh * 128] for r in rows])
    seen = [total - chunk + r + 1 for r in rows]
    row_pages = [(n + 15) // 16 for n in seen]
    expected, expected_lse = oracle.paged_prefill(
        spec_rows, q_rows, k, v, np.arange(len(rows) + 1),
        np.concatenate([[0], np.cumsum(row_pages)]).astype(np.int32),
        np.concatenate([indices[:n] for n in row_pages]), [(n - 1) % 16 + 1 for n in seen],
        threads=16)
    sample = np.concatenate([shared[r * qh * 128:(r + 1) * qh * 128] for r in rows])
    sample_lse = np.concatenate([shared_lse[r * qh:(r + 1) * qh] for r in rows])
    check(sample, sample_lse, expected, expected_lse, gate=False)


def test_plan_chosen_chunks_follow_the_kv_length_met(provider, oracle):
    """A plan cannot know the KV lengths (an engine's pool is its whole cache): the count it
    chooses is an upper bound, and on the device a tile takes one chunk per sixteen 64-token
    blocks it really has.  Short requests are finished by the first command alone -- their
    states are never written -- long ones are shared out, in one call."""
    rng = np.random.default_rng(91)
    qh, kvh, pool = 16, 4, 4000
    qo_lens, kv_lens = [64, 96, 32], [2500, 3900, 64]
    case = ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool)
    dims = (3, sum(qo_lens), pool, qh, kvh)
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), *case, threads=16)
    run = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case, algorithm=0, partitions=0)
    info = run.plan.info()
    assert run.plan.algorithm() == lk.Bf16PagedPrefillAlgorithm.Tiled
    assert (info.partitions, info.min_chunk_blocks, info.commands) == (12, 16, 2)
    actual, actual_lse = run.run()
    check(actual, actual_lse, expected, expected_lse, gate=False)
    states = run.workspace.cpu().numpy().reshape(sum(qo_lens), qh, 12, 130)
    # 2500 keys = 40 blocks (two chunks of sixteen do not pay) and 64 keys = 1 block: one chunk,
    # no state; 3900 keys = 61 blocks: 3
    assert np.isnan(states[:64]).all() and np.isnan(states[160:]).all()
    assert np.isfinite(states[64:160, :, :3]).all() and np.isnan(states[64:160, :, 3:]).all()
    forced = PrefillRun(provider, lk.Bf16PagedPrefillSpec.new(*dims), *case, algorithm=TILED,
                        partitions=16)
    assert forced.plan.info().min_chunk_blocks == 1
    actual, actual_lse = forced.run()
    check(actual, actual_lse, expected, expected_lse, gate=False)
