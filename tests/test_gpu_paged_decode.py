"""GPU parity of the paged decode path against the CPU oracle, through the C ABI.

Gate cases follow crates/loom-infer-validation/src/gates/paged_batch_decode.rs:316-363 and the
split-K cases crates/loom-infer-validation/src/gates/single_decode.rs:416-580 of the reference.
"""
import json
import os

import numpy as np
import pytest

import loom_kernels_b200 as lk
from tests import helpers as H

pytestmark = pytest.mark.gpu
GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_digests.json")))
K_SALT, V_SALT = 0x4B455900, 0x56414C554500


@pytest.fixture(scope="module")
def provider():
    return lk.DecodeProvider.load(0)


def fixture_case(oracle, case):
    batch, pages, qh, kvh = case["spec"]
    salt = int(case["salt"], 16)
    q = oracle.fixture_bf16(batch * qh * 128, salt)
    k = oracle.fixture_bf16(pages * 16 * kvh * 128, salt ^ K_SALT)
    v = oracle.fixture_bf16(pages * 16 * kvh * 128, salt ^ V_SALT)
    return q, k, v


@pytest.mark.parametrize("name", ["mha_b1_l1", "mqa_b3_mixed", "gqa4_b4_reuse"])
@pytest.mark.parametrize("partitions,merge_in_kernel", [(1, 0), (2, 0), (3, 0), (2, 1), (3, 1)])
def test_reference_gate_cases(oracle, provider, name, partitions, merge_in_kernel):
    # split plans in both forms: merged by a second command (the reference's form) and by the
    # last CTA of an item (merge_in_kernel=1, one command)
    case = GOLDEN["paged_decode"]["cases"][name]
    batch, pages, qh, kvh = case["spec"]
    if partitions > pages:
        pytest.skip("more partitions than pages in the pool")
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pages, qh, kvh)
    q, k, v = fixture_case(oracle, case)
    run = H.DecodeRun(spec, q, k, v, case["indptr"], case["indices"], case["last"],
                      partitions=partitions, provider=provider, merge_in_kernel=merge_in_kernel)
    out, lse = run.run()
    assert run.submitted == (2 if partitions > 1 and merge_in_kernel != 1 else 1)
    if partitions == 1:  # and once more through the heuristic's choice for this shape
        auto = H.DecodeRun(spec, q, k, v, case["indptr"], case["indices"], case["last"],
                           provider=provider)
        out2, lse2 = auto.run()
        eo2, el2 = oracle.paged_decode(oracle.paged_spec(batch, pages, qh, kvh), q, k, v,
                                       case["indptr"], case["indices"], case["last"])
        H.check_decode(out2, lse2, eo2, el2, lse_limit=H.SPLIT_LSE_MAX_ABS, gate=True)
    ospec = oracle.paged_spec(batch, pages, qh, kvh)
    eo, el = oracle.paged_decode(ospec, q, k, v, case["indptr"], case["indices"], case["last"])
    assert f"{oracle.digest_bf16(eo):016x}" == case["output"]  # the checker is the pinned one
    H.check_decode(out, lse, eo, el, lse_limit=H.SPLIT_LSE_MAX_ABS, gate=True)


def test_short_metadata_is_rejected_before_submission(oracle, provider):
    # gates/paged_batch_decode.rs:150-222
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 8, 16, 4)
    case = GOLDEN["paged_decode"]["cases"]["gqa4_b4_reuse"]
    q, k, v = fixture_case(oracle, case)
    run = H.DecodeRun(spec, q, k, v, case["indptr"][:-1], case["indices"], case["last"],
                      provider=provider)
    scope = run.queue.begin(run.bind())
    with pytest.raises(lk.EnqueueError) as info:
        run.plan.enqueue_into(scope, run.args())
    assert (info.value.variant, info.value.operand) == ("LengthMismatch", "page_indptr")
    assert info.value.payload[:2] == (5, 4)
    completion = scope.finish()
    assert completion.submitted() == 0
    bindings = completion.wait()
    out = H.host_bits(bindings.take_read_write(run.h_out))
    assert np.all(np.isnan(H.bits_to_f32(out)))


def test_invalid_page_guard_keeps_sentinels(provider):
    # gates/paged_batch_decode.rs:224-308: request 1 names page 2 of a 2-page pool
    spec = lk.Bf16PagedBatchDecodeSpec.new(2, 2, 4, 2)
    zeros = np.zeros(spec.kv_pages_numel(), np.uint16)
    run = H.DecodeRun(spec, np.zeros(spec.query_numel(), np.uint16), zeros, zeros, [0, 1, 2],
                      [0, 2], [16, 16], provider=provider)
    out, lse = run.run()
    o = H.bits_to_f32(out).reshape(2, -1)
    assert np.all(o[0] == 0.0) and np.all(lse[:4] == 4.0)
    assert np.all(np.isnan(o[1])) and np.all(np.isnan(lse[4:]))
    # the same guard holds when the request is split: the merge must not publish it
    run = H.DecodeRun(spec, np.zeros(spec.query_numel(), np.uint16), zeros, zeros, [0, 1, 2],
                      [0, 2], [16, 16], partitions=2, provider=provider)
    out, lse = run.run()
    o = H.bits_to_f32(out).reshape(2, -1)
    assert np.all(o[0] == 0.0) and np.all(lse[:4] == 4.0)
    assert np.all(np.isnan(o[1])) and np.all(np.isnan(lse[4:]))


def test_invalid_request_metadata_guard(provider):
    # decode.rs:238-248: a zero last_page_len skips that request only
    spec = lk.Bf16PagedBatchDecodeSpec.new(2, 4, 4, 2)
    rng = np.random.default_rng(3)
    k, v = H.normal_bf16(rng, spec.kv_pages_numel()), H.normal_bf16(rng, spec.kv_pages_numel())
    q = H.normal_bf16(rng, spec.query_numel())
    run = H.DecodeRun(spec, q, k, v, [0, 2, 4], [0, 1, 2, 3], [0, 5], provider=provider)
    out, lse = run.run()
    o = H.bits_to_f32(out).reshape(2, -1)
    assert np.all(np.isnan(o[0])) and np.all(np.isfinite(o[1]))


SHAPES = [
    # (batch, qh, kvh, heads_per_cta, partitions)
    (3, 8, 8, 0, 1), (3, 8, 8, 8, 1), (2, 8, 8, 2, 2),
    (3, 8, 1, 0, 1), (5, 16, 4, 4, 1), (5, 16, 4, 2, 1), (5, 16, 4, 1, 3),
    (4, 32, 8, 8, 1), (4, 32, 8, 1, 1), (2, 64, 8, 4, 4), (2, 64, 8, 0, 16),
    (3, 32, 1, 0, 1), (3, 32, 1, 1, 5), (2, 12, 3, 0, 1), (2, 6, 6, 2, 2),
    (2, 40, 1, 0, 1), (1, 72, 1, 0, 2), (2, 160, 1, 0, 1), (1, 4, 2, 1, 1),
    # more than 8 KV heads: several head blocks per request (MHA 32/32, 16/16, GQA4 64/16)
    (1, 32, 32, 0, 0), (1, 32, 32, 4, 3), (2, 16, 16, 0, 1), (2, 16, 16, 2, 2), (3, 64, 16, 0, 1),
    (3, 64, 16, 8, 4),
]


@pytest.mark.parametrize("batch,qh,kvh,hc,partitions", SHAPES)
def test_random_ragged_batches(oracle, provider, batch, qh, kvh, hc, partitions):
    ragged_case(oracle, provider, batch, qh, kvh, hc, partitions, balanced=2)


@pytest.mark.parametrize("batch,qh,kvh,hc,partitions", [s for s in SHAPES if s[4] > 1])
def test_random_ragged_batches_split_merged_in_kernel(oracle, provider, batch, qh, kvh, hc,
                                                      partitions):
    ragged_case(oracle, provider, batch, qh, kvh, hc, partitions, balanced=2, merge_in_kernel=1)


@pytest.mark.parametrize("merge_in_kernel", [1, 2])
@pytest.mark.parametrize("batch,qh,kvh,hc,partitions", SHAPES)
def test_random_ragged_batches_balanced(oracle, provider, batch, qh, kvh, hc, partitions,
                                        merge_in_kernel):
    # the same batches through the page-balanced algorithm (pages cut evenly over the SMs), the
    # cut items merged in the decode kernel (1) or by the merge kernel (2)
    ragged_case(oracle, provider, batch, qh, kvh, hc, 0, balanced=1,
                merge_in_kernel=merge_in_kernel)


@pytest.mark.parametrize("options", [dict(producer_warps=1), dict(producer_warps=4),
                                     dict(max_stages=3), dict(producer_warps=4, max_stages=2)])
def test_balanced_producer_and_ring_options(oracle, provider, options):
    # one KV head per CTA (4 KB boxes): one producer warp for all four page slots or one per slot,
    # and a ring capped below what shared memory allows, give the same results
    ragged_case(oracle, provider, 3, 32, 1, 0, 0, balanced=1, merge_in_kernel=2, **options)
    info = provider.plan_bf16_paged_batch(lk.Bf16PagedBatchDecodeSpec.new(3, 96, 32, 1),
                                          balanced=1, **options).info()
    assert info.block == (8 + options.get("producer_warps", 4)) * 32
    if "max_stages" in options:
        assert info.stages == options["max_stages"]
    with pytest.raises(lk.PlanError):  # neither 1 nor the plan's page slots per stage
        provider.plan_bf16_paged_batch(lk.Bf16PagedBatchDecodeSpec.new(3, 96, 32, 1), balanced=1,
                                       producer_warps=3)


def ragged_case(oracle, provider, batch, qh, kvh, hc, partitions, balanced, merge_in_kernel=0,
                **plan_options):
    rng = np.random.default_rng(batch * 1000 + qh * 10 + kvh + hc + partitions)
    pool = 96
    kv_lens = rng.integers(1, 16 * 18, size=batch)
    kv_lens[0] = 16 * 17 + 1  # a lone token on the last page
    if batch > 1:
        kv_lens[1] = 5
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool)
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pool, qh, kvh)
    # pool rows past each request's length are NaN: they must never reach the output
    k = H.normal_bf16(rng, spec.kv_pages_numel())
    v = H.normal_bf16(rng, spec.kv_pages_numel())
    kr, vr = k.reshape(pool, 16, -1), v.reshape(pool, 16, -1)
    for r in range(batch):
        page = indices[indptr[r + 1] - 1]
        kr[page, last[r]:] = 0x7FC0
        vr[page, last[r]:] = 0x7FC0
    q = H.normal_bf16(rng, spec.query_numel())
    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, partitions=partitions,
                      heads_per_cta=hc, provider=provider, balanced=balanced,
                      merge_in_kernel=merge_in_kernel, **plan_options)
    if balanced == 1:
        assert run.plan.algorithm() == lk.Bf16PagedBatchDecodeAlgorithm.Balanced
    if partitions > 1 or balanced == 1:
        assert run.plan.merged_in_kernel() == (merge_in_kernel == 1)
        assert run.plan.commands() == (1 if merge_in_kernel == 1 else 2)
    out, lse = run.run()
    assert run.submitted == run.plan.commands()
    if run.plan.merged_in_kernel():
        # the items' counting words are back at zero: the same queue serves the next call, with
        # the output reset in between so that stale rows cannot pass
        run.out.fill_(float("nan"))
        again_out, again_lse = run.run()
        assert np.array_equal(again_out, out) and np.array_equal(again_lse, lse)
    ospec = oracle.paged_spec(batch, pool, qh, kvh)
    eo, el = oracle.paged_decode(ospec, q, k, v, indptr, indices, last, threads=4)
    H.check_decode(out, lse, eo, el, lse_limit=H.SPLIT_LSE_MAX_ABS)


CLUSTER_SHAPES = [
    # (batch, qh, kvh, heads_per_cta, partitions): the chunks of a request form one cluster
    (1, 32, 32, 4, 8), (1, 32, 32, 0, 0), (1, 8, 8, 0, 2), (2, 16, 4, 2, 3), (3, 32, 8, 4, 5),
    (2, 32, 1, 0, 4), (1, 64, 2, 0, 8), (2, 24, 1, 0, 2), (4, 12, 3, 1, 7),
]


@pytest.mark.parametrize("batch,qh,kvh,hc,partitions", CLUSTER_SHAPES)
def test_cluster_split_is_one_command(oracle, provider, batch, qh, kvh, hc, partitions):
    """Split-K whose chunk states are merged inside a thread-block cluster: one command, no
    workspace, the results of the two-command split (requests shorter than the chunk count leave
    chunks without pages)."""
    rng = np.random.default_rng(batch * 77 + qh + kvh + partitions)
    pool = 256 if batch == 1 else 96
    kv_lens = rng.integers(1, 16 * 18, size=batch)
    kv_lens[0] = 16 * 64 if batch == 1 else 16 * 17 + 1
    if batch > 1:
        kv_lens[1] = 5  # one page: every chunk but the first is empty
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool)
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pool, qh, kvh)
    q, k, v = (H.normal_bf16(rng, n) for n in (spec.query_numel(), spec.kv_pages_numel(),
                                               spec.kv_pages_numel()))
    options = dict(partitions=partitions, heads_per_cta=hc, cluster=True) if partitions else {}
    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, provider=provider, **options)
    assert run.plan.algorithm() == lk.Bf16PagedBatchDecodeAlgorithm.ClusterSplit
    assert run.plan.commands() == 1 and run.plan.workspace_required_numel() == 0
    out, lse = run.run()
    assert run.submitted == 1
    eo, el = oracle.paged_decode(oracle.paged_spec(batch, pool, qh, kvh), q, k, v, indptr, indices,
                                 last, threads=4)
    H.check_decode(out, lse, eo, el, lse_limit=H.SPLIT_LSE_MAX_ABS)
    # an out-of-range page in one chunk: that request keeps its sentinels, the others do not
    if batch > 1:
        broken = indices.copy()
        broken[indptr[0] + 9] = pool
        run = H.DecodeRun(spec, q, k, v, indptr, broken, last, provider=provider, **options)
        out, lse = run.run()
        rows = H.bits_to_f32(out).reshape(batch, -1)
        assert np.all(np.isnan(rows[0])) and np.all(np.isfinite(rows[1:]))


def test_balanced_guards_keep_sentinels(provider):
    # the page-balanced algorithm keeps the reference's device guards: an out-of-range page or
    # a bad last_page_len leaves that request (and only it) unwritten
    spec = lk.Bf16PagedBatchDecodeSpec.new(2, 2, 4, 2)
    zeros = np.zeros(spec.kv_pages_numel(), np.uint16)
    run = H.DecodeRun(spec, np.zeros(spec.query_numel(), np.uint16), zeros, zeros, [0, 1, 2],
                      [0, 2], [16, 16], provider=provider, balanced=1)
    out, lse = run.run()
    o = H.bits_to_f32(out).reshape(2, -1)
    assert np.all(o[0] == 0.0) and np.all(lse[:4] == 4.0)
    assert np.all(np.isnan(o[1])) and np.all(np.isnan(lse[4:]))
    spec = lk.Bf16PagedBatchDecodeSpec.new(3, 64, 8, 2)
    rng = np.random.default_rng(8)
    k, v = H.normal_bf16(rng, spec.kv_pages_numel()), H.normal_bf16(rng, spec.kv_pages_numel())
    q = H.normal_bf16(rng, spec.query_numel())
    indptr, indices, last = H.make_page_table(rng, [300, 200, 150], 64)
    indices = indices.copy()
    indices[indptr[1] + 5] = 64  # request 1 names a page outside the pool, mid-way
    last = last.copy()
    last[2] = 17                 # request 2 has an impossible last page length
    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, provider=provider, balanced=1)
    out, lse = run.run()
    o = H.bits_to_f32(out).reshape(3, -1)
    assert np.all(np.isfinite(o[0])) and np.all(np.isnan(o[1])) and np.all(np.isnan(o[2]))
    assert np.all(np.isfinite(lse[:8])) and np.all(np.isnan(lse[8:]))


def test_split_k_states_match_the_partial_state_contract(oracle, provider):
    # workspace layout [batch, qh, partitions, 130] = [max_log2, normaliser, wv[128]]
    rng = np.random.default_rng(11)
    batch, qh, kvh, pool, partitions = 3, 16, 4, 64, 4
    kv_lens = [16 * 9 + 3, 16 * 2, 7]  # the last request leaves three chunks without pages
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool)
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pool, qh, kvh)
    q, k, v = (H.normal_bf16(rng, n) for n in (spec.query_numel(), spec.kv_pages_numel(),
                                               spec.kv_pages_numel()))
    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, partitions=partitions,
                      provider=provider)
    assert run.plan.algorithm() == lk.Bf16PagedBatchDecodeAlgorithm.SplitK
    assert run.plan.workspace_required_numel() == batch * qh * partitions * 130
    out, lse = run.run()
    ws = run.workspace.cpu().numpy().reshape(batch * qh, partitions, 130)
    ospec = oracle.paged_spec(batch, pool, qh, kvh)
    eo, el, ews = oracle.paged_split_k(ospec, partitions, q, k, v, indptr, indices, last)
    ews = ews.reshape(batch * qh, partitions, 130)
    H.check_decode(out, lse, eo, el, lse_limit=H.SPLIT_LSE_MAX_ABS)
    # empty chunks are exactly [0, 0, 0...]
    empty = ews[:, :, 1] == 0.0
    assert empty.any() and np.all(ws[empty] == 0.0)
    # a state is defined up to its running max: compare in the normalised form
    live = ~empty
    lse_state = ws[live][:, 0] + np.log2(ws[live][:, 1])
    lse_expect = ews[live][:, 0] + np.log2(ews[live][:, 1])
    assert np.abs(lse_state - lse_expect).max() <= H.SPLIT_LSE_MAX_ABS
    mean_state = ws[live][:, 2:] / ws[live][:, 1:2]
    mean_expect = ews[live][:, 2:] / ews[live][:, 1:2]
    assert np.abs(mean_state - mean_expect).max() <= H.DECODE_MAX_ABS


def test_split_k_preflight(oracle, provider):
    # gates/single_decode.rs:416-513: capacity for both commands is required before any launch,
    # and the workspace length is exact
    rng = np.random.default_rng(5)
    spec = lk.Bf16PagedBatchDecodeSpec.new(1, 8, 8, 1)
    indptr, indices, last = H.make_page_table(rng, [100], 8)
    q, k, v = (H.normal_bf16(rng, n) for n in (spec.query_numel(), spec.kv_pages_numel(),
                                               spec.kv_pages_numel()))
    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, partitions=3, provider=provider,
                      max_commands=1)
    scope = run.queue.begin(run.bind())
    with pytest.raises(lk.CommandError) as info:
        run.plan.enqueue_into(scope, run.args())
    assert (info.value.variant, info.value.payload[0]) == ("CommandCapacityExceeded", 1)
    completion = scope.finish()
    assert completion.submitted() == 0
    completion.wait()

    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, partitions=3, provider=provider)
    run.workspace = run.workspace[:-1].clone()
    scope = run.queue.begin(run.bind())
    with pytest.raises(lk.EnqueueError) as info:
        run.plan.enqueue_into(scope, run.args())
    assert (info.value.variant, info.value.operand) == ("LengthMismatch", "workspace")
    assert scope.finish().submitted() == 0


def test_large_logits_and_outlier_token(oracle, provider):
    # gates/single_decode.rs:253-280 on one page, plus an outlier token scaled x8 in a long row
    spec = lk.Bf16PagedBatchDecodeSpec.new(1, 2, 1, 1)
    q = H.bf16_bits(np.full(128, 64.0, np.float32))
    k = np.zeros(spec.kv_pages_numel(), np.uint16)
    v = np.zeros(spec.kv_pages_numel(), np.uint16)
    for token, (kv, vv) in enumerate([(-64.0, -1.0), (0.0, 0.5), (64.0, 2.0)]):
        k[(16 + token) * 128:(17 + token) * 128] = H.bf16_bits(np.full(128, kv, np.float32))
        v[(16 + token) * 128:(17 + token) * 128] = H.bf16_bits(np.full(128, vv, np.float32))
    run = H.DecodeRun(spec, q, k, v, [0, 1], [1], [3], provider=provider)
    out, lse = run.run()
    eo, el = oracle.paged_decode(oracle.paged_spec(1, 2, 1, 1), q, k, v, [0, 1], [1], [3])
    H.check_decode(out, lse, eo, el, lse_limit=H.SPLIT_LSE_MAX_ABS)

    rng = np.random.default_rng(44)
    batch, qh, kvh, pool = 2, 64, 8, 160
    kv_lens = [16 * 64, 16 * 61 + 9]
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool)
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pool, qh, kvh)
    kf = rng.standard_normal(spec.kv_pages_numel(), dtype=np.float32).reshape(pool, 16, -1)
    vf = rng.standard_normal(spec.kv_pages_numel(), dtype=np.float32).reshape(pool, 16, -1)
    for r in range(batch):
        token = int(rng.integers(0, kv_lens[r]))
        page = indices[indptr[r] + token // 16]
        kf[page, token % 16] *= 8.0
        vf[page, token % 16] *= 8.0
    k, v = H.bf16_bits(kf.ravel()), H.bf16_bits(vf.ravel())
    q = H.normal_bf16(rng, spec.query_numel())
    ospec = oracle.paged_spec(batch, pool, qh, kvh)
    eo, el = oracle.paged_decode(ospec, q, k, v, indptr, indices, last, threads=8)
    for partitions, balanced in ((1, 0), (16, 0), (0, 1)):
        run = H.DecodeRun(spec, q, k, v, indptr, indices, last, partitions=partitions,
                          provider=provider, balanced=balanced)
        out, lse = run.run()
        H.check_decode(out, lse, eo, el, lse_limit=H.SPLIT_LSE_MAX_ABS)


def test_plan_is_immutable_and_reports_its_shape(provider):
    spec = lk.Bf16PagedBatchDecodeSpec.new(64, 20000, 32, 8)
    plan = provider.plan_bf16_paged_batch(spec, partitions=1)
    assert plan.spec() == spec and plan.algorithm() == lk.Bf16PagedBatchDecodeAlgorithm.Direct
    assert plan.commands() == 1 and plan.workspace_required_numel() == 0
    plan = provider.plan_bf16_paged_batch(lk.Bf16PagedBatchDecodeSpec.new(8, 20000, 64, 8),
                                          partitions=16)
    assert plan.commands() == 2 and not plan.merged_in_kernel() and plan.partitions() == 16
    assert plan.workspace_required_bytes() == 8 * 64 * 16 * 130 * 4
    plan = provider.plan_bf16_paged_batch(lk.Bf16PagedBatchDecodeSpec.new(8, 20000, 64, 8),
                                          partitions=16, merge_in_kernel=1)
    assert plan.commands() == 1 and plan.merged_in_kernel()
    assert plan.workspace_required_bytes() == 8 * 64 * 16 * 130 * 4
    with pytest.raises(lk.PlanError):
        provider.plan_bf16_paged_batch(spec, heads_per_cta=3)
