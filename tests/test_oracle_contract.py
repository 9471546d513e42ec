"""The reference's CPU-side contract tests, restated against the oracle.

Cases follow crates/loom-infer/src/attention/paged_decode/tests.rs,
.../paged_append/tests.rs, crates/loom-infer/src/rope/tests.rs and the split-K part of
.../single_decode/tests.rs.
"""
import math

import numpy as np
import pytest


def err(oracle, fn, *args, **kw):
    with pytest.raises(oracle.OracleError) as info:
        fn(*args, **kw)
    return info.value


def test_spec_rejects_unsupported_shapes_and_overflow(oracle):
    # paged_decode/tests.rs:54-104
    for dims in [(0, 1, 1, 1, 128, 16), (1, 0, 1, 1, 128, 16), (1, 1, 0, 1, 128, 16),
                 (1, 1, 1, 0, 128, 16), (1, 1, 1, 1, 0, 16), (1, 1, 1, 1, 128, 0)]:
        assert err(oracle, oracle.paged_spec, *dims).variant == "ZeroDimension"
    e = err(oracle, oracle.paged_spec, 1, 1, 1, 1, 64, 16)
    assert (e.variant, e.payload[:2]) == ("UnsupportedHeadDimension", (128, 64))
    e = err(oracle, oracle.paged_spec, 1, 1, 1, 1, 128, 8)
    assert (e.variant, e.payload[:2]) == ("UnsupportedPageSize", (16, 8))
    e = err(oracle, oracle.paged_spec, 1, 1, 6, 4, 128, 16)
    assert (e.variant, e.payload[:2]) == ("InvalidHeadMapping", (6, 4))
    assert err(oracle, oracle.paged_spec, 2**64 - 1, 1, 1, 1).variant == "ElementCountOverflow"
    assert err(oracle, oracle.paged_spec, 1, 2**64 - 1, 1, 1).variant == "ElementCountOverflow"


def test_page_table_lengths_and_token_mapping(oracle):
    # paged_decode/tests.rs:107-133
    spec = oracle.paged_spec(3, 8, 4, 2)
    indptr, indices, last = [0, 2, 3, 6], [5, 1, 7, 2, 0, 6], [3, 16, 1]
    oracle.validate_page_table(spec, indptr, indices, last)
    assert list(oracle.request_kv_lens(indptr, last)) == [19, 16, 33]
    # token -> slot through the explicit-append validation, which uses the same mapping
    slots = oracle.append_tokens_validate(spec, 6, [0, 0, 0, 0, 1, 2], [0, 15, 16, 18, 15, 32],
                                          indptr, indices, last)
    assert slots == [(5, 0), (5, 15), (1, 0), (1, 2), (7, 15), (6, 0)]
    e = err(oracle, oracle.append_tokens_validate, spec, 1, [0], [19], indptr, indices, last)
    assert e.variant == "AppendPositionOutOfRange"


def test_page_table_rejects_malformed_metadata(oracle):
    # paged_decode/tests.rs:136-217
    spec = oracle.paged_spec(2, 4, 4, 2)
    cases = [
        (([0, 1], [0, 1], [16, 16]), ("LengthMismatch", "page_indptr", (3, 2))),
        (([0, 1, 2], [0, 1], [16]), ("LengthMismatch", "last_page_len", (2, 1))),
        (([1, 2, 3], [0, 1, 2], [16, 16]), ("InvalidPageIndptrStart", "", (1,))),
        (([0, 2, 1], [0], [16, 16]), ("NonMonotonicPageIndptr", "", (1, 2, 1))),
        (([0, 0, 1], [0], [16, 16]), ("EmptyPagedRequest", "", (0,))),
        (([0, 1, 2], [0, 1], [0, 16]), ("InvalidLastPageLength", "", (0, 0, 16))),
        (([0, 1, 2], [0, 1], [16, 17]), ("InvalidLastPageLength", "", (1, 17, 16))),
        (([0, 1, 2], [0], [16, 16]), ("LengthMismatch", "page_indices", (2, 1))),
        (([0, 1, 2], [-1, 1], [16, 16]), ("PageIndexOutOfRange", "", (0, -1, 4))),
        (([0, 1, 2], [0, 4], [16, 16]), ("PageIndexOutOfRange", "", (1, 4, 4))),
    ]
    for args, (variant, buffer, payload) in cases:
        e = err(oracle, oracle.validate_page_table, spec, *args)
        assert (e.variant, e.buffer, e.payload[:len(payload)]) == (variant, buffer, payload)


def test_paged_reference_matches_contiguous_decode(oracle):
    # paged_decode/tests.rs:220-291
    spec = oracle.paged_spec(3, 7, 8, 2)
    indptr, indices, last = [0, 1, 3, 6], [4, 6, 1, 5, 0, 3], [1, 7, 16]
    q = oracle.fixture_bf16(3 * 8 * 128, 0x504147454451)
    k = oracle.fixture_bf16(7 * 16 * 2 * 128, 0x50414745444B)
    v = oracle.fixture_bf16(7 * 16 * 2 * 128, 0x504147454456)
    out, lse = oracle.paged_decode(spec, q, k, v, indptr, indices, last)
    lens = oracle.request_kv_lens(indptr, last)
    kr, vr = k.reshape(7, 16, 256), v.reshape(7, 16, 256)
    for r in range(3):
        rows = [(indices[indptr[r] + t // 16], t % 16) for t in range(lens[r])]
        ck = np.concatenate([kr[p, o] for p, o in rows])
        cv = np.concatenate([vr[p, o] for p, o in rows])
        eo, el = oracle.single_decode(int(lens[r]), 8, 2, q[r * 1024:(r + 1) * 1024], ck, cv)
        assert np.array_equal(out[r * 1024:(r + 1) * 1024], eo)
        assert np.array_equal(lse[r * 8:(r + 1) * 8].view(np.uint32), el.view(np.uint32))


def test_paged_reference_requires_exact_lengths(oracle):
    # paged_decode/tests.rs:294-401
    spec = oracle.paged_spec(2, 2, 2, 1)
    q = np.zeros(2 * 2 * 128, np.uint16)
    kv = np.zeros(2 * 16 * 128, np.uint16)
    table = ([0, 1, 2], [0, 1], [16, 16])
    e = err(oracle, oracle.paged_decode, spec, q[:-1], kv, kv, *table)
    assert (e.variant, e.buffer, e.payload[:2]) == ("LengthMismatch", "Q", (512, 511))
    e = err(oracle, oracle.paged_decode, spec, q, kv[:-1], kv, *table)
    assert (e.variant, e.buffer) == ("LengthMismatch", "K_pages")
    e = err(oracle, oracle.paged_decode, spec, q, kv, kv[:-1], *table)
    assert (e.variant, e.buffer) == ("LengthMismatch", "V_pages")
    e = err(oracle, oracle.paged_decode, spec, q, kv, kv, *table, out=np.zeros(511, np.uint16))
    assert (e.variant, e.buffer) == ("LengthMismatch", "O")
    e = err(oracle, oracle.paged_decode, spec, q, kv, kv, *table, lse=np.zeros(3, np.float32))
    assert (e.variant, e.buffer) == ("LengthMismatch", "LSE")


def test_two_token_softmax_and_gqa_mapping(oracle):
    # single_decode/tests.rs:22-64
    q = np.zeros(128, np.uint16)
    q[0] = oracle.bf16_from_f32([math.sqrt(128.0)])[0]
    k = np.zeros(256, np.uint16)
    k[128] = 0x3F80
    v = np.zeros(256, np.uint16)
    v[128:] = oracle.bf16_from_f32([2.0])[0]
    out, lse = oracle.single_decode(2, 1, 1, q, k, v)
    score = np.float32(oracle.bf16_to_f32(q[:1])[0]) * np.float32(1.0 / math.sqrt(128.0))
    prob = np.exp(score) / (np.float32(1.0) + np.exp(score))
    assert np.all(out == oracle.bf16_from_f32([2.0 * prob])[0])
    assert abs(lse[0] - np.log1p(np.exp(score)) * 1.4426950408889634) < 1e-6

    v = np.concatenate([oracle.bf16_from_f32(np.full(128, 1.5)), oracle.bf16_from_f32(np.full(128, -2.0))])
    out, lse = oracle.single_decode(1, 4, 2, np.zeros(512, np.uint16), np.zeros(256, np.uint16), v)
    assert np.array_equal(oracle.bf16_to_f32(out), np.repeat([1.5, 1.5, -2.0, -2.0], 128).astype(np.float32))
    assert np.array_equal(lse, np.zeros(4, np.float32))


def test_split_k_partition_rule_and_state_layout(oracle):
    # single_decode/tests.rs:230-252,274-300
    assert [oracle.split_k_partition_range(10, 4, p) for p in range(5)] == \
        [(0, 3), (3, 6), (6, 8), (8, 10), None]
    for partitions in (0, 8):
        e = err(oracle, oracle.split_k_partials, 7, 8, 1, partitions, np.zeros(1024, np.uint16),
                np.zeros(7 * 128, np.uint16), np.zeros(7 * 128, np.uint16))
        assert (e.variant, e.payload[:2]) == ("InvalidPartitionCount", (partitions, 7))
    q = np.zeros(128, np.uint16)
    q[0] = oracle.bf16_from_f32([math.sqrt(128.0)])[0]
    k = np.zeros(256, np.uint16)
    k[128] = 0x3F80
    v = np.concatenate([oracle.bf16_from_f32(np.full(128, 1.5)), oracle.bf16_from_f32(np.full(128, -2.0))])
    ws = oracle.split_k_partials(2, 1, 1, 2, q, k, v)
    first, second = ws[:130], ws[130:]
    assert first[0] == 0.0 and first[1] == 1.0 and np.all(first[2:] == 1.5)
    expect = np.float32(oracle.bf16_to_f32(q[:1])[0]) * np.float32(1 / math.sqrt(128.0)) * np.float32(1.4426950408889634)
    assert second[0] == expect and second[1] == 1.0 and np.all(second[2:] == -2.0)


def test_split_k_matches_direct_across_shapes(oracle):
    # single_decode/tests.rs:303-352
    for kv_len, qh, kvh, parts, salt in [(1, 8, 8, 1, 0x1001), (7, 8, 1, 3, 0x2001),
                                         (33, 8, 1, 8, 0x3001), (127, 16, 4, 8, 0x4001)]:
        q = oracle.fixture_bf16(qh * 128, salt)
        k = oracle.fixture_bf16(kv_len * kvh * 128, salt ^ 0x4B455900)
        v = oracle.fixture_bf16(kv_len * kvh * 128, salt ^ 0x56414C554500)
        eo, el = oracle.single_decode(kv_len, qh, kvh, q, k, v)
        ws = oracle.split_k_partials(kv_len, qh, kvh, parts, q, k, v)
        ao, al = oracle.split_k_merge(qh, parts, ws)
        assert np.array_equal(ao, eo)
        assert np.max(np.abs(al - el)) <= 1e-6


def test_split_k_large_logits_finite_and_lengths(oracle):
    # single_decode/tests.rs:355-441
    q = oracle.bf16_from_f32(np.full(128, 64.0))
    k = oracle.bf16_from_f32(np.repeat([-64.0, 0.0, 64.0], 128))
    v = oracle.bf16_from_f32(np.ones(384))
    ws = oracle.split_k_partials(3, 1, 1, 3, q, k, v)
    out, lse = oracle.split_k_merge(1, 3, ws)
    assert np.all(np.isfinite(ws)) and np.all(np.isfinite(oracle.bf16_to_f32(out))) and np.all(np.isfinite(lse))
    e = err(oracle, oracle.split_k_partials, 2, 2, 1, 2, np.zeros(256, np.uint16),
            np.zeros(256, np.uint16), np.zeros(256, np.uint16),
            workspace=np.zeros(2 * 2 * 130 - 1, np.float32))
    assert (e.variant, e.buffer, e.payload[:2]) == ("LengthMismatch", "workspace", (520, 519))


def test_paged_split_k_matches_direct_paged_reference(oracle):
    # extension: page-balanced paged split-K == direct paged reference (O bit-exact, LSE 1e-6
    # in the spirit of single_decode/tests.rs:303-352), including chunks with no pages
    spec = oracle.paged_spec(3, 9, 8, 2)
    indptr, indices, last = [0, 1, 4, 9], [4, 6, 1, 5, 0, 3, 8, 2, 7], [1, 7, 16]
    q = oracle.fixture_bf16(3 * 8 * 128, 77)
    k = oracle.fixture_bf16(9 * 16 * 2 * 128, 78)
    v = oracle.fixture_bf16(9 * 16 * 2 * 128, 79)
    eo, el = oracle.paged_decode(spec, q, k, v, indptr, indices, last)
    for parts in (1, 2, 3, 4, 7):
        ao, al, ws = oracle.paged_split_k(spec, parts, q, k, v, indptr, indices, last)
        assert np.max(np.abs(oracle.bf16_to_f32(ao) - oracle.bf16_to_f32(eo))) <= 2 ** -9
        assert np.max(np.abs(al - el)) <= 1e-5
        assert np.all(np.isfinite(ws))


def test_rope_known_answers(oracle):
    # rope/tests.rs:3-131
    q = oracle.bf16_from_f32([1, 2, 3, 4, 5, 6])
    qo, ko = oracle.rope(1, 1, 1, q, q, [1], head_dim=6, rotary_dim=4)
    f = np.float32
    c1, s1 = f(math.cos(1.0)), f(math.sin(1.0))
    # angle for pair 1: 10000^-0.5 = 0.01
    a1 = np.float32(10000.0) ** np.float32(-0.5)
    ca, sa = f(math.cos(float(a1))), f(math.sin(float(a1)))
    exp = oracle.bf16_from_f32([f(1) * c1 - f(3) * s1, f(2) * ca - f(4) * sa,
                                f(3) * c1 + f(1) * s1, f(4) * ca + f(2) * sa])
    assert list(qo[:4]) == list(exp)
    assert list(qo[4:]) == list(q[4:]) and list(qo) == list(ko)

    q = oracle.bf16_from_f32(np.arange(256) / 256.0 - 0.5)
    k = oracle.bf16_from_f32(np.arange(128) / 128.0 - 0.25)
    qo, ko = oracle.rope(1, 2, 1, q, k, [0])
    assert np.array_equal(qo, q) and np.array_equal(ko, k)

    qo, ko = oracle.rope(1, 1, 1, oracle.bf16_from_f32(np.full(128, 0.25)),
                         oracle.bf16_from_f32(np.full(128, -0.5)), [32767])
    assert np.all(np.isfinite(oracle.bf16_to_f32(qo))) and np.all(np.isfinite(oracle.bf16_to_f32(ko)))

    z = np.zeros(128, np.uint16)
    e = err(oracle, oracle.rope, 1, 1, 1, z, z, [0], rotary_dim=127)
    assert (e.variant, e.payload[:2]) == ("InvalidRotaryDimension", (127, 128))
    assert err(oracle, oracle.rope, 1, 1, 1, z, z, [0], scale=0.0).variant == "InvalidRopeScale"
    assert err(oracle, oracle.rope, 1, 1, 1, z, z, [0], theta=1.0).variant == "InvalidRopeTheta"
    z2 = np.zeros(2, np.uint16)
    e = err(oracle, oracle.rope, 1, 1, 1, z2, z2, [-1], head_dim=2, rotary_dim=2)
    assert (e.variant, e.payload[:2]) == ("NegativePositionId", (0, -1))
    e = err(oracle, oracle.rope, 1, 1, 1, z2[:1], z2, [0], head_dim=2, rotary_dim=2)
    assert (e.variant, e.buffer, e.payload[:2]) == ("LengthMismatch", "query", (2, 1))


def test_append_to_arbitrary_final_pages(oracle):
    # paged_append/tests.rs:15-69
    spec = oracle.paged_spec(3, 8, 4, 2)
    indptr, indices, last = [0, 1, 3, 5], [7, 2, 6, 5, 1], [3, 1, 16]
    q = oracle.fixture_bf16(3 * 4 * 128, 1)
    k = oracle.fixture_bf16(3 * 2 * 128, 2)
    v = oracle.fixture_bf16(3 * 2 * 128, 3)
    ks, vs = oracle.bf16_from_f32([-7.0])[0], oracle.bf16_from_f32([9.0])[0]
    pool = 8 * 16 * 2 * 128
    qo, kp, vp = oracle.rope_append(spec, q, k, v, indptr, indices, last,
                                    np.full(pool, ks, np.uint16), np.full(pool, vs, np.uint16))
    touched = np.zeros(pool, bool)
    for request, (page, off) in enumerate([(7, 2), (6, 0), (1, 15)]):
        for h in range(2):
            dst = ((page * 16 + off) * 2 + h) * 128
            src = (request * 2 + h) * 128
            assert np.array_equal(vp[dst:dst + 128], v[src:src + 128])
            assert np.all(kp[dst:dst + 128] != ks)
            touched[dst:dst + 128] = True
    assert np.all(kp[~touched] == ks) and np.all(vp[~touched] == vs)
    assert np.all(np.isfinite(oracle.bf16_to_f32(qo)))


def test_append_rejects_duplicates_and_short_buffers(oracle):
    # paged_append/tests.rs:72-115
    spec = oracle.paged_spec(2, 2, 2, 1)
    e = err(oracle, oracle.append_validate_page_table, spec, [0, 1, 2], [1, 1], [4, 4])
    assert (e.variant, e.payload) == ("DuplicatePageAppendSlot", (0, 1, 1, 3))
    spec = oracle.paged_spec(1, 1, 1, 1)
    z = np.zeros(128, np.uint16)
    pool = np.zeros(16 * 128, np.uint16)
    e = err(oracle, oracle.rope_append, spec, z[:-1], z, z, [0, 1], [0], [1], pool, pool)
    assert (e.variant, e.buffer, e.payload[:2]) == ("LengthMismatch", "query", (128, 127))


def test_explicit_append_shuffled_tokens(oracle):
    # paged_append/tests.rs:117-184
    spec = oracle.paged_spec(3, 8, 4, 2)
    indptr, indices, last = [0, 2, 4, 6], [7, 3, 2, 6, 3, 1], [5, 8, 4]
    batch_indices, positions = [2, 0, 1, 0, 2, 1], [17, 3, 20, 16, 16, 19]
    expected = [(1, 1), (7, 3), (6, 4), (3, 0), (1, 0), (6, 3)]
    assert oracle.append_tokens_validate(spec, 6, batch_indices, positions, indptr, indices,
                                         last) == expected
    q = oracle.fixture_bf16(6 * 4 * 128, 11)
    k = oracle.fixture_bf16(6 * 2 * 128, 12)
    v = oracle.fixture_bf16(6 * 2 * 128, 13)
    ks, vs = oracle.bf16_from_f32([-7.0])[0], oracle.bf16_from_f32([9.0])[0]
    pool = 8 * 16 * 2 * 128
    qo, kp, vp = oracle.rope_append_tokens(spec, 6, q, k, v, batch_indices, positions, indptr,
                                           indices, last, np.full(pool, ks, np.uint16),
                                           np.full(pool, vs, np.uint16))
    for token, (page, off) in enumerate(expected):
        for h in range(2):
            src = (token * 2 + h) * 128
            dst = ((page * 16 + off) * 2 + h) * 128
            assert np.array_equal(vp[dst:dst + 128], v[src:src + 128])
            assert np.all(kp[dst:dst + 128] != ks)
    assert np.all(np.isfinite(oracle.bf16_to_f32(qo)))


def test_explicit_append_rejects_invalid_mappings(oracle):
    # paged_append/tests.rs:186-247
    spec = oracle.paged_spec(2, 4, 2, 1)
    table = ([0, 2, 4], [3, 1, 3, 2], [4, 4])
    e = err(oracle, oracle.append_tokens_validate, spec, 2, [0, 2], [1, 17], *table)
    assert (e.variant, e.payload[:3]) == ("AppendBatchIndexOutOfRange", (1, 2, 2))
    e = err(oracle, oracle.append_tokens_validate, spec, 2, [0, 1], [1, 20], *table)
    assert (e.variant, e.payload) == ("AppendPositionOutOfRange", (1, 1, 20, 20))
    e = err(oracle, oracle.append_tokens_validate, spec, 2, [0, 1], [2, 2], *table)
    assert (e.variant, e.payload) == ("DuplicatePageAppendTokenSlot", (0, 1, 3, 2))
    spec = oracle.paged_spec(1, 1, 1, 1)
    e = err(oracle, oracle.append_tokens_validate, spec, 65, [0] * 65, [0] * 65, [0, 1], [0], [16])
    assert (e.variant, e.payload[:2]) == ("UnsupportedAppendTokenCount", (64, 65))


def test_chunked_explicit_append_equals_one_extended_call(oracle):
    # The extended (any-total) append equals the contract's <=64-token calls applied in
    # chunks: chunks write disjoint slots, and Q rows are per token.
    rng = np.random.default_rng(5)
    batch, pages_per, qh, kvh = 4, 6, 4, 2
    spec = oracle.paged_spec(batch, 64, qh, kvh)
    perm = rng.permutation(64)[:batch * pages_per]
    indptr = list(range(0, batch * pages_per + 1, pages_per))
    last = [16] * batch
    tokens = 150
    pairs = rng.permutation(batch * pages_per * 16)[:tokens]
    batch_indices = (pairs // (pages_per * 16)).astype(np.int32)
    positions = (pairs % (pages_per * 16)).astype(np.int32)
    q = oracle.fixture_bf16(tokens * qh * 128, 21)
    k = oracle.fixture_bf16(tokens * kvh * 128, 22)
    v = oracle.fixture_bf16(tokens * kvh * 128, 23)
    pool = 64 * 16 * kvh * 128
    kp0, vp0 = oracle.fixture_bf16(pool, 24), oracle.fixture_bf16(pool, 25)
    qo, kp, vp = oracle.rope_append_tokens(spec, tokens, q, k, v, batch_indices, positions,
                                           indptr, perm, last, kp0, vp0, max_tokens=0)
    kc, vc, qc = kp0.copy(), vp0.copy(), []
    for start in range(0, tokens, 64):
        stop = min(tokens, start + 64)
        qi, kc, vc = oracle.rope_append_tokens(
            spec, stop - start, q[start * qh * 128:stop * qh * 128],
            k[start * kvh * 128:stop * kvh * 128], v[start * kvh * 128:stop * kvh * 128],
            batch_indices[start:stop], positions[start:stop], indptr, perm, last, kc, vc)
        qc.append(qi)
    assert np.array_equal(np.concatenate(qc), qo)
    assert np.array_equal(kc, kp) and np.array_equal(vc, vp)
