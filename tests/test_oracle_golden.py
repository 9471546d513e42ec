"""Pins the CPU oracle against every digest the reference published for this path."""
import json
import os

import numpy as np

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_digests.json")))
K_SALT, V_SALT = 0x4B455900, 0x56414C554500


def hx(value):
    return f"{value:016x}"


def test_digest_known_answer(oracle):
    g = GOLDEN["digest_self_test"]
    assert hx(oracle.digest_bf16(oracle.bf16_from_f32(g["bf16_values"]))) == g["digest"]


def test_bf16_rounding_matches_scalar(oracle):
    rng = np.random.default_rng(1)
    bits = rng.integers(0, 2**32, size=20000, dtype=np.uint64).astype(np.uint32)
    values = bits.view(np.float32)
    vector = oracle.bf16_from_f32(values)
    scalar = np.array([oracle.lib().lo_bf16_from_f32(float(v)) if not np.isnan(v) else 0
                       for v in values], dtype=np.uint16)
    ok = ~np.isnan(values)
    assert np.array_equal(vector[ok], scalar[ok])
    assert oracle.bf16_from_f32([np.nan])[0] == 0x7FC0
    # ties to even
    assert oracle.bf16_from_f32(np.array([0x3F808000], dtype=np.uint32).view(np.float32))[0] == 0x3F80
    assert oracle.bf16_from_f32(np.array([0x3F818000], dtype=np.uint32).view(np.float32))[0] == 0x3F82


def test_paged_decode_fixture_and_output_digests(oracle):
    for name, case in GOLDEN["paged_decode"]["cases"].items():
        batch, pages, qh, kvh = case["spec"]
        salt = int(case["salt"], 16)
        spec = oracle.paged_spec(batch, pages, qh, kvh)
        q = oracle.fixture_bf16(batch * qh * 128, salt)
        k = oracle.fixture_bf16(pages * 16 * kvh * 128, salt ^ K_SALT)
        v = oracle.fixture_bf16(pages * 16 * kvh * 128, salt ^ V_SALT)
        assert hx(oracle.digest_bf16(q)) == case["query"], name
        assert hx(oracle.digest_bf16(k)) == case["key_pages"], name
        assert hx(oracle.digest_bf16(v)) == case["value_pages"], name
        assert hx(oracle.digest_i32(case["indptr"])) == case["page_indptr"], name
        assert hx(oracle.digest_i32(case["indices"])) == case["page_indices"], name
        assert hx(oracle.digest_i32(case["last"])) == case["last_page_len"], name
        out, lse = oracle.paged_decode(spec, q, k, v, case["indptr"], case["indices"], case["last"])
        assert hx(oracle.digest_bf16(out)) == case["output"], name
        assert np.all(np.isfinite(lse))
        # threads do not change a single bit
        out_mt, lse_mt = oracle.paged_decode(spec, q, k, v, case["indptr"], case["indices"],
                                             case["last"], threads=4)
        assert np.array_equal(out, out_mt) and np.array_equal(lse.view(np.uint32), lse_mt.view(np.uint32))


def test_single_decode_output_digests(oracle):
    for name, case in GOLDEN["single_decode"]["cases"].items():
        kv_len, qh, kvh, salt = case["kv_len"], case["qh"], case["kvh"], int(case["salt"], 16)
        q = oracle.fixture_bf16(qh * 128, salt)
        k = oracle.fixture_bf16(kv_len * kvh * 128, salt ^ K_SALT)
        v = oracle.fixture_bf16(kv_len * kvh * 128, salt ^ V_SALT)
        out, _ = oracle.single_decode(kv_len, qh, kvh, q, k, v)
        assert hx(oracle.digest_bf16(out)) == case["output"], name


def test_single_decode_large_logits_digest(oracle):
    g = GOLDEN["single_decode"]["large_logits_l3"]
    q = oracle.bf16_from_f32(np.full(128, g["query"], dtype=np.float32))
    k = oracle.bf16_from_f32(np.repeat(np.array(g["key"], dtype=np.float32), 128))
    v = oracle.bf16_from_f32(np.repeat(np.array(g["value"], dtype=np.float32), 128))
    out, lse = oracle.single_decode(3, 1, 1, q, k, v)
    assert hx(oracle.digest_bf16(out)) == g["output"]
    assert hx(oracle.digest_f32(lse)) == g["lse"]


def _salted(oracle, salts, sizes):
    return {name: oracle.fixture_bf16(sizes[name], int(salts[name], 16)) for name in sizes}


def test_rope_paged_append_digests(oracle):
    g = GOLDEN["rope_paged_append"]
    batch, pages, qh, kvh = g["spec"]
    spec = oracle.paged_spec(batch, pages, qh, kvh)
    pool = pages * 16 * kvh * 128
    f = _salted(oracle, g["salts"], {"query": batch * qh * 128, "key": batch * kvh * 128,
                                     "value": batch * kvh * 128, "key_pages": pool,
                                     "value_pages": pool})
    q_out, kp, vp = oracle.rope_append(spec, f["query"], f["key"], f["value"], g["indptr"],
                                       g["indices"], g["last"], f["key_pages"], f["value_pages"])
    assert hx(oracle.digest_bf16(q_out)) == g["query_output"]
    assert hx(oracle.digest_bf16(kp)) == g["key_pages"]
    assert hx(oracle.digest_bf16(vp)) == g["value_pages"]
    lens = oracle.request_kv_lens(g["indptr"], g["last"])
    assert list(lens - 1) == g["positions"]


def test_rope_paged_append_tokens_digests(oracle):
    g = GOLDEN["rope_paged_append_tokens"]["six_tokens"]
    tokens, batch, pages, qh, kvh = g["spec"]
    spec = oracle.paged_spec(batch, pages, qh, kvh)
    pool = pages * 16 * kvh * 128
    f = _salted(oracle, g["salts"], {"query": tokens * qh * 128, "key": tokens * kvh * 128,
                                     "value": tokens * kvh * 128, "key_pages": pool,
                                     "value_pages": pool})
    slots = oracle.append_tokens_validate(spec, tokens, g["batch_indices"], g["positions"],
                                          g["indptr"], g["indices"], g["last"])
    assert [list(s) for s in slots] == g["slots"]
    q_out, kp, vp = oracle.rope_append_tokens(spec, tokens, f["query"], f["key"], f["value"],
                                              g["batch_indices"], g["positions"], g["indptr"],
                                              g["indices"], g["last"], f["key_pages"],
                                              f["value_pages"])
    assert hx(oracle.digest_bf16(q_out)) == g["query_output"]
    assert hx(oracle.digest_bf16(vp)) == g["value_pages"]

    g = GOLDEN["rope_paged_append_tokens"]["limit_64_tokens"]
    tokens, batch, pages, qh, kvh = g["spec"]
    spec = oracle.paged_spec(batch, pages, qh, kvh)
    pool = pages * 16 * kvh * 128
    f = _salted(oracle, g["salts"], {"query": tokens * qh * 128, "key": tokens * kvh * 128,
                                     "value": tokens * kvh * 128, "key_pages": pool,
                                     "value_pages": pool})
    q_out, kp, vp = oracle.rope_append_tokens(spec, tokens, f["query"], f["key"], f["value"],
                                              [0] * 64, list(range(64)), g["indptr"],
                                              g["indices"], g["last"], f["key_pages"],
                                              f["value_pages"])
    assert hx(oracle.digest_bf16(kp)) == g["key_pages"]
    assert hx(oracle.digest_bf16(vp)) == g["value_pages"]
