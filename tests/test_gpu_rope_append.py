"""GPU parity of fused NeoX RoPE + paged KV append against the CPU oracle, through the C ABI.

Cases follow crates/loom-infer-validation/src/gates/rope.rs:249-691,855-1086 of the reference.
Gates: V bit-exact, page/slot indexing bit-exact (every untouched pool element unchanged),
rotated Q/K within one BF16 ulp of the CPU reference.
"""
import json
import os

import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from tests import helpers as H

pytestmark = pytest.mark.gpu
GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_digests.json")))


@pytest.fixture(scope="module")
def provider():
    return lk.RopeProvider.load(0)


def ulp_distance(a_bits, b_bits):
    """Distance in BF16 ulps on the ordered-integer line (sign-magnitude -> two's complement)."""
    def ordered(bits):
        bits = bits.astype(np.int32)
        return np.where(bits & 0x8000, -(bits & 0x7FFF), bits)
    return np.abs(ordered(a_bits) - ordered(b_bits))


class AppendRun:
    def __init__(self, provider, spec, q, k, v, indptr, indices, last, k_pages, v_pages,
                 batch_indices=None, positions=None, max_commands=1, one_command=False):
        self.spec = spec
        self.provider = provider
        self.explicit = batch_indices is not None
        self.plan = (provider.plan_bf16_paged_append_tokens(spec, one_command=one_command)
                     if self.explicit else provider.plan_bf16_paged_append(spec))
        self.stream = torch.cuda.Stream()
        self.queue = lk.CommandQueue(self.stream, max(max_commands, self.plan.commands()))
        numel = self.plan.workspace_required_numel()  # extended plans: validate, then scatter
        self.workspace = (torch.full((numel,), -1, dtype=torch.int32, device="cuda:0")
                          if numel else None)
        self.t = dict(query=H.dev_bf16(q), key=H.dev_bf16(k), value=H.dev_bf16(v),
                      page_indptr=H.dev_i32(indptr), page_indices=H.dev_i32(indices),
                      last_page_len=H.dev_i32(last))
        if self.explicit:
            self.t["batch_indices"] = H.dev_i32(batch_indices)
            self.t["positions"] = H.dev_i32(positions)
        self.q_out = torch.full((len(q),), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        self.k_pages = H.dev_bf16(k_pages)
        self.v_pages = H.dev_bf16(v_pages)
        torch.cuda.synchronize()

    def bind(self, bindings=None):
        b = bindings or self.queue.bindings(12)
        order = (["query", "key", "value", "batch_indices", "positions", "page_indptr",
                  "page_indices", "last_page_len"] if self.explicit else
                 ["query", "key", "value", "page_indptr", "page_indices", "last_page_len"])
        self.h = {name: b.bind_read(self.t[name]) for name in order}
        self.h_q = b.bind_read_write(self.q_out)
        self.h_k = b.bind_read_write(self.k_pages)
        self.h_v = b.bind_read_write(self.v_pages)
        self.h_ws = b.bind_read_write(self.workspace) if self.workspace is not None else None
        return b

    def args(self):
        if not self.explicit:
            return lk.Bf16RopePagedKvAppendArgs(query_output=self.h_q.write(),
                                                key_pages=self.h_k.write(),
                                                value_pages=self.h_v.write(), **self.h)
        return lk.Bf16RopePagedKvAppendTokensArgs(query_output=self.h_q.write(),
                                                  key_pages=self.h_k.write(),
                                                  value_pages=self.h_v.write(),
                                                  workspace=self.h_ws, **self.h)

    def run(self):
        scope = self.queue.begin(self.bind())
        self.plan.enqueue_into(scope, self.args())
        completion = scope.finish()
        self.submitted = completion.submitted()
        b = completion.wait()
        # (only the checked build of the library writes this word: an index outside its operand)
        assert self.provider.device_status() == 0
        return (H.host_bits(b.take_read_write(self.h_q)), H.host_bits(b.take_read_write(self.h_k)),
                H.host_bits(b.take_read_write(self.h_v)))


def within_one_ulp(actual, expected, label="rotated"):
    """Rotated rows are within one BF16 ulp of the CPU reference.

    A rotation output is a difference of two products, so where it cancels to almost nothing its
    own ulp says little; there the bound is one BF16 ulp at the magnitude of the rotated pair
    (i, i+64), which the rotation preserves.  What the comparison found is printed (run pytest
    with -s): how many elements differ at all, the worst distance in ulps of the element itself,
    and how many elements needed the pair-magnitude bound (the reference's own GPU kernel reports
    its mismatching bits the same way, docs/results/h20-bf16-rope-paged-kv-append-tokens-
    correctness-20260806.json)."""
    distance = ulp_distance(actual, expected)
    differing = int((distance > 0).sum())
    loose = distance > 1
    print(f"{label}: {differing} of {distance.size} elements differ from the CPU reference, "
          f"worst {int(distance.max()) if distance.size else 0} ulp, "
          f"{int(loose.sum())} beyond 1 ulp of themselves (checked at the pair's magnitude)")
    if not loose.any():
        return True
    e = np.abs(H.bits_to_f32(expected)).reshape(-1, 2, 64)
    pair = np.sqrt(e[:, 0] ** 2 + e[:, 1] ** 2)
    pair_ulp = 2.0 ** (np.floor(np.log2(np.maximum(pair, 2.0 ** -120))) - 7)
    bound = np.stack([pair_ulp, pair_ulp], axis=1).reshape(-1)
    err = np.abs(H.bits_to_f32(actual) - H.bits_to_f32(expected))
    return bool(np.all(err[loose] <= bound[loose])) and loose.mean() < 1e-4


def check_append(actual, expected):
    (q, kp, vp), (eq, ekp, evp) = actual, expected
    assert np.array_equal(vp, evp), "V pages must be bit-exact"
    assert np.all(np.isfinite(H.bits_to_f32(q)))
    assert within_one_ulp(q, eq, "rotated Q"), "rotated Q beyond one BF16 ulp"
    # K pages: untouched elements are bit-identical, touched rows within one ulp
    changed = kp != ekp
    assert within_one_ulp(kp, ekp, "K pages"), "rotated K beyond one BF16 ulp"
    assert np.abs(H.bits_to_f32(q) - H.bits_to_f32(eq)).max() <= H.GATE_OUTPUT_MAX_ABS
    return int((q != eq).sum() + changed.sum())


def salted(oracle, salts, sizes):
    return {name: oracle.fixture_bf16(sizes[name], int(salts[name], 16)) for name in sizes}


def test_paged_append_gate_case(oracle, provider):
    g = GOLDEN["rope_paged_append"]
    batch, pages, qh, kvh = g["spec"]
    pool = pages * 16 * kvh * 128
    f = salted(oracle, g["salts"], {"query": batch * qh * 128, "key": batch * kvh * 128,
                                    "value": batch * kvh * 128, "key_pages": pool,
                                    "value_pages": pool})
    spec = lk.Bf16RopePagedKvAppendSpec.new(batch, pages, qh, kvh)
    table = spec.validate_page_table(g["indptr"], g["indices"], g["last"])
    slots = [table.physical_page_for_token(r, table.request_kv_len(r) - 1) for r in range(batch)]
    assert [list(s) for s in slots] == g["slots"]
    run = AppendRun(provider, spec, f["query"], f["key"], f["value"], g["indptr"], g["indices"],
                    g["last"], f["key_pages"], f["value_pages"])
    actual = run.run()
    assert run.submitted == 1
    expected = oracle.rope_append(oracle.paged_spec(batch, pages, qh, kvh), f["query"], f["key"],
                                  f["value"], g["indptr"], g["indices"], g["last"],
                                  f["key_pages"], f["value_pages"])
    assert f"{oracle.digest_bf16(expected[2]):016x}" == g["value_pages"]
    check_append(actual, expected)
    assert f"{oracle.digest_bf16(actual[2]):016x}" == g["value_pages"]


@pytest.mark.parametrize("name", ["six_tokens", "limit_64_tokens"])
def test_paged_append_tokens_gate_cases(oracle, provider, name):
    g = GOLDEN["rope_paged_append_tokens"][name]
    tokens, batch, pages, qh, kvh = g["spec"]
    pool = pages * 16 * kvh * 128
    f = salted(oracle, g["salts"], {"query": tokens * qh * 128, "key": tokens * kvh * 128,
                                    "value": tokens * kvh * 128, "key_pages": pool,
                                    "value_pages": pool})
    batch_indices = g.get("batch_indices", [0] * tokens)
    positions = g.get("positions", list(range(tokens)))
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new(tokens, batch, pages, qh, kvh)
    slots = spec.validate_metadata(batch_indices, positions, g["indptr"], g["indices"], g["last"])
    if "slots" in g:
        assert [list(s) for s in slots] == g["slots"]
    run = AppendRun(provider, spec, f["query"], f["key"], f["value"], g["indptr"], g["indices"],
                    g["last"], f["key_pages"], f["value_pages"], batch_indices, positions)
    actual = run.run()
    assert run.submitted == 1
    expected = oracle.rope_append_tokens(oracle.paged_spec(batch, pages, qh, kvh), tokens,
                                         f["query"], f["key"], f["value"], batch_indices,
                                         positions, g["indptr"], g["indices"], g["last"],
                                         f["key_pages"], f["value_pages"])
    check_append(actual, expected)
    assert f"{oracle.digest_bf16(actual[2]):016x}" == g["value_pages"]


def test_short_metadata_is_rejected_before_submission(oracle, provider):
    # gates/rope.rs:622-691
    g = GOLDEN["rope_paged_append_tokens"]["six_tokens"]
    tokens, batch, pages, qh, kvh = g["spec"]
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new(tokens, batch, pages, qh, kvh)
    pool = pages * 16 * kvh * 128
    z = np.zeros
    run = AppendRun(provider, spec, z(tokens * qh * 128, np.uint16), z(tokens * kvh * 128, np.uint16),
                    z(tokens * kvh * 128, np.uint16), g["indptr"], g["indices"], g["last"],
                    z(pool, np.uint16), z(pool, np.uint16), g["batch_indices"][:-1], g["positions"])
    scope = run.queue.begin(run.bind())
    with pytest.raises(lk.EnqueueError) as info:
        run.plan.enqueue_into(scope, run.args())
    assert (info.value.variant, info.value.operand) == ("LengthMismatch", "batch_indices")
    assert info.value.payload[:2] == (6, 5)
    completion = scope.finish()
    assert completion.submitted() == 0
    completion.wait()


def guard_run(provider, spec, indptr, indices, last, batch_indices=None, positions=None,
              one_command=False):
    tokens = spec.tokens() if batch_indices is not None else spec.batch_size()
    qh, kvh = spec.num_query_heads(), spec.num_kv_heads()
    ks, vs = H.bf16_bits(np.array([-7.0], np.float32))[0], H.bf16_bits(np.array([9.0], np.float32))[0]
    pool = spec.kv_pages_numel()
    run = AppendRun(provider, spec, np.zeros(tokens * qh * 128, np.uint16),
                    np.zeros(tokens * kvh * 128, np.uint16), np.zeros(tokens * kvh * 128, np.uint16),
                    indptr, indices, last, np.full(pool, ks, np.uint16), np.full(pool, vs, np.uint16),
                    batch_indices, positions, one_command=one_command)
    q, kp, vp = run.run()
    assert np.all(np.isnan(H.bits_to_f32(q))), "Q output written despite invalid metadata"
    assert np.all(kp == ks) and np.all(vp == vs), "page pools written despite invalid metadata"


def test_device_guards_preserve_every_sentinel(provider):
    # gates/rope.rs:994-1086
    spec = lk.Bf16RopePagedKvAppendSpec.new(2, 2, 2, 1)
    guard_run(provider, spec, [0, 1, 2], [1, 1], [4, 4])        # duplicate final slot
    guard_run(provider, spec, [0, 2, 3], [2, 0, 1], [4, 5])     # invalid non-final page
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new(2, 2, 4, 2, 1)
    table = ([0, 2, 4], [3, 1, 3, 2], [4, 4])
    guard_run(provider, spec, *table, batch_indices=[0, 1], positions=[2, 2])    # duplicate slot
    guard_run(provider, spec, *table, batch_indices=[0, 2], positions=[1, 1])    # batch index
    guard_run(provider, spec, *table, batch_indices=[0, 1], positions=[1, 20])   # position
    guard_run(provider, spec, [0, 2, 4], [4, 1, 3, 2], [4, 4], batch_indices=[0, 1],
              positions=[16, 16])                                                # page index
    # the same through the any-total plan, as two commands and as one (the token CTAs wait for
    # the validators' verdict inside the kernel)
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new_extended(2, 2, 4, 2, 1)
    for one_command in (False, True):
        guard_run(provider, spec, *table, batch_indices=[0, 1], positions=[2, 2],
                  one_command=one_command)
        guard_run(provider, spec, *table, batch_indices=[0, 2], positions=[1, 1],
                  one_command=one_command)
        guard_run(provider, spec, [0, 2, 4], [4, 1, 3, 2], [4, 4], batch_indices=[0, 1],
                  positions=[16, 16], one_command=one_command)


def draw_append_batch(rng, batch, pool_pages, max_new=64, max_prior=2048):
    new = rng.integers(1, max_new + 1, size=batch)
    prior = rng.integers(0, max_prior + 1, size=batch)
    kv_lens = prior + new
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool_pages)
    batch_indices = np.repeat(np.arange(batch), new).astype(np.int32)
    positions = np.concatenate([prior[r] + np.arange(new[r]) for r in range(batch)]).astype(np.int32)
    return indptr, indices, last, batch_indices, positions


@pytest.mark.parametrize("one_command", [False, True])
@pytest.mark.parametrize("shuffle", [False, True])
def test_extended_append_equals_chunked_reference(oracle, provider, shuffle, one_command):
    # 32 requests x 1-64 new tokens, 32 q / 8 kv heads, priors 0-2048, shuffled 8192-page pool:
    # one extended command == the reference applied in <=64-token chunks
    rng = np.random.default_rng(0xC2)
    batch, pool_pages, qh, kvh = 32, 8192, 32, 8
    indptr, indices, last, batch_indices, positions = draw_append_batch(rng, batch, pool_pages)
    tokens = len(batch_indices)
    if shuffle:
        order = rng.permutation(tokens)
        batch_indices, positions = batch_indices[order], positions[order]
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new_extended(tokens, batch, pool_pages, qh, kvh)
    q = H.normal_bf16(rng, tokens * qh * 128)
    k = H.normal_bf16(rng, tokens * kvh * 128)
    v = H.normal_bf16(rng, tokens * kvh * 128)
    pool = spec.kv_pages_numel()
    kp0, vp0 = H.normal_bf16(rng, pool), H.normal_bf16(rng, pool)
    run = AppendRun(provider, spec, q, k, v, indptr, indices, last, kp0, vp0, batch_indices,
                    positions, one_command=one_command)
    actual = run.run()
    assert run.submitted == run.plan.commands() == (1 if one_command else 2)
    if one_command:
        # the words of the queue the token CTAs waited on are zero again: the same queue serves
        # the next call (outputs reset in between, so that stale rows cannot pass)
        run.q_out.fill_(float("nan"))
        again = run.run()
        assert all(np.array_equal(x, y) for x, y in zip(again, actual))
    ospec = oracle.paged_spec(batch, pool_pages, qh, kvh)
    kc, vc, qc = kp0, vp0, []
    for start in range(0, tokens, 64):
        stop = min(tokens, start + 64)
        qi, kc, vc = oracle.rope_append_tokens(
            ospec, stop - start, q[start * qh * 128:stop * qh * 128],
            k[start * kvh * 128:stop * kvh * 128], v[start * kvh * 128:stop * kvh * 128],
            batch_indices[start:stop], positions[start:stop], indptr, indices, last, kc, vc)
        qc.append(qi)
    mismatching = check_append(actual, (np.concatenate(qc), kc, vc))
    # property: rotation preserves the pair norm, so K pages keep every row norm within rounding
    assert mismatching <= 0.02 * (tokens * (qh + kvh) * 128)


def test_one_token_per_request_large_batch(oracle, provider):
    rng = np.random.default_rng(17)
    batch, pool_pages, qh, kvh = 300, 4096, 8, 2
    kv_lens = rng.integers(1, 200, size=batch)
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool_pages)
    spec = lk.Bf16RopePagedKvAppendSpec.new(batch, pool_pages, qh, kvh)
    q = H.normal_bf16(rng, batch * qh * 128)
    k = H.normal_bf16(rng, batch * kvh * 128)
    v = H.normal_bf16(rng, batch * kvh * 128)
    pool = spec.kv_pages_numel()
    kp0, vp0 = H.normal_bf16(rng, pool), H.normal_bf16(rng, pool)
    run = AppendRun(provider, spec, q, k, v, indptr, indices, last, kp0, vp0)
    actual = run.run()
    expected = oracle.rope_append(oracle.paged_spec(batch, pool_pages, qh, kvh), q, k, v, indptr,
                                  indices, last, kp0, vp0)
    check_append(actual, expected)


def test_position_zero_is_an_identity_and_large_positions_stay_finite(oracle, provider):
    # crates/loom-infer/src/rope/tests.rs:43-82 through the append path
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new(2, 2, 4096, 2, 1)
    q = H.bf16_bits((np.arange(2 * 2 * 128) / 256.0 - 0.5).astype(np.float32))
    k = H.bf16_bits((np.arange(2 * 128) / 128.0 - 0.25).astype(np.float32))
    v = H.bf16_bits(np.ones(2 * 128, np.float32))
    pool = spec.kv_pages_numel()
    indptr, indices, last = [0, 1, 2049], np.arange(2049, dtype=np.int32), [1, 16]
    run = AppendRun(provider, spec, q, k, v, indptr, indices, last, np.zeros(pool, np.uint16),
                    np.zeros(pool, np.uint16), [0, 1], [0, 32767])
    qo, kp, vp = run.run()
    assert np.array_equal(qo[:256], q[:256])                  # position 0: bit-exact identity
    assert np.array_equal(kp[:128], k[:128])
    assert np.all(np.isfinite(H.bits_to_f32(qo))) and np.all(np.isfinite(H.bits_to_f32(kp)))
    expected = oracle.rope_append_tokens(oracle.paged_spec(2, 4096, 2, 1), 2, q, k, v, [0, 1],
                                         [0, 32767], indptr, indices, last,
                                         np.zeros(pool, np.uint16), np.zeros(pool, np.uint16))
    check_append((qo, kp, vp), expected)
