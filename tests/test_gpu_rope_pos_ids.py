"""GPU parity of the stand-alone NeoX RoPE provider against the CPU oracle, through the C ABI.

Cases follow crates/loom-infer-validation/src/gates/rope.rs:22-247 of the reference: the
five-token reference case through position 32767, a short buffer rejected before submission, a
negative position id leaving the output sentinels of that token in place, and a partial rotary
dimension rejected at plan time.
"""
import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from tests import helpers as H
from tests.test_gpu_rope_append import within_one_ulp

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def provider():
    return lk.RopeProvider.load(0)


def run(provider, spec, q, k, positions, sentinel=float("nan")):
    plan = provider.plan_bf16_pos_ids(spec)
    stream = torch.cuda.Stream()
    queue = lk.CommandQueue(stream, 1)
    q_out = torch.full((spec.query_numel(),), sentinel, dtype=torch.bfloat16, device="cuda:0")
    k_out = torch.full((spec.key_numel(),), sentinel, dtype=torch.bfloat16, device="cuda:0")
    tensors = (H.dev_bf16(q), H.dev_bf16(k), H.dev_i32(positions))
    torch.cuda.synchronize()
    b = queue.bindings(5)
    reads = [b.bind_read(t) for t in tensors]
    hq, hk = b.bind_read_write(q_out), b.bind_read_write(k_out)
    scope = queue.begin(b)
    plan.enqueue_into(scope, lk.Bf16RopePosIdsArgs(*reads, hq.write(), hk.write()))
    completion = scope.finish()
    assert completion.submitted() == 1
    b = completion.wait()
    return H.host_bits(b.take_read_write(hq)), H.host_bits(b.take_read_write(hk))


def test_reference_case_matches_the_cpu_reference(provider, oracle):
    """rope.rs:22-116: tokens 5, 16/4 heads, positions 0, 1, 127, 4096, 32767."""
    spec = lk.Bf16RopePosIdsSpec.new(5, 16, 4, 128, 128, 1.0, 10000.0)
    positions = [0, 1, 127, 4096, 32767]
    q = oracle.fixture_bf16(spec.query_numel(), 0x524F5045)
    k = oracle.fixture_bf16(spec.key_numel(), 0x4B455900)
    eq, ek = oracle.rope(5, 16, 4, q, k, positions)
    aq, ak = run(provider, spec, q, k, positions)
    assert within_one_ulp(aq, eq) and within_one_ulp(ak, ek)
    assert np.abs(H.bits_to_f32(aq) - H.bits_to_f32(eq)).max() <= H.GATE_OUTPUT_MAX_ABS
    assert np.abs(H.bits_to_f32(ak) - H.bits_to_f32(ek)).max() <= H.GATE_OUTPUT_MAX_ABS
    # position 0 is the identity rotation: bit-exact copy of the input rows
    assert np.array_equal(aq[:16 * 128], q[:16 * 128]) and np.array_equal(ak[:4 * 128], k[:4 * 128])


@pytest.mark.parametrize("tokens,qh,kh,theta,scale", [(1, 1, 1, 10000.0, 1.0),
                                                      (37, 32, 8, 500000.0, 1.0),
                                                      (300, 8, 1, 10000.0, 4.0)])
def test_shapes_thetas_and_scales(provider, oracle, tokens, qh, kh, theta, scale):
    rng = np.random.default_rng(tokens)
    spec = lk.Bf16RopePosIdsSpec.new(tokens, qh, kh, 128, 128, scale, theta)
    positions = rng.integers(0, 131072, size=tokens).astype(np.int32)
    q = H.normal_bf16(rng, spec.query_numel())
    k = H.normal_bf16(rng, spec.key_numel())
    eq, ek = oracle.rope(tokens, qh, kh, q, k, positions, scale=scale, theta=theta)
    aq, ak = run(provider, spec, q, k, positions)
    assert within_one_ulp(aq, eq) and within_one_ulp(ak, ek)


@pytest.mark.parametrize("scale", [1.0, 0.25])
def test_largest_positions(provider, oracle, scale):
    """Positions up to 2^31 - 1: angles up to 2.1e9 stay inside the in-kernel reduction (scale 1);
    with scale 0.25 they reach 8.6e9 and take the library routine."""
    positions = np.array([2147483647, 2147483646, 1073741824, 1999999999, 65536, 3],
                         dtype=np.int32)
    rng = np.random.default_rng(11)
    spec = lk.Bf16RopePosIdsSpec.new(len(positions), 4, 2, 128, 128, scale, 10000.0)
    q = H.normal_bf16(rng, spec.query_numel())
    k = H.normal_bf16(rng, spec.key_numel())
    eq, ek = oracle.rope(len(positions), 4, 2, q, k, positions, scale=scale)
    aq, ak = run(provider, spec, q, k, positions)
    assert within_one_ulp(aq, eq) and within_one_ulp(ak, ek)


def test_negative_position_keeps_that_tokens_sentinels(provider, oracle):
    """rope.rs: negative_position_guard_preserves_output_sentinels.  The guard is per token
    (crates/loom-infer-cuda/src/rope/mod.rs:64-67): the other tokens are still rotated."""
    spec = lk.Bf16RopePosIdsSpec.new(3, 4, 2)
    rng = np.random.default_rng(3)
    q = H.normal_bf16(rng, spec.query_numel())
    k = H.normal_bf16(rng, spec.key_numel())
    aq, ak = run(provider, spec, q, k, [5, -1, 9], sentinel=-7.0)
    sentinel = H.host_bits(torch.tensor([-7.0], dtype=torch.bfloat16))[0]
    assert np.all(aq[4 * 128:8 * 128] == sentinel) and np.all(ak[2 * 128:4 * 128] == sentinel)
    eq, ek = oracle.rope(3, 4, 2, q, k, [5, 0, 9])
    for lo, hi, actual, expected in ((0, 4 * 128, aq, eq), (8 * 128, 12 * 128, aq, eq),
                                     (0, 2 * 128, ak, ek), (4 * 128, 6 * 128, ak, ek)):
        assert within_one_ulp(actual[lo:hi], expected[lo:hi])


def test_short_buffer_and_partial_rotary_are_rejected_before_submission(provider):
    spec = lk.Bf16RopePosIdsSpec.new(5, 16, 4)
    plan = provider.plan_bf16_pos_ids(spec)
    queue = lk.CommandQueue(torch.cuda.Stream(), 1)
    b = queue.bindings(5)
    q = b.bind_read(torch.zeros(spec.query_numel() - 1, dtype=torch.bfloat16, device="cuda:0"))
    k = b.bind_read(torch.zeros(spec.key_numel(), dtype=torch.bfloat16, device="cuda:0"))
    p = b.bind_read(torch.zeros(5, dtype=torch.int32, device="cuda:0"))
    qo = b.bind_read_write(torch.zeros(spec.query_numel(), dtype=torch.bfloat16, device="cuda:0"))
    ko = b.bind_read_write(torch.zeros(spec.key_numel(), dtype=torch.bfloat16, device="cuda:0"))
    scope = queue.begin(b)
    with pytest.raises(lk.EnqueueError) as e:
        plan.enqueue_into(scope, lk.Bf16RopePosIdsArgs(q, k, p, qo.write(), ko.write()))
    assert (e.value.variant, e.value.operand) == ("LengthMismatch", "query")
    assert scope.finish().submitted() == 0
    with pytest.raises(lk.LoomError) as e:
        provider.plan_bf16_pos_ids(lk.Bf16RopePosIdsSpec.new(5, 16, 4, 128, 64))
    assert e.value.variant == "UnsupportedRotaryDimension"
