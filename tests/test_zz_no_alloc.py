"""The split-K decode entry point for hosts that cannot allocate device memory.

Some hosts of this library are handed device pointers but may not create any themselves: a plug-in
inside an engine that claimed all device memory for its own pool and forbids cudaMalloc, or a loop
that must never enter the allocator.  They cannot bind the workspace a split plan needs, so
`lb_paged_decode_split_noalloc` keeps the partial states in a fixed array inside the library.  This
file checks, through the C ABI, that it gives what the workspace-based entry point gives, on two
calls in a row (the second finds the first call's states in the shared array), and that a request
larger than the array is refused before anything is launched.

Collected last on purpose: a failure here must not hide the result of any other test.
"""
import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from loom_kernels_b200 import _abi
from tests import helpers as H

pytestmark = pytest.mark.gpu


def run_both(oracle, rng, batch, qh, kvh, pool, kv_lens, partitions):
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool)
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pool, qh, kvh)
    q, k, v = (H.normal_bf16(rng, n) for n in (spec.query_numel(), spec.kv_pages_numel(),
                                               spec.kv_pages_numel()))
    # the existing entry point: split plan + caller-owned workspace
    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, partitions=partitions)
    expected_out, expected_lse = run.run()
    # the new entry point: same device inputs, raw pointers, no workspace
    out = torch.full((spec.output_numel(),), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    lse = torch.full((spec.lse_numel(),), float("nan"), dtype=torch.float32, device="cuda:0")
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    lk.paged_decode_split_noalloc(spec, partitions, stream, run.q, run.k, run.v, run.indptr,
                                  run.indices, run.last, out, lse)
    stream.synchronize()
    actual_out, actual_lse = H.host_bits(out), lse.cpu().numpy()
    # same kernels, same partition rule: the two entry points agree to the bit ...
    assert np.array_equal(actual_out, expected_out)
    assert np.array_equal(actual_lse.view(np.uint32), expected_lse.view(np.uint32))
    # ... and both are within the decode tolerances of the CPU reference
    eo, el = oracle.paged_decode(oracle.paged_spec(batch, pool, qh, kvh), q, k, v, indptr,
                                 indices, last, threads=4)
    H.check_decode(actual_out, actual_lse, eo, el, lse_limit=H.SPLIT_LSE_MAX_ABS)


def test_noalloc_entry_matches_the_workspace_entry_on_two_calls_in_a_row(oracle):
    rng = np.random.default_rng(2024)
    # first call: GQA4, ragged, one request with fewer pages than partitions (empty chunks)
    run_both(oracle, rng, 3, 32, 8, 80, [16 * 20 + 5, 16 * 2, 16 * 33], partitions=4)
    # second call right after it, another shape: it finds the first call's states in the array
    run_both(oracle, rng, 2, 64, 8, 96, [16 * 40, 16 * 37 + 9], partitions=8)
    # no CTA of either call gave up on a bounded wait (the entry point's own status word)
    assert lk.paged_decode_split_noalloc_status(0) == 0


def test_noalloc_entry_refuses_what_the_static_array_cannot_hold():
    limit = lk.paged_decode_split_noalloc_max_states()
    assert limit == 16384
    spec = lk.Bf16PagedBatchDecodeSpec.new(64, 4096, 32, 8)  # 64*32*16 = 32768 states
    dummy = torch.zeros(16, dtype=torch.bfloat16, device="cuda:0")
    ints = torch.zeros(128, dtype=torch.int32, device="cuda:0")
    lse = torch.zeros(16, dtype=torch.float32, device="cuda:0")
    before = _abi.load().lb_test_launch_count()
    with pytest.raises(lk.LoomError) as info:
        lk.paged_decode_split_noalloc(spec, 16, torch.cuda.current_stream(), dummy, dummy, dummy,
                                      ints, ints, ints, dummy, lse)
    assert info.value.variant == "StaticScratchExceeded"
    assert info.value.payload[:2] == (64 * 32 * 16 * 130, limit * 130)
    assert _abi.load().lb_test_launch_count() == before
    with pytest.raises(lk.ContractError) as info:  # it is the split variant: one chunk is refused
        lk.paged_decode_split_noalloc(spec, 1, torch.cuda.current_stream(), dummy, dummy, dummy,
                                      ints, ints, ints, dummy, lse)
    assert info.value.variant == "InvalidPartitionCount"
    # a request that fits is checked operand by operand before anything is launched
    small = lk.Bf16PagedBatchDecodeSpec.new(2, 8, 32, 8)
    with pytest.raises(lk.EnqueueError) as info:
        lk.paged_decode_split_noalloc(small, 2, torch.cuda.current_stream(), dummy, dummy, dummy,
                                      ints, ints, ints, dummy, lse)
    assert (info.value.variant, info.value.operand) == ("LengthMismatch", "Q")
    assert _abi.load().lb_test_launch_count() == before
