"""The give-up path of the kernels' bounded waits, exercised without faulting or hanging the GPU.

Every wait of the decode kernels (a consumer for the bytes of a page, the producer for a free
stage, the last CTA of a gathering command for the other ranks) has a limit.  A test plan lowers
the limit to a millisecond and makes one page's barrier expect more bytes than its copies deliver
(`test_skip_page`), which is all a lost copy would look like: the consumers of that page wait for
bytes that never arrive, give
up, the CTA writes nothing and sets the provider's status word, and the kernel returns by itself.
The next call on the same provider, with a normal plan, must be correct.
"""
import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("partitions", [1, 3])
def test_a_lost_copy_ends_in_a_status_word_not_a_hang(oracle, partitions):
    rng = np.random.default_rng(31)
    batch, qh, kvh, pool = 3, 16, 4, 96
    kv_lens = [16 * 12 + 5, 16 * 9, 16 * 14 + 1]
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool)
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pool, qh, kvh)
    q, k, v = (H.normal_bf16(rng, n) for n in (spec.query_numel(), spec.kv_pages_numel(),
                                               spec.kv_pages_numel()))
    provider = lk.DecodeProvider.load(0)
    assert provider.device_status() == 0

    broken = H.DecodeRun(spec, q, k, v, indptr, indices, last, provider=provider)
    broken.plan = provider.plan_bf16_paged_batch(spec, partitions=partitions, wait_limit_us=1000,
                                                 test_skip_page=2)  # page 1 of every CTA's chunk
    numel = broken.plan.workspace_required_numel()
    broken.workspace = (torch.zeros(numel, dtype=torch.float32, device="cuda:0") if numel else None)
    scope = broken.queue.begin(broken.bind())
    broken.plan.enqueue_into(scope, broken.args())
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record(broken.stream)
    bindings = scope.finish().wait()  # the kernel returns by itself
    end.record(broken.stream)
    end.synchronize()
    assert provider.device_status() == 1  # read and cleared
    assert provider.device_status() == 0
    out = H.bits_to_f32(H.host_bits(bindings.take_read_write(broken.h_out)))
    lse = bindings.take_read_write(broken.h_lse).cpu().numpy()
    if partitions == 1:
        # a CTA that gave up wrote nothing: every request has more than one page, so every CTA
        # lost a copy and every output keeps its sentinel
        assert np.all(np.isnan(out)) and np.all(np.isnan(lse))

    # the provider and the device are as usable as before
    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, provider=provider,
                      partitions=partitions)
    good_out, good_lse = run.run()
    eo, el = oracle.paged_decode(oracle.paged_spec(batch, pool, qh, kvh), q, k, v, indptr, indices,
                                 last, threads=4)
    H.check_decode(good_out, good_lse, eo, el, lse_limit=H.SPLIT_LSE_MAX_ABS)


def test_wait_limit_option_leaves_results_unchanged():
    """A plan with a short limit and nothing skipped gives the bits of the default plan."""
    rng = np.random.default_rng(32)
    batch, qh, kvh, pool = 2, 32, 8, 64
    indptr, indices, last = H.make_page_table(rng, [16 * 20 + 3, 16 * 7], pool)
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pool, qh, kvh)
    q, k, v = (H.normal_bf16(rng, n) for n in (spec.query_numel(), spec.kv_pages_numel(),
                                               spec.kv_pages_numel()))
    provider = lk.DecodeProvider.load(0)
    base = H.DecodeRun(spec, q, k, v, indptr, indices, last, provider=provider, partitions=1).run()
    limited = H.DecodeRun(spec, q, k, v, indptr, indices, last, provider=provider, partitions=1)
    limited.plan = provider.plan_bf16_paged_batch(spec, partitions=1, wait_limit_us=50000)
    got = limited.run()
    assert np.array_equal(base[0], got[0]) and np.array_equal(base[1], got[1])


def test_tiled_prefill_gives_up_without_a_hang(oracle):
    """The tcgen05 prefill kernel: the barrier of every CTA's first K block expects more bytes
    than arrive (`test_lost_copy`), the MMA warp's wait for it runs out after a millisecond, the
    other roles' waits follow, the producer and the MMA warp wait -- bounded again -- for what they
    have in flight, the CTA frees its TMEM and writes nothing; status 1, sentinels kept, and the
    next plan on the same provider is correct."""
    from tests.test_gpu_prefill import PrefillRun, check, ragged_case

    rng = np.random.default_rng(33)
    qh, kvh, pool = 8, 2, 64
    qo_lens, kv_lens = [200, 131], [200, 300]
    q, k, v, qo_indptr, indptr, indices, last = ragged_case(rng, qo_lens, kv_lens, qh, kvh, pool)
    dims = (len(qo_lens), int(qo_indptr[-1]), pool, qh, kvh)
    spec = lk.Bf16PagedPrefillSpec.new(*dims)
    provider = lk.PrefillProvider.load(0)
    assert provider.device_status() == 0

    broken = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last, algorithm=2)
    broken.plan = provider.plan_bf16_paged(spec, algorithm=2, partitions=1, wait_limit_us=1000,
                                           test_lost_copy=True)
    b = broken.queue.bindings(10)
    reads = [b.bind_read(t) for t in broken.tensors]
    h_out, h_lse = b.bind_read_write(broken.out), b.bind_read_write(broken.lse)
    scope = broken.queue.begin(b)
    broken.plan.enqueue_into(scope, lk.Bf16PagedPrefillArgs(*reads, h_out.write(), h_lse.write(),
                                                            None))
    b = scope.finish().wait()  # the kernel returns by itself
    assert provider.device_status() == 1  # read and cleared
    assert provider.device_status() == 0
    out = H.bits_to_f32(H.host_bits(b.take_read_write(h_out)))
    assert np.all(np.isnan(out)) and np.all(np.isnan(b.take_read_write(h_lse).cpu().numpy()))

    # the provider and the device are as usable as before
    good, good_lse = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last,
                                algorithm=2).run()
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(*dims), q, k, v, qo_indptr,
                                                  indptr, indices, last)
    check(good, good_lse, expected, expected_lse, gate=False)
    # and a short limit with nothing lost changes no bit
    limited = PrefillRun(provider, spec, q, k, v, qo_indptr, indptr, indices, last, algorithm=2)
    limited.plan = provider.plan_bf16_paged(spec, algorithm=2, partitions=1, wait_limit_us=50000)
    again, again_lse = limited.run()
    assert np.array_equal(again, good) and np.array_equal(again_lse, good_lse)
