"""The `indices_capacity` plan option: `page_indices` bound longer than the table in use, so that
one fixed-address Graph of [append newest token, decode] serves steps whose total page count
differs (no reference counterpart: the reference ties a Graph to one page count through the
guard page_indptr[batch] == page_indices.len(), crates/loom-infer-cuda/src/attention/
decode.rs:239-240).

Each step rewrites only the CONTENTS of the bound metadata and token buffers; results are
checked against the CPU oracle run on exactly the table in use.
"""
import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from tests import helpers as H
from tests.test_gpu_rope_append import within_one_ulp

pytestmark = pytest.mark.gpu
BATCH, QH, KVH, POOL, CAPACITY = 4, 16, 4, 96, 64


def table_for(rng, kv_lens, taken):
    """Page table over pages not in `taken`; returns (indptr, indices, last)."""
    pages = [(int(n) + 15) // 16 for n in kv_lens]
    free = np.array(sorted(set(range(POOL)) - set(taken)))
    ids = rng.permutation(free)[:sum(pages)].astype(np.int32)
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    last = np.array([(int(n) - 1) % 16 + 1 for n in kv_lens], dtype=np.int32)
    return indptr, ids, last


@pytest.mark.parametrize("decode_options", [dict(partitions=1), dict(partitions=3),
                                            dict(balanced=1)])
def test_one_graph_serves_steps_with_different_page_counts(oracle, decode_options):
    rng = np.random.default_rng(5)
    rope, decode = lk.RopeProvider.load(0), lk.DecodeProvider.load(0)
    spec = lk.Bf16PagedBatchDecodeSpec.new(BATCH, POOL, QH, KVH)
    ospec = oracle.paged_spec(BATCH, POOL, QH, KVH)
    append_plan = rope.plan_bf16_paged_append(
        lk.Bf16RopePagedKvAppendSpec.new(BATCH, POOL, QH, KVH), indices_capacity=True)
    decode_plan = decode.plan_bf16_paged_batch(spec, indices_capacity=True, **decode_options)

    k_pages, v_pages = (H.normal_bf16(rng, spec.kv_pages_numel()) for _ in range(2))
    dev = dict(q=torch.zeros(BATCH * QH * 128, dtype=torch.bfloat16, device="cuda:0"),
               k=torch.zeros(BATCH * KVH * 128, dtype=torch.bfloat16, device="cuda:0"),
               v=torch.zeros(BATCH * KVH * 128, dtype=torch.bfloat16, device="cuda:0"),
               indptr=torch.zeros(BATCH + 1, dtype=torch.int32, device="cuda:0"),
               indices=torch.full((CAPACITY,), -1, dtype=torch.int32, device="cuda:0"),
               last=torch.zeros(BATCH, dtype=torch.int32, device="cuda:0"))
    q_rot = torch.zeros(BATCH * QH * 128, dtype=torch.bfloat16, device="cuda:0")
    kp, vp = H.dev_bf16(k_pages), H.dev_bf16(v_pages)
    out = torch.zeros(spec.output_numel(), dtype=torch.bfloat16, device="cuda:0")
    lse = torch.zeros(spec.lse_numel(), dtype=torch.float32, device="cuda:0")
    numel = decode_plan.workspace_required_numel()
    workspace = torch.zeros(numel, dtype=torch.float32, device="cuda:0") if numel else None

    graph_queue = lk.GraphQueue(0, 1 + decode_plan.commands())
    b = graph_queue.bindings(12)
    r = {name: b.bind_read(t) for name, t in dev.items()}
    h_qrot, h_kp, h_vp = b.bind_read_write(q_rot), b.bind_read_write(kp), b.bind_read_write(vp)
    h_out, h_lse = b.bind_read_write(out), b.bind_read_write(lse)
    h_ws = b.bind_read_write(workspace) if workspace is not None else None

    def record(scope):
        append_plan.enqueue_into(scope, lk.Bf16RopePagedKvAppendArgs(
            r["q"], r["k"], r["v"], r["indptr"], r["indices"], r["last"], h_qrot.write(),
            h_kp.write(), h_vp.write()))
        decode_plan.enqueue_into(scope, lk.Bf16PagedBatchDecodeArgs(
            h_qrot.read(), h_kp.read(), h_vp.read(), r["indptr"], r["indices"], r["last"],
            h_out.write(), h_lse.write(), h_ws))

    exec_ = graph_queue.capture(b, record).instantiate()
    host_k, host_v = k_pages.copy(), v_pages.copy()
    for kv_lens in ([40, 16, 97, 5], [41, 17, 98, 6], [300, 1, 33, 64], [16, 16, 16, 16]):
        indptr, indices, last = table_for(rng, kv_lens, ())
        assert len(indices) <= CAPACITY
        q, k, v = (H.normal_bf16(rng, BATCH * heads * 128) for heads in (QH, KVH, KVH))
        padded = np.full(CAPACITY, -1, dtype=np.int32)  # the tail past the table is never read
        padded[:len(indices)] = indices
        for name, array in (("indptr", indptr), ("indices", padded), ("last", last)):
            dev[name].copy_(torch.from_numpy(array))
        for name, bits in (("q", q), ("k", k), ("v", v)):
            dev[name].copy_(H.dev_bf16(bits))
        torch.cuda.synchronize()
        exec_.launch().wait()
        assert decode.device_status() == 0
        eq, host_k, host_v = oracle.rope_append(ospec, q, k, v, indptr, indices, last, host_k,
                                                host_v)
        assert np.array_equal(H.host_bits(vp), host_v), "V pages differ"
        assert within_one_ulp(H.host_bits(kp), host_k) and within_one_ulp(H.host_bits(q_rot), eq)
        # decode is checked on exactly what the device decoded from; the pools carry over
        host_k = H.host_bits(kp)
        eo, el = oracle.paged_decode(ospec, H.host_bits(q_rot), host_k, host_v, indptr, indices,
                                     last)
        H.check_decode(H.host_bits(out), lse.cpu().numpy(), eo, el, lse_limit=1e-3)
    exec_.into_bindings()


def test_the_reference_rule_still_holds_without_the_option():
    """Without the option a table shorter than the bound page_indices is invalid metadata: the
    decode writes nothing (sentinels stay)."""
    rng = np.random.default_rng(8)
    spec = lk.Bf16PagedBatchDecodeSpec.new(BATCH, POOL, QH, KVH)
    indptr, indices, last = table_for(rng, [40, 16, 97, 5], ())
    padded = np.concatenate([indices, np.zeros(7, np.int32)])
    run = H.DecodeRun(spec, H.normal_bf16(rng, spec.query_numel()),
                      H.normal_bf16(rng, spec.kv_pages_numel()),
                      H.normal_bf16(rng, spec.kv_pages_numel()), indptr, padded, last,
                      partitions=1)
    out, lse = run.run()
    assert np.all(np.isnan(H.bits_to_f32(out))) and np.all(np.isnan(lse))


@pytest.mark.parametrize("algorithm,partitions", [(1, 1), (2, 1), (2, 3)])
def test_prefill_accepts_a_longer_page_indices_binding(oracle, algorithm, partitions):
    """The same option on the prefill plans (token-parallel, tiled, tiled with split KV): the table
    in use may be shorter than the bound page_indices (the tail is never read); without the
    option such a call writes nothing."""
    rng = np.random.default_rng(12)
    qo_lens, kv_lens = [37, 5, 70], [90, 200, 70]
    qo_indptr = np.concatenate([[0], np.cumsum(qo_lens)]).astype(np.int32)
    indptr, indices, last = table_for(rng, kv_lens, ())
    padded = np.concatenate([indices, np.full(11, -1, np.int32)])
    nnz = int(qo_indptr[-1])
    spec = lk.Bf16PagedPrefillSpec.new(3, nnz, POOL, QH, KVH)
    q = H.normal_bf16(rng, spec.query_numel())
    k, v = (H.normal_bf16(rng, spec.kv_pages_numel()) for _ in range(2))
    expected, expected_lse = oracle.paged_prefill(oracle.prefill_spec(3, nnz, POOL, QH, KVH), q, k, v,
                                                  qo_indptr, indptr, indices, last, threads=4)
    provider = lk.PrefillProvider.load(0)
    for capacity in (True, False):
        plan = provider.plan_bf16_paged(spec, algorithm=algorithm, indices_capacity=capacity,
                                        partitions=partitions)
        workspace = torch.zeros(plan.workspace_required_numel(), dtype=torch.float32,
                                device="cuda:0") if plan.workspace_required_numel() else None
        out = torch.full((spec.output_numel(),), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        lse = torch.full((spec.lse_numel(),), float("nan"), dtype=torch.float32, device="cuda:0")
        tensors = [H.dev_bf16(q), H.dev_bf16(k), H.dev_bf16(v), H.dev_i32(qo_indptr),
                   H.dev_i32(indptr), H.dev_i32(padded), H.dev_i32(last)]
        torch.cuda.synchronize()
        queue = lk.CommandQueue(torch.cuda.Stream(), 2)
        b = queue.bindings(10)
        reads = [b.bind_read(t) for t in tensors]
        h_out, h_lse = b.bind_read_write(out), b.bind_read_write(lse)
        h_ws = b.bind_read_write(workspace) if workspace is not None else None
        scope = queue.begin(b)
        plan.enqueue_into(scope, lk.Bf16PagedPrefillArgs(*reads, h_out.write(), h_lse.write(),
                                                         h_ws))
        scope.finish().wait()
        assert provider.device_status() == 0
        if capacity:
            H.check_decode(H.host_bits(out), lse.cpu().numpy(), expected, expected_lse,
                           lse_limit=1e-3, large_outputs=True)
        else:
            assert np.all(np.isnan(lse.cpu().numpy()))
