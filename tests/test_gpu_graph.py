"""Fixed-address CUDA Graph capture of the append -> decode chain on a real device.

Follows the graph gate crates/loom-infer-validation/src/gates/rope.rs:693-853 of the reference:
capture once, drop every external owner, replay twice (one waited, one dropped), and read the
buffers back through the returned bindings.  Per-step variation travels only through the
contents of the bound buffers.
"""
import gc

import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("merge_in_kernel", [0, 1])
def test_append_then_decode_graph_replays(oracle, merge_in_kernel):
    # the split decode in both forms: merged by a second command, or by the last CTA of an item
    # (its counting words belong to the Graph's own queue and are zero again after every replay)
    rng = np.random.default_rng(21)
    batch, qh, kvh, pool = 3, 16, 4, 64
    kv_lens = np.array([40, 16, 97])
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool)
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pool, qh, kvh)
    ospec = oracle.paged_spec(batch, pool, qh, kvh)
    k_pages, v_pages = (H.normal_bf16(rng, spec.kv_pages_numel()) for _ in range(2))
    q, k, v = (H.normal_bf16(rng, batch * heads * 128) for heads in (qh, kvh, kvh))

    rope = lk.RopeProvider.load(0)
    decode = lk.DecodeProvider.load(0)
    append_plan = rope.plan_bf16_paged_append(lk.Bf16RopePagedKvAppendSpec.new(batch, pool, qh, kvh))
    decode_plan = decode.plan_bf16_paged_batch(spec, partitions=2, merge_in_kernel=merge_in_kernel)
    tensors = dict(q=H.dev_bf16(q), k=H.dev_bf16(k), v=H.dev_bf16(v), indptr=H.dev_i32(indptr),
                   indices=H.dev_i32(indices), last=H.dev_i32(last))
    q_rot = torch.full((q.size,), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    kp, vp = H.dev_bf16(k_pages), H.dev_bf16(v_pages)
    out = torch.full((q.size,), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    lse = torch.full((batch * qh,), float("nan"), dtype=torch.float32, device="cuda:0")
    workspace = torch.zeros(decode_plan.workspace_required_numel(), dtype=torch.float32, device="cuda:0")
    torch.cuda.synchronize()

    graph_queue = lk.GraphQueue(0, 3)
    b = graph_queue.bindings(12)
    r = {name: b.bind_read(t) for name, t in tensors.items()}
    h_qrot, h_kp, h_vp = b.bind_read_write(q_rot), b.bind_read_write(kp), b.bind_read_write(vp)
    h_out, h_lse, h_ws = b.bind_read_write(out), b.bind_read_write(lse), b.bind_read_write(workspace)

    def record(scope):
        append_plan.enqueue_into(scope, lk.Bf16RopePagedKvAppendArgs(
            r["q"], r["k"], r["v"], r["indptr"], r["indices"], r["last"], h_qrot.write(),
            h_kp.write(), h_vp.write()))
        decode_plan.enqueue_into(scope, lk.Bf16PagedBatchDecodeArgs(
            h_qrot.read(), h_kp.read(), h_vp.read(), r["indptr"], r["indices"], r["last"],
            h_out.write(), h_lse.write(), h_ws))

    captured = graph_queue.capture(b, record)
    # append + partials (+ merge)
    assert captured.commands() == (2 if merge_in_kernel == 1 else 3)
    # nothing ran during capture
    assert torch.isnan(out.float()).all()
    exec_ = captured.instantiate()
    del append_plan, decode_plan, rope, captured  # the executable owns what it needs
    gc.collect()

    eq, ekp, evp = oracle.rope_append(ospec, q, k, v, indptr, indices, last, k_pages, v_pages)

    completion = exec_.launch()
    assert completion.launch_index() == 1
    with pytest.raises(lk.GraphError) as e:
        exec_.launch()
    assert e.value.variant == "ReplayInFlight"
    completion.wait()
    first = H.host_bits(out)
    # second replay with new query/key/value CONTENTS at the same addresses
    q2, k2, v2 = (H.normal_bf16(rng, batch * heads * 128) for heads in (qh, kvh, kvh))
    tensors["q"].copy_(H.dev_bf16(q2))
    tensors["k"].copy_(H.dev_bf16(k2))
    tensors["v"].copy_(H.dev_bf16(v2))
    torch.cuda.synchronize()
    dropped = exec_.launch()
    del dropped  # dropping the completion settles the replay
    assert exec_.launches() == 2
    assert exec_.measure_launch_ms() > 0.0
    bindings = exec_.into_bindings()
    out_t, lse_t = bindings.take_read_write(h_out), bindings.take_read_write(h_lse)
    kp_t, vp_t = bindings.take_read_write(h_kp), bindings.take_read_write(h_vp)
    assert decode.device_status() == 0

    kp1 = ekp  # after replay 1
    eo1, el1 = oracle.paged_decode(ospec, eq, kp1, evp, indptr, indices, last)
    assert np.abs(H.bits_to_f32(first) - H.bits_to_f32(eo1)).max() <= H.DECODE_MAX_ABS
    eq2, ekp2, evp2 = oracle.rope_append(ospec, q2, k2, v2, indptr, indices, last, ekp, evp)
    assert np.array_equal(H.host_bits(vp_t), evp2)
    kp_bits = H.host_bits(kp_t)
    assert np.abs(H.bits_to_f32(kp_bits) - H.bits_to_f32(ekp2)).max() <= 2.0 ** -6
    eo2, el2 = oracle.paged_decode(ospec, eq2, kp_bits, evp2, indptr, indices, last)
    H.check_decode(H.host_bits(out_t), lse_t.cpu().numpy(), eo2, el2, lse_limit=5e-3)


def test_graph_rejects_an_empty_capture_and_keeps_the_device_usable():
    graph_queue = lk.GraphQueue(0, 1)
    b = graph_queue.bindings(1)
    b.bind_read(torch.zeros(4, device="cuda:0"))
    with pytest.raises(lk.GraphError) as e:
        graph_queue.capture(b, lambda scope: None)
    assert e.value.variant == "EmptyCapture"
    assert float(torch.ones(4, device="cuda:0").sum()) == 4.0
