"""One process per GPU (run under torch.distributed.run by tests/test_gpu_peer_gather.py): a ragged
batch split by request over the ranks, every rank's rows stored into every rank's copy of the
gathered result by the decode kernels themselves, for the direct, split-K and balanced plans, and
one request split by KV head.  No host barrier separates a rank's fence from its check: the
command completes only when every rank's rows have arrived."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import loom_kernels_b200 as lk  # noqa: E402
from loom_kernels_b200 import sharding  # noqa: E402
from tests import helpers as H  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(device))
    group = lk.PeerGroup.from_torch_distributed(local)
    provider = lk.DecodeProvider.load(local)
    rng = np.random.default_rng(77)  # the same draw on every rank
    batch, qh, kvh, pool = 11, 32, 8, 256
    kv_lens = rng.integers(1, 16 * 40, size=batch)
    assignment = sharding.balanced_assignment(kv_lens, world)
    owned = assignment[rank]
    spec = lk.Bf16PagedBatchDecodeSpec.new(len(owned), pool, qh, kvh)
    local_rng = np.random.default_rng(1000 + rank)
    indptr, indices, last = H.make_page_table(local_rng, kv_lens[owned], pool)
    q, k, v = (H.normal_bf16(local_rng, n) for n in (spec.query_numel(), spec.kv_pages_numel(),
                                                     spec.kv_pages_numel()))
    g_out = [group.buffer(batch * qh * 128, lk.BF16) for _ in range(2)]
    g_lse = [group.buffer(batch * qh, lk.F32) for _ in range(2)]
    step = 0
    for options in ({"partitions": 1}, {"partitions": 3}, {"partitions": 3, "merge_in_kernel": 1},
                    {"balanced": 1, "merge_in_kernel": 2}, {"balanced": 1, "merge_in_kernel": 1}):
        run = H.DecodeRun(spec, q, k, v, indptr, indices, last, device=device, provider=provider,
                          max_commands=4, **options)
        plain_out, plain_lse = run.run()
        for _ in range(3):
            which = step % 2
            step += 1
            b = run.bind_extra(3)
            h_out, h_lse = (b.bind_read_write(g_out[which].span),
                            b.bind_read_write(g_lse[which].span))
            rows = b.bind_read(H.dev_i32(owned.astype(np.int32), device))
            scope = run.queue.begin(b)
            args = lk.Bf16PagedBatchDecodeArgs(output=h_out.write(), lse=h_lse.write(),
                                               workspace=run.h_ws, **run.h)
            run.plan.enqueue_gathered_into(scope, args, rows, group, g_out[which], g_lse[which],
                                           batch)
            scope.finish().wait()
            assert provider.device_status() == 0
            got = H.host_bits(g_out[which].tensor(device)).reshape(batch, qh * 128)
            got_lse = g_lse[which].tensor(device).cpu().numpy().reshape(batch, qh)
            # every rank's plain rows, exchanged on the host side of torch.distributed
            everyone = [None] * world
            dist.all_gather_object(everyone, (owned, plain_out, plain_lse))
            for ids, out, lse in everyone:
                assert np.array_equal(got[ids].reshape(-1), out), (rank, options)
                assert np.array_equal(got_lse[ids].reshape(-1).view(np.uint32), lse.view(np.uint32))

    # two gathering commands in one step: the first only stores and fences its rows, the second
    # publishes the epoch and waits, and its completion covers the rows of both
    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, device=device, provider=provider,
                      max_commands=4, balanced=1)
    plain_out, plain_lse = run.run()
    for buffer in g_out:
        buffer.tensor(device).zero_()
    torch.cuda.synchronize()
    dist.barrier()
    b = run.bind_extra(5)
    handles = [(b.bind_read_write(g_out[i].span), b.bind_read_write(g_lse[i].span)) for i in (0, 1)]
    rows = b.bind_read(H.dev_i32(owned.astype(np.int32), device))
    scope = run.queue.begin(b)
    for i, (h_out, h_lse) in enumerate(handles):
        args = lk.Bf16PagedBatchDecodeArgs(output=h_out.write(), lse=h_lse.write(),
                                           workspace=run.h_ws, **run.h)
        run.plan.enqueue_gathered_into(scope, args, rows, group, g_out[i], g_lse[i], batch,
                                       defer_wait=i == 0)
    scope.finish().wait()
    assert provider.device_status() == 0
    everyone = [None] * world
    dist.all_gather_object(everyone, (owned, plain_out))
    for i in (0, 1):
        got = H.host_bits(g_out[i].tensor(device)).reshape(batch, qh * 128)
        for ids, out in everyone:
            assert np.array_equal(got[ids].reshape(-1), out), (rank, "deferred", i)

    # one request split by KV head: every rank computes qh / world heads of the same request
    if kvh % world == 0:
        kv_lo, kv_hi, q_lo, q_hi = sharding.kv_head_range(kvh, qh, world, rank)
        one_rng = np.random.default_rng(5)
        indptr, indices, last = H.make_page_table(one_rng, [16 * 30 + 7], pool)
        full_spec = lk.Bf16PagedBatchDecodeSpec.new(1, pool, qh, kvh)
        fq, fk, fv = (H.normal_bf16(one_rng, n) for n in (full_spec.query_numel(),
                                                          full_spec.kv_pages_numel(),
                                                          full_spec.kv_pages_numel()))
        whole = H.DecodeRun(full_spec, fq, fk, fv, indptr, indices, last, device=device,
                            provider=provider, partitions=1, heads_per_cta=2)
        whole_out, whole_lse = whole.run()
        part_spec = lk.Bf16PagedBatchDecodeSpec.new(1, pool, q_hi - q_lo, kv_hi - kv_lo)
        pq = np.ascontiguousarray(fq.reshape(1, qh, 128)[:, q_lo:q_hi]).reshape(-1)
        pk, pv = (np.ascontiguousarray(x.reshape(pool, 16, kvh, 128)[:, :, kv_lo:kv_hi]).reshape(-1)
                  for x in (fk, fv))
        run = H.DecodeRun(part_spec, pq, pk, pv, indptr, indices, last, device=device,
                          provider=provider, max_commands=4, partitions=1, heads_per_cta=2)
        h_out_buf, h_lse_buf = group.buffer(qh * 128, lk.BF16), group.buffer(qh, lk.F32)
        b = run.bind_extra(3)
        h_out, h_lse = b.bind_read_write(h_out_buf.span), b.bind_read_write(h_lse_buf.span)
        rows = b.bind_read(H.dev_i32([0], device))
        scope = run.queue.begin(b)
        args = lk.Bf16PagedBatchDecodeArgs(output=h_out.write(), lse=h_lse.write(),
                                           workspace=run.h_ws, **run.h)
        run.plan.enqueue_gathered_into(scope, args, rows, group, h_out_buf, h_lse_buf, 1, qh, q_lo)
        scope.finish().wait()
        assert provider.device_status() == 0
        # the same plan shape (two KV heads per CTA) on 8 heads and on 8 / world heads: per-head
        # arithmetic is identical, so the gathered heads equal the unsharded result to the bit
        assert np.array_equal(H.host_bits(h_out_buf.tensor(device)), whole_out)
        assert np.array_equal(h_lse_buf.tensor(device).cpu().numpy().view(np.uint32),
                              whole_lse.view(np.uint32))

    torch.cuda.synchronize()
    dist.barrier()
    group.close()
    if rank == 0:
        print(f"peer gather ok on {world} ranks", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
