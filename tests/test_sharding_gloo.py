"""Multi-rank host logic on CPU (gloo, world size 2): request sharding with pool-local page ids,
KV-head sharding, the ragged balanced assignment, and the all-gather of output rows.  The decode
itself is stood in for by the CPU oracle (no GPU here); what is under test is the partitioning
and the collective plumbing."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from loom_kernels_b200 import sharding


def test_request_ranges_and_partition_choice():
    assert [sharding.request_range(64, 8, r) for r in (0, 7)] == [(0, 8), (56, 64)]
    assert [sharding.request_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert sharding.choose_partition(512, 8, 8) == "request"
    assert sharding.choose_partition(1, 32, 8) == "kv_head"
    assert sharding.choose_partition(1, 1, 8) == "replicas"
    assert sharding.kv_head_range(32, 32, 8, 3) == (12, 16, 12, 16)
    assert sharding.kv_head_range(8, 32, 2, 1) == (4, 8, 16, 32)
    with pytest.raises(ValueError):
        sharding.kv_head_range(1, 32, 8, 0)


def test_balanced_assignment_and_unpermute():
    rng = np.random.default_rng(0xC5)
    lens = np.floor(np.exp(rng.uniform(np.log(128), np.log(16384), 512))).astype(np.int64)
    owned = sharding.balanced_assignment(lens, 8)
    assert sorted(np.concatenate(owned).tolist()) == list(range(512))
    loads = np.array([lens[ids].sum() for ids in owned])
    assert loads.max() / loads.mean() < 1.01  # contiguous ranges would be off by far more
    rows = np.arange(512)[np.concatenate(owned)]
    assert np.array_equal(sharding.unpermute_rows(rows, owned), np.arange(512))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, result_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle
        rng = np.random.default_rng(99)
        batch, qh, kvh, pool = 5, 8, 2, 40
        kv_lens = np.array([70, 16, 33, 120, 5])
        pages = (kv_lens + 15) // 16
        indices = rng.permutation(pool)[:pages.sum()].astype(np.int32)
        indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
        last = ((kv_lens - 1) % 16 + 1).astype(np.int32)
        q = oracle.fixture_bf16(batch * qh * 128, 1)
        k = oracle.fixture_bf16(pool * 16 * kvh * 128, 2)
        v = oracle.fixture_bf16(pool * 16 * kvh * 128, 3)
        full_o, full_lse = oracle.paged_decode(oracle.paged_spec(batch, pool, qh, kvh), q, k, v,
                                               indptr, indices, last)
        if mode == "request":
            shard = sharding.shard_by_request(indptr, indices, last, world, rank)
            n = shard.hi - shard.lo
            # the rank's own pool holds only its pages, under local ids
            kr = k.reshape(pool, -1)[shard.global_pages].ravel()
            vr = v.reshape(pool, -1)[shard.global_pages].ravel()
            o, lse = oracle.paged_decode(
                oracle.paged_spec(n, len(shard.global_pages), qh, kvh),
                q[shard.lo * qh * 128:shard.hi * qh * 128], kr, vr, shard.indptr, shard.indices,
                shard.last)
            counts = [hi - lo for lo, hi in (sharding.request_range(batch, world, r)
                                             for r in range(world))]
            rows = torch.from_numpy(o.view(np.uint8).reshape(n, qh * 256).copy())  # gloo has no int16
            gathered = sharding.gather_output_rows(rows, counts)
            got = gathered.numpy().view(np.uint16).ravel()
            lse_all = sharding.gather_output_rows(torch.from_numpy(lse.reshape(n, qh).copy()), counts)
            ok = np.array_equal(got, full_o) and np.array_equal(lse_all.numpy().ravel(), full_lse)
        else:
            kv_lo, kv_hi, q_lo, q_hi = sharding.kv_head_range(kvh, qh, world, rank)
            heads = kv_hi - kv_lo
            kr = k.reshape(pool * 16, kvh, 128)[:, kv_lo:kv_hi].ravel()
            vr = v.reshape(pool * 16, kvh, 128)[:, kv_lo:kv_hi].ravel()
            qr = q.reshape(batch, qh, 128)[:, q_lo:q_hi].ravel()
            o, _ = oracle.paged_decode(oracle.paged_spec(batch, pool, q_hi - q_lo, heads), qr, kr,
                                       vr, indptr, indices, last)
            rows = torch.from_numpy(o.view(np.uint8).reshape(1, -1).copy())
            gathered = sharding.gather_output_rows(rows)  # [world, batch*(qh/world)*128]
            got = gathered.numpy().view(np.uint16).reshape(world, batch, (q_hi - q_lo) * 128)
            got = np.transpose(got, (1, 0, 2)).ravel()
            ok = np.array_equal(got, full_o)
        result_queue.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def _prefill_worker(rank, world, port, result_queue):
    """A ragged prefill batch split by request over two ranks (weights: causal pairs): each rank
    runs its sub-batch on its own pool with local page ids; the gathered query rows, put back in
    batch order, equal the unsharded result bit for bit."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle
        rng = np.random.default_rng(123)
        qh, kvh, pool = 8, 2, 64
        qo_lens = np.array([9, 1, 40, 3, 17])
        kv_lens = np.array([70, 16, 40, 120, 33])
        pages = (kv_lens + 15) // 16
        indices = rng.permutation(pool)[:pages.sum()].astype(np.int32)
        indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
        qo_indptr = np.concatenate([[0], np.cumsum(qo_lens)]).astype(np.int32)
        last = ((kv_lens - 1) % 16 + 1).astype(np.int32)
        nnz = int(qo_indptr[-1])
        q = oracle.fixture_bf16(nnz * qh * 128, 1)
        k = oracle.fixture_bf16(pool * 16 * kvh * 128, 2)
        v = oracle.fixture_bf16(pool * 16 * kvh * 128, 3)
        full_o, full_lse = oracle.paged_prefill(oracle.prefill_spec(len(qo_lens), nnz, pool, qh, kvh),
                                                q, k, v, qo_indptr, indptr, indices, last)
        owned = sharding.prefill_assignment(qo_lens, kv_lens, world)
        shards = [sharding.shard_prefill(qo_indptr, indptr, indices, last, ids) for ids in owned]
        mine = shards[rank]
        n, rows = len(mine.requests), len(mine.query_rows)
        qr = q.reshape(nnz, qh * 128)[mine.query_rows].ravel()
        kr = k.reshape(pool, -1)[mine.global_pages].ravel()
        vr = v.reshape(pool, -1)[mine.global_pages].ravel()
        o, lse = oracle.paged_prefill(
            oracle.prefill_spec(n, rows, len(mine.global_pages), qh, kvh), qr, kr, vr,
            mine.qo_indptr, mine.indptr, mine.indices, mine.last)
        counts = [len(s.query_rows) for s in shards]
        gathered = sharding.gather_output_rows(
            torch.from_numpy(o.view(np.uint8).reshape(rows, qh * 256).copy()), counts)
        got = sharding.unpermute_query_rows(gathered.numpy(), [s.query_rows for s in shards])
        lse_all = sharding.gather_output_rows(torch.from_numpy(lse.reshape(rows, qh).copy()), counts)
        got_lse = sharding.unpermute_query_rows(lse_all.numpy(), [s.query_rows for s in shards])
        ok = (np.array_equal(got.view(np.uint16).ravel(), full_o)
              and np.array_equal(got_lse.ravel(), full_lse)
              and sorted(np.concatenate(owned).tolist()) == list(range(len(qo_lens))))
        result_queue.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_prefill_assignment_balances_causal_pairs():
    qo = np.array([8192, 512, 128, 2048, 64, 4096, 1024, 33])
    kv = np.array([8192, 16384, 16384, 2048, 8192, 4096, 9000, 33])
    owned = sharding.prefill_assignment(qo, kv, 4)
    assert sorted(np.concatenate(owned).tolist()) == list(range(8))
    pairs = qo * (kv - qo) + qo * (qo + 1) // 2
    loads = np.array([pairs[ids].sum() for ids in owned])
    assert loads.max() == pairs.max()  # the longest prompt has a rank to itself
    shard = sharding.shard_prefill(np.concatenate([[0], np.cumsum(qo)]),
                                   np.concatenate([[0], np.cumsum((kv + 15) // 16)]),
                                   np.arange(((kv + 15) // 16).sum()), (kv - 1) % 16 + 1, owned[1])
    assert shard.qo_indptr[-1] == qo[owned[1]].sum() == len(shard.query_rows)
    assert shard.indptr[-1] == len(shard.indices) == len(shard.global_pages)
    assert np.array_equal(shard.global_pages[shard.indices[:3]],
                          np.arange(((kv + 15) // 16).sum())[
                              np.concatenate([[0], np.cumsum((kv + 15) // 16)])[owned[1][0]]:][:3])


def test_two_rank_prefill_sharding_reproduces_the_full_batch(oracle):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_prefill_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = dict(results.get(timeout=5) for _ in range(2))
    assert got == {0: True, 1: True}


def _failing_worker(rank, world, port, result_queue):
    """Rank 1's enqueue fails on the host (a launch failure injected through the fake driver);
    it reports that instead of skipping the collective, and every rank gets ShardFailure."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=30))
    try:
        import loom_kernels_b200 as lk
        from loom_kernels_b200 import _abi
        lib = _abi.load()
        lib.lb_test_use_fake_driver(1, 148)
        spec = lk.Bf16PagedBatchDecodeSpec.new(2, 4, 4, 2)
        plan = lk.DecodeProvider.load(0).plan_bf16_paged_batch(spec, partitions=1)
        queue = lk.CommandQueue(0x100, 1)
        b = queue.bindings(9)
        sizes = [spec.query_numel(), spec.kv_pages_numel(), spec.kv_pages_numel(), 3, 4, 2]
        reads = [b.bind_read(lk.DeviceSpan(0x10000000 + i * 0x1000000, n,
                                           _abi.BF16 if i < 3 else _abi.I32))
                 for i, n in enumerate(sizes)]
        out = b.bind_read_write(lk.DeviceSpan(0x17000000, spec.output_numel(), _abi.BF16))
        lse = b.bind_read_write(lk.DeviceSpan(0x18000000, spec.lse_numel(), _abi.F32))
        if rank == 1:
            lib.lb_test_fake_fail(b"launch", 1, 719)
        scope = queue.begin(b)
        enqueued = True
        try:
            plan.enqueue_into(scope, lk.Bf16PagedBatchDecodeArgs(*reads, out.write(), lse.write()))
        except lk.LoomError:
            enqueued = False
        scope.finish()
        try:
            sharding.gather_output_rows_checked(torch.zeros(2, 8), enqueued)
            outcome = "gathered"
        except sharding.ShardFailure:
            outcome = "shard failure"
        result_queue.put((rank, enqueued, outcome))
        del scope, queue, b, plan
        import gc
        gc.collect()
        lib.lb_test_use_fake_driver(0, 0)
    finally:
        dist.destroy_process_group()


def test_a_failed_rank_stops_the_gather_on_every_rank():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = sorted(results.get(timeout=5) for _ in range(2))
    assert got == [(0, True, "shard failure"), (1, False, "shard failure")]


@pytest.mark.parametrize("mode", ["request", "kv_head"])
def test_two_rank_sharding_reproduces_the_full_batch(mode, oracle):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = dict(results.get(timeout=5) for _ in range(2))
    assert got == {0: True, 1: True}
