"""Output rows gathered over the ranks of a peer group, through the C ABI.

On one GPU a group of one rank exercises everything but the NVLink hop: the row map
(dest_rows, head offset), the 16-byte row stores of the decode kernels, the merge kernels' row
stores, the CTA count and epoch of the command's last kernel, and the library all-gather recorded
as a command.  With two or more GPUs visible the same checks run as one process per GPU
(tests/peer_gather_ranks.py under torch.distributed.run): every rank's rows, stored by the kernels
of the OTHER ranks, against that rank's own plain result, with no host barrier in between.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from tests import helpers as H

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def group():
    g = lk.PeerGroup(0, 1, 0, lk.PeerGroup.unique_id())
    yield g
    torch.cuda.synchronize()
    g.close()


@pytest.mark.parametrize("options", [{"partitions": 1}, {"partitions": 3}, {"balanced": 1},
                                     {"partitions": 3, "merge_in_kernel": 1},
                                     {"balanced": 1, "merge_in_kernel": 1},
                                     {"partitions": 1, "heads_per_cta": 1}])
@pytest.mark.parametrize("batch,qh,kvh", [(5, 32, 8), (3, 8, 1), (2, 40, 2), (4, 16, 16)])
def test_gathered_rows_equal_the_plain_result(oracle, group, options, batch, qh, kvh):
    rng = np.random.default_rng(batch * 100 + qh + kvh)
    pool = 128
    kv_lens = rng.integers(1, 16 * 20, size=batch)
    kv_lens[0] = 16 * 19 + 3
    indptr, indices, last = H.make_page_table(rng, kv_lens, pool)
    spec = lk.Bf16PagedBatchDecodeSpec.new(batch, pool, qh, kvh)
    q, k, v = (H.normal_bf16(rng, n) for n in (spec.query_numel(), spec.kv_pages_numel(),
                                               spec.kv_pages_numel()))
    run = H.DecodeRun(spec, q, k, v, indptr, indices, last, max_commands=4, **options)
    expected_out, expected_lse = run.run()
    eo, el = oracle.paged_decode(oracle.paged_spec(batch, pool, qh, kvh), q, k, v, indptr, indices,
                                 last, threads=4)
    H.check_decode(expected_out, expected_lse, eo, el, lse_limit=H.SPLIT_LSE_MAX_ABS)

    # the gathered result: 3 more requests than this rank owns, 8 more heads per request than
    # this rank computes, this rank's heads at offset 4; rows in a shuffled order
    total, gathered_qh, head_offset = batch + 3, qh + 8, 4
    dest = rng.permutation(total)[:batch].astype(np.int32)
    g_out = group.buffer(total * gathered_qh * 128, lk.BF16)
    g_lse = group.buffer(total * gathered_qh, lk.F32)
    out_t, lse_t = g_out.tensor("cuda:0"), g_lse.tensor("cuda:0")
    out_t.fill_(float("nan"))
    lse_t.fill_(float("nan"))
    torch.cuda.synchronize()
    for repeat in range(2):  # twice: the CTA counter must be back at zero, the epoch one further
        b = run.bind_extra(3)
        h_out, h_lse = b.bind_read_write(g_out.span), b.bind_read_write(g_lse.span)
        rows = b.bind_read(H.dev_i32(dest))
        scope = run.queue.begin(b)
        args = lk.Bf16PagedBatchDecodeArgs(output=h_out.write(), lse=h_lse.write(),
                                           workspace=run.h_ws, **run.h)
        run.plan.enqueue_gathered_into(scope, args, rows, group, g_out, g_lse, total, gathered_qh,
                                       head_offset)
        completion = scope.finish()
        assert completion.submitted() == run.plan.commands()
        completion.wait()
        assert run.provider.device_status() == 0
        got = H.host_bits(out_t).reshape(total, gathered_qh, 128)
        got_lse = lse_t.cpu().numpy().reshape(total, gathered_qh)
        mine = got[dest, head_offset:head_offset + qh]
        assert np.array_equal(mine.reshape(-1), expected_out)
        assert np.array_equal(got_lse[dest, head_offset:head_offset + qh].reshape(-1).view(np.uint32),
                              expected_lse.view(np.uint32))
        # everything else keeps its sentinel
        mask = np.ones((total, gathered_qh), dtype=bool)
        mask[dest, head_offset:head_offset + qh] = False
        assert np.all(np.isnan(H.bits_to_f32(got[mask].reshape(-1))))
        assert np.all(np.isnan(got_lse[mask]))
    g_out.close()
    g_lse.close()


def test_all_gather_command_of_one_rank(group):
    rows, row_numel = 7, 32 * 128
    stream = torch.cuda.Stream()
    queue = lk.CommandQueue(stream, 2)
    local = torch.randn(rows * row_numel, device="cuda:0").to(torch.bfloat16)
    gathered = torch.zeros_like(local)
    torch.cuda.synchronize()
    plan = lk.OutputGatherPlan(group, lk.BF16, [rows], row_numel)
    b = queue.bindings(2)
    h_local, h_gathered = b.bind_read(local), b.bind_read_write(gathered)
    scope = queue.begin(b)
    plan.enqueue_into(scope, lk.OutputGatherArgs(h_local, h_gathered.write()))
    completion = scope.finish()
    assert completion.submitted() == 1
    completion.wait()
    assert torch.equal(local.view(torch.int16), gathered.view(torch.int16))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_store_into_each_other():
    ranks = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
         "--master-addr", "127.0.0.1", "--master-port", "29631",
         os.path.join(ROOT, "tests", "peer_gather_ranks.py")],
        capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]
    assert f"peer gather ok on {ranks} ranks" in result.stdout
