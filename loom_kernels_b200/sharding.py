"""Multi-GPU partitioning of the paged-decode path (host logic; one process per GPU).

The reference is a single-GPU operator layer with no collective call site
(crates/loom-infer-cuda/src/command/binding.rs:109-123 rejects cross-device buffers).  Attention
over a paged KV cache has no exchange step: every (request, KV head) is independent.  So a batch
is partitioned

  * by request when batch >= GPUs: rank g owns a contiguous range of requests and the pages of
    those requests in its own pool with local page ids; or
  * by KV head when batch < GPUs and the GPU count divides kv_heads: rank g owns a contiguous
    block of KV heads (and their query heads) of every request.

Each rank builds its own spec, plan, queue and bindings; nothing is shared.  When the caller wants
one contiguous result on every rank there are three ways, in order of cost: a gathering decode
command (`Bf16PagedBatchDecodePlan.enqueue_gathered_into` over an `api.PeerGroup`: the kernel that
finishes a row stores it into every rank's result), the all-gather as a command of the same scope
(`api.OutputGatherPlan`, NCCL on the queue's stream), or `gather_output_rows` here, a
`torch.distributed` all-gather after the completion fence.  A ragged prefill batch is
partitioned the same way, by request, with the causal pair count as the weight
(`prefill_assignment`, `shard_prefill`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np


def request_range(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced split: the first batch % world ranks take one extra request."""
    base, rem = divmod(batch, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def choose_partition(batch: int, kv_heads: int, world: int) -> str:
    """'request', 'kv_head', or 'replicas' (nothing to split, e.g. one MQA request)."""
    if world == 1 or batch >= world:
        return "request"
    if kv_heads % world == 0:
        return "kv_head"
    return "replicas"


@dataclass
class RequestShard:
    """The part of a paged batch one rank owns, with pool-local page ids."""
    lo: int
    hi: int
    indptr: np.ndarray        # [hi - lo + 1], starts at 0
    indices: np.ndarray       # local page ids
    last: np.ndarray
    global_pages: np.ndarray  # local id -> page id in the caller's global pool


def shard_by_request(indptr, indices, last, world: int, rank: int) -> RequestShard:
    indptr = np.asarray(indptr, dtype=np.int64)
    batch = len(indptr) - 1
    lo, hi = request_range(batch, world, rank)
    pages = np.asarray(indices)[indptr[lo]:indptr[hi]]
    global_pages, local = np.unique(pages, return_inverse=True)
    return RequestShard(lo, hi, (indptr[lo:hi + 1] - indptr[lo]).astype(np.int32),
                        local.astype(np.int32), np.asarray(last)[lo:hi].astype(np.int32),
                        global_pages.astype(np.int64))


def kv_head_range(kv_heads: int, q_heads: int, world: int, rank: int):
    """(kv_lo, kv_hi, q_lo, q_hi) of the head block rank owns; requires world | kv_heads."""
    if kv_heads % world != 0:
        raise ValueError(f"{world} GPUs do not divide {kv_heads} KV heads")
    per = kv_heads // world
    group = q_heads // kv_heads
    return rank * per, (rank + 1) * per, rank * per * group, (rank + 1) * per * group


def balanced_assignment(kv_lens, world: int) -> List[np.ndarray]:
    """Longest-processing-time assignment of requests to ranks by KV bytes (ragged batches).

    Returns, per rank, the request ids it owns in ascending order.  `unpermute_rows` restores
    request order after a gather."""
    kv_lens = np.asarray(kv_lens, dtype=np.int64)
    order = np.argsort(-kv_lens, kind="stable")
    loads = np.zeros(world, dtype=np.int64)
    owned: List[List[int]] = [[] for _ in range(world)]
    for request in order:
        rank = int(np.argmin(loads))
        owned[rank].append(int(request))
        loads[rank] += kv_lens[request]
    return [np.array(sorted(ids), dtype=np.int64) for ids in owned]


def prefill_assignment(qo_lens, kv_lens, world: int) -> List[np.ndarray]:
    """As balanced_assignment, for a ragged prefill batch: the weight of a request is its number
    of visible (query, key) pairs under the bottom-right causal mask, qo * (kv - qo) +
    qo * (qo + 1) / 2, which is what its attention costs."""
    qo = np.asarray(qo_lens, dtype=np.int64)
    kv = np.asarray(kv_lens, dtype=np.int64)
    return balanced_assignment(qo * (kv - qo) + qo * (qo + 1) // 2, world)


@dataclass
class PrefillShard:
    """The requests of a ragged prefill batch one rank owns, with pool-local page ids."""
    requests: np.ndarray      # global request ids, ascending
    qo_indptr: np.ndarray     # [n + 1], starts at 0
    indptr: np.ndarray        # [n + 1], starts at 0
    indices: np.ndarray       # local page ids
    last: np.ndarray
    global_pages: np.ndarray  # local id -> page id in the caller's global pool
    query_rows: np.ndarray    # global query-token rows of the owned requests, in local order


def shard_prefill(qo_indptr, indptr, indices, last, requests) -> PrefillShard:
    """The sub-batch of `requests` (e.g. one entry of prefill_assignment): every request is
    independent, so a rank needs only the query rows and the pages of its own requests."""
    qo_indptr = np.asarray(qo_indptr, dtype=np.int64)
    indptr = np.asarray(indptr, dtype=np.int64)
    indices = np.asarray(indices)
    requests = np.asarray(requests, dtype=np.int64)
    qo_lens = qo_indptr[requests + 1] - qo_indptr[requests]
    pages = indptr[requests + 1] - indptr[requests]
    rows = (np.concatenate([np.arange(qo_indptr[r], qo_indptr[r + 1]) for r in requests])
            if len(requests) else np.zeros(0, dtype=np.int64))
    used = (np.concatenate([indices[indptr[r]:indptr[r + 1]] for r in requests])
            if len(requests) else np.zeros(0, dtype=np.int64))
    global_pages, local = np.unique(used, return_inverse=True)
    return PrefillShard(requests,
                        np.concatenate([[0], np.cumsum(qo_lens)]).astype(np.int32),
                        np.concatenate([[0], np.cumsum(pages)]).astype(np.int32),
                        local.astype(np.int32), np.asarray(last)[requests].astype(np.int32),
                        global_pages.astype(np.int64), rows.astype(np.int64))


def unpermute_query_rows(gathered_rows, shards_query_rows: List[np.ndarray]):
    """gathered_rows: per-rank query-token rows concatenated in rank order -> rows in the order of
    the unsharded batch.  shards_query_rows: PrefillShard.query_rows of every rank."""
    order = np.concatenate(shards_query_rows)
    inverse = np.empty_like(order)
    inverse[order] = np.arange(len(order))
    return gathered_rows[inverse]


def unpermute_rows(gathered_rows, assignment: List[np.ndarray]):
    """gathered_rows: per-rank row blocks concatenated in rank order -> rows in request order."""
    order = np.concatenate(assignment)
    inverse = np.empty_like(order)
    inverse[order] = np.arange(len(order))
    return gathered_rows[inverse]


def gather_output_rows(local_rows, row_counts: Optional[List[int]] = None, group=None):
    """All-gathers per-rank output rows `[rows_r, ...]` into `[sum rows, ...]` on every rank.

    Runs on the current stream of the tensor's device (NCCL for CUDA tensors), so it orders
    after the decode that produced `local_rows` when called under that stream.  Equal row counts
    use one all_gather_into_tensor; unequal counts pad to the maximum."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if row_counts is None:
        row_counts = [local_rows.shape[0]] * world
    if len(set(row_counts)) == 1:
        out = local_rows.new_empty((world * row_counts[0],) + tuple(local_rows.shape[1:]))
        dist.all_gather_into_tensor(out, local_rows.contiguous(), group=group)
        return out
    widest = max(row_counts)
    padded = local_rows.new_zeros((widest,) + tuple(local_rows.shape[1:]))
    padded[:local_rows.shape[0]] = local_rows
    out = local_rows.new_empty((world * widest,) + tuple(local_rows.shape[1:]))
    dist.all_gather_into_tensor(out, padded, group=group)
    blocks = out.view((world, widest) + tuple(local_rows.shape[1:]))
    return torch.cat([blocks[r, :row_counts[r]] for r in range(world)], dim=0)


class ShardFailure(RuntimeError):
    """A rank could not enqueue its shard; no rank entered the collective."""


_HOST_GROUP = None


def _host_group():
    """A gloo group for host-side agreement (the default group when it is gloo already)."""
    import torch.distributed as dist

    global _HOST_GROUP
    if dist.get_backend() == "gloo":
        return None
    if _HOST_GROUP is None:
        _HOST_GROUP = dist.new_group(backend="gloo")  # collective: every rank calls it once
    return _HOST_GROUP


def all_ranks_ok(ok: bool) -> bool:
    """Host-side agreement before a collective: True only if every rank passes ok=True.

    A rank whose enqueue failed (contract error, poisoned queue, launch failure) reports False
    instead of skipping the collective, so the others never wait for it on the GPU."""
    import torch
    import torch.distributed as dist

    flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=_host_group())
    return bool(flag.item())


def gather_output_rows_checked(local_rows, enqueued_ok: bool,
                               row_counts: Optional[List[int]] = None, group=None):
    """`gather_output_rows` guarded by `all_ranks_ok`: raises ShardFailure on EVERY rank when
    any rank failed, before the all-gather is started."""
    if not all_ranks_ok(enqueued_ok):
        raise ShardFailure("a rank failed to enqueue its shard; the all-gather was not started")
    return gather_output_rows(local_rows, row_counts, group)
