"""Host-side mirror of the reference's paged causal prefill interface.

Same names, argument meaning and error behaviour as Bf16PagedPrefillSpec / Bf16PagedPrefillMetadata
(crates/loom-infer/src/attention/paged_prefill/mod.rs:19-359) and PrefillProvider /
Bf16PagedPrefillPlan / Bf16PagedPrefillArgs (crates/loom-infer-cuda/src/attention/prefill.rs:
2278-2330,2440-2584,2853-2891); every method is a thin call through the C ABI.  Nothing here
computes on the CPU.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int32, c_size_t, c_void_p
from dataclasses import dataclass
from typing import Optional

from . import _abi
from ._abi import HEAD_DIM, PAGE_SIZE
from .api import CommandScope, Read, ReadWrite, Write, _check, _dispose, _i32

_I32P = ctypes.POINTER(c_int32)


class Bf16PagedPrefillSpec:
    """paged_prefill/mod.rs:19-159."""

    def __init__(self, raw: _abi.PrefillSpec):
        self._raw = raw

    @classmethod
    def new(cls, batch_size, nnz_qo, max_num_pages, num_query_heads, num_kv_heads,
            head_dim=HEAD_DIM, page_size=PAGE_SIZE):
        raw = _abi.PrefillSpec()
        _check(_abi.load().lb_prefill_spec_new(batch_size, nnz_qo, max_num_pages, num_query_heads,
                                               num_kv_heads, head_dim, page_size, byref(raw)))
        return cls(raw)

    def key(self):
        return (self.batch_size(), self.nnz_qo(), self.max_num_pages(), self.num_query_heads(),
                self.num_kv_heads())

    def __eq__(self, other):
        return isinstance(other, Bf16PagedPrefillSpec) and self.key() == other.key()

    def batch_size(self): return self._raw.batch_size
    def nnz_qo(self): return self._raw.nnz_qo
    def max_num_pages(self): return self._raw.max_num_pages
    def num_query_heads(self): return self._raw.num_query_heads
    def num_kv_heads(self): return self._raw.num_kv_heads
    def head_dim(self): return HEAD_DIM
    def page_size(self): return PAGE_SIZE
    def softmax_scale(self): return self._raw.softmax_scale
    def gqa_group_size(self): return self.num_query_heads() // self.num_kv_heads()
    def query_numel(self): return _abi.load().lb_prefill_spec_query_numel(byref(self._raw))
    def kv_pages_numel(self): return _abi.load().lb_prefill_spec_kv_pages_numel(byref(self._raw))
    def output_numel(self): return self.query_numel()
    def lse_numel(self): return _abi.load().lb_prefill_spec_lse_numel(byref(self._raw))
    def indptr_numel(self): return self.batch_size() + 1
    def last_page_len_numel(self): return self.batch_size()

    def kv_head_for_query_head(self, query_head: int) -> Optional[int]:
        if query_head >= self.num_query_heads():
            return None
        return query_head // self.gqa_group_size()

    def validate_metadata(self, qo_indptr, page_indptr, page_indices, last_page_len):
        qo, qop, qol = _i32(qo_indptr)
        ip, ipp, ipl = _i32(page_indptr)
        ix, ixp, ixl = _i32(page_indices)
        la, lap, lal = _i32(last_page_len)
        _check(_abi.load().lb_prefill_spec_validate_metadata(byref(self._raw), qop, qol, ipp, ipl,
                                                             ixp, ixl, lap, lal))
        return Bf16PagedPrefillMetadata(self, qo, ip, ix, la)


class Bf16PagedPrefillMetadata:
    """Validated dynamic metadata of one call, paged_prefill/mod.rs:268-359."""

    def __init__(self, spec, qo_indptr, page_indptr, page_indices, last_page_len):
        self._spec, self._qo, self._indptr = spec, qo_indptr, page_indptr
        self._indices, self._last = page_indices, last_page_len

    def spec(self): return self._spec
    def qo_indptr(self): return self._qo
    def page_indptr(self): return self._indptr
    def page_indices(self): return self._indices
    def last_page_len(self): return self._last

    def request_query_range(self, request):
        if request >= self._spec.batch_size():
            return None
        return int(self._qo[request]), int(self._qo[request + 1])

    def request_page_range(self, request):
        if request >= self._spec.batch_size():
            return None
        return int(self._indptr[request]), int(self._indptr[request + 1])

    def request_kv_len(self, request) -> Optional[int]:
        pages = self.request_page_range(request)
        if pages is None:
            return None
        return (pages[1] - pages[0] - 1) * PAGE_SIZE + int(self._last[request])

    def causal_kv_end(self, request, query_index) -> Optional[int]:
        out = c_size_t()
        ok = _abi.load().lb_prefill_metadata_causal_kv_end(
            byref(self._spec._raw), self._qo.ctypes.data_as(_I32P),
            self._indptr.ctypes.data_as(_I32P), self._last.ctypes.data_as(_I32P), request,
            query_index, byref(out))
        return out.value if ok else None

    def physical_page_for_token(self, request, logical_token):
        kv_len = self.request_kv_len(request)
        if kv_len is None or logical_token >= kv_len:
            return None
        start = int(self._indptr[request])
        return int(self._indices[start + logical_token // PAGE_SIZE]), logical_token % PAGE_SIZE


class Bf16PagedPrefillAlgorithm:
    TokenParallel = 0
    Tiled = 1


@dataclass
class Bf16PagedPrefillArgs:
    """prefill.rs:2853-2891, plus the ReadWrite F32 workspace a plan with partitions > 1 needs
    (plan.workspace_required_numel() elements; None otherwise)."""
    query: Read
    key_pages: Read
    value_pages: Read
    qo_indptr: Read
    page_indptr: Read
    page_indices: Read
    last_page_len: Read
    output: Write
    lse: Write
    workspace: Optional[ReadWrite] = None


class PrefillProvider:
    """prefill.rs:2278-2330."""

    def __init__(self, ptr, device):
        self._ptr, self._device = ptr, device

    @classmethod
    def load(cls, device: int = 0) -> "PrefillProvider":
        out = c_void_p()
        _check(_abi.load().lb_prefill_provider_load(device, byref(out)))
        return cls(out.value, device)

    def __del__(self):
        _dispose(self, "lb_prefill_provider_destroy")

    def device_status(self) -> int:
        out = c_int32()
        _check(_abi.load().lb_prefill_provider_device_status(self._ptr, byref(out)))
        return out.value

    def plan_bf16_paged(self, spec: Bf16PagedPrefillSpec, q_tiles: int = 0,
                        indices_capacity: bool = False, algorithm: int = 0,
                        partitions: int = 0, wait_limit_us: int = 0,
                        test_lost_copy: bool = False) -> "Bf16PagedPrefillPlan":
        """algorithm: 0 heuristic, 1 token-parallel, 2 tiled (tcgen05).  q_tiles (token-parallel):
        0 heuristic, else the 16-row tiles of packed query rows one CTA owns (1, 2, 4 or 8).
        partitions (tiled): 0 heuristic, 1 one CTA per tile, N > 1 the KV blocks of every tile
        shared out to N CTAs whose states a second command merges (needs the workspace).
        indices_capacity as for the decode plan.  wait_limit_us (tiled): limit of the kernel's
        bounded waits, 0 = about two seconds; test_lost_copy: tests of the give-up path only."""
        options = _abi.PrefillOptions(q_tiles=q_tiles, algorithm=algorithm, partitions=partitions,
                                      indices_capacity=1 if indices_capacity else 0,
                                      wait_limit_us=wait_limit_us,
                                      test_lost_copy=1 if test_lost_copy else 0)
        out = c_void_p()
        _check(_abi.load().lb_paged_prefill_plan_create(self._ptr, byref(spec._raw),
                                                        byref(options), byref(out)))
        return Bf16PagedPrefillPlan(out.value)


def choose_paged_prefill(spec: Bf16PagedPrefillSpec, sm_count: int, q_tiles: int = 0,
                         algorithm: int = 0, partitions: int = 0):
    """The plan-time launch shape as a pure function (no device needed)."""
    options = _abi.PrefillOptions(q_tiles=q_tiles, algorithm=algorithm, partitions=partitions)
    info = _abi.PrefillPlanInfo()
    _check(_abi.load().lb_paged_prefill_choose(byref(spec._raw), sm_count, byref(options),
                                               byref(info)))
    return info


class Bf16PagedPrefillPlan:
    """prefill.rs:2440-2584; immutable."""

    def __init__(self, ptr):
        self._ptr = ptr
        self._spec = _abi.PrefillSpec()
        self._info = _abi.PrefillPlanInfo()
        _check(_abi.load().lb_paged_prefill_plan_info_get(ptr, byref(self._spec),
                                                          byref(self._info)))

    def __del__(self):
        _dispose(self, "lb_paged_prefill_plan_destroy")

    def spec(self): return Bf16PagedPrefillSpec(self._spec)
    def algorithm(self): return self._info.algorithm
    def info(self): return self._info
    def commands(self): return self._info.commands
    def partitions(self): return self._info.partitions
    def workspace_required_numel(self): return self._info.workspace_numel
    def workspace_required_bytes(self): return self._info.workspace_numel * 4

    def enqueue_into(self, scope: CommandScope, args: Bf16PagedPrefillArgs):
        raw = _abi.PrefillArgs(
            query=args.query._raw, key_pages=args.key_pages._raw,
            value_pages=args.value_pages._raw, qo_indptr=args.qo_indptr._raw,
            page_indptr=args.page_indptr._raw, page_indices=args.page_indices._raw,
            last_page_len=args.last_page_len._raw, output=args.output._raw, lse=args.lse._raw)
        if args.workspace is not None:
            raw.workspace = args.workspace._raw
        _check(_abi.load().lb_paged_prefill_enqueue(self._ptr, scope._ptr, byref(raw)))
