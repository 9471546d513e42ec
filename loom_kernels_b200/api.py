"""Host-side mirror of the Loom Infer operator interface for the paged-decode path.

Same names, argument meaning and error behaviour as the reference's Rust API
(crates/loom-infer/src/attention/{paged_decode,paged_append}/mod.rs,
crates/loom-infer-cuda/src/{command,graph,attention/decode.rs,rope/mod.rs}); every method is a
thin call through the C ABI in include/loom_b200.h.  Nothing here computes on the CPU.

Buffers are CUDA torch tensors (torch owns device memory; this layer only passes pointers) or
`DeviceSpan` values (a raw device pointer with a length), which is what a non-torch engine binds.
"""
from __future__ import annotations

import ctypes
import gc
from ctypes import byref, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import numpy as np

from . import _abi
from ._abi import (ACCESS_READ, ACCESS_READ_WRITE, ACCESS_WRITE, BF16, F16, F32, HEAD_DIM, I32,
                   PAGE_SIZE, PARTIAL_STATE_WIDTH, U8)

# ---- errors --------------------------------------------------------------------------------------


class LoomError(Exception):
    """One reference error variant: `variant` is its name, `operand` and `payload` its fields."""

    def __init__(self, info: _abi.ErrorInfo):
        self.status = info.status
        self.variant = info.name.decode()
        self.operand = info.operand.decode()
        self.payload = (info.a, info.b, info.c, info.d)
        super().__init__(f"{self.variant}: {info.message.decode()}")


class ContractError(LoomError):
    pass


class CommandError(LoomError):
    pass


class EnqueueError(LoomError):
    """PagedBatchDecodeEnqueueError / RopeEnqueueError (own variants; Command(..) is CommandError)."""


class PlanError(LoomError):
    pass


class GraphError(LoomError):
    pass


def _raise(status: int):
    info = _abi.ErrorInfo()
    _abi.load().lb_last_error(byref(info))
    if status < 100:
        raise ContractError(info)
    if status < 200:
        raise CommandError(info)
    if status < 300:
        raise EnqueueError(info)
    if status < 400:
        raise PlanError(info)
    if status < 500:
        raise GraphError(info)
    raise LoomError(info)


def _check(status: int):
    if status != 0:
        _raise(status)


def _dispose(owner, symbol: str):
    """Hand `owner._ptr` to the library's destroy/abandon entry point exactly once.  At interpreter
    exit module globals are already cleared, and the process is about to release everything."""
    ptr = getattr(owner, "_ptr", None)
    owner._ptr = None
    load = getattr(_abi, "load", None)
    if ptr and load is not None:
        getattr(load(), symbol)(ptr)


def _i32(values):
    array = np.ascontiguousarray(values, dtype=np.int32)
    return array, array.ctypes.data_as(ctypes.POINTER(c_int32)), c_size_t(array.size)


# ---- contract --------------------------------------------------------------------------------------


class Bf16PagedBatchDecodeSpec:
    """crates/loom-infer/src/attention/paged_decode/mod.rs:17-214."""

    def __init__(self, raw: _abi.PagedSpec):
        self._raw = raw

    @classmethod
    def new(cls, batch_size, max_num_pages, num_query_heads, num_kv_heads, head_dim=HEAD_DIM,
            page_size=PAGE_SIZE):
        raw = _abi.PagedSpec()
        _check(_abi.load().lb_paged_spec_new(batch_size, max_num_pages, num_query_heads,
                                             num_kv_heads, head_dim, page_size, byref(raw)))
        return cls(raw)

    def __eq__(self, other):
        return isinstance(other, Bf16PagedBatchDecodeSpec) and self.key() == other.key()

    def key(self):
        return (self.batch_size(), self.max_num_pages(), self.num_query_heads(),
                self.num_kv_heads())

    def batch_size(self): return self._raw.batch_size
    def max_num_pages(self): return self._raw.max_num_pages
    def num_query_heads(self): return self._raw.num_query_heads
    def num_kv_heads(self): return self._raw.num_kv_heads
    def head_dim(self): return HEAD_DIM
    def page_size(self): return PAGE_SIZE
    def softmax_scale(self): return self._raw.softmax_scale
    def gqa_group_size(self): return _abi.load().lb_paged_spec_gqa_group_size(byref(self._raw))
    def query_numel(self): return _abi.load().lb_paged_spec_query_numel(byref(self._raw))
    def kv_pages_numel(self): return _abi.load().lb_paged_spec_kv_pages_numel(byref(self._raw))
    def output_numel(self): return self.query_numel()
    def lse_numel(self): return _abi.load().lb_paged_spec_lse_numel(byref(self._raw))
    def page_indptr_numel(self): return self.batch_size() + 1
    def last_page_len_numel(self): return self.batch_size()

    def kv_head_for_query_head(self, query_head: int) -> Optional[int]:
        head = _abi.load().lb_paged_spec_kv_head_for_query_head(byref(self._raw), query_head)
        return None if head < 0 else head

    def validate_page_table(self, page_indptr, page_indices, last_page_len):
        ip, ipp, ipl = _i32(page_indptr)
        ix, ixp, ixl = _i32(page_indices)
        la, lap, lal = _i32(last_page_len)
        _check(_abi.load().lb_paged_spec_validate_page_table(byref(self._raw), ipp, ipl, ixp, ixl,
                                                             lap, lal))
        return Bf16PagedBatchDecodePageTable(self, ip, ix, la)


class Bf16PagedBatchDecodePageTable:
    """Validated page-table view, paged_decode/mod.rs:216-279."""

    def __init__(self, spec, indptr, indices, last):
        self._spec, self._indptr, self._indices, self._last = spec, indptr, indices, last

    def spec(self): return self._spec
    def page_indptr(self): return self._indptr
    def page_indices(self): return self._indices
    def last_page_len(self): return self._last

    def request_page_range(self, request):
        if request >= self._spec.batch_size():
            return None
        return int(self._indptr[request]), int(self._indptr[request + 1])

    def request_kv_len(self, request) -> Optional[int]:
        out = c_size_t()
        ok = _abi.load().lb_page_table_request_kv_len(
            byref(self._spec._raw), self._indptr.ctypes.data_as(ctypes.POINTER(c_int32)),
            self._last.ctypes.data_as(ctypes.POINTER(c_int32)), request, byref(out))
        return out.value if ok else None

    def physical_page_for_token(self, request, logical_token):
        page, offset = c_size_t(), c_size_t()
        ok = _abi.load().lb_page_table_physical_page_for_token(
            byref(self._spec._raw), self._indptr.ctypes.data_as(ctypes.POINTER(c_int32)),
            self._indices.ctypes.data_as(ctypes.POINTER(c_int32)),
            self._last.ctypes.data_as(ctypes.POINTER(c_int32)), request, logical_token,
            byref(page), byref(offset))
        return (page.value, offset.value) if ok else None


class Bf16RopePagedKvAppendSpec:
    """crates/loom-infer/src/attention/paged_append/mod.rs:14-132."""

    def __init__(self, paged: Bf16PagedBatchDecodeSpec):
        self._paged = paged

    @classmethod
    def new(cls, batch_size, max_num_pages, num_query_heads, num_kv_heads, head_dim=HEAD_DIM,
            page_size=PAGE_SIZE):
        return cls(Bf16PagedBatchDecodeSpec.new(batch_size, max_num_pages, num_query_heads,
                                                num_kv_heads, head_dim, page_size))

    def paged(self): return self._paged
    def batch_size(self): return self._paged.batch_size()
    def max_num_pages(self): return self._paged.max_num_pages()
    def num_query_heads(self): return self._paged.num_query_heads()
    def num_kv_heads(self): return self._paged.num_kv_heads()
    def query_numel(self): return self._paged.query_numel()
    def key_numel(self): return self.batch_size() * self.num_kv_heads() * HEAD_DIM
    def value_numel(self): return self.key_numel()
    def query_output_numel(self): return self.query_numel()
    def kv_pages_numel(self): return self._paged.kv_pages_numel()

    def validate_page_table(self, page_indptr, page_indices, last_page_len):
        ip, ipp, ipl = _i32(page_indptr)
        ix, ixp, ixl = _i32(page_indices)
        la, lap, lal = _i32(last_page_len)
        _check(_abi.load().lb_append_spec_validate_page_table(byref(self._paged._raw), ipp, ipl,
                                                              ixp, ixl, lap, lal))
        return Bf16PagedBatchDecodePageTable(self._paged, ip, ix, la)


class Bf16RopePagedKvAppendTokensSpec:
    """paged_append/mod.rs:134-318.  `new_extended` lifts the 64-token total cap."""

    def __init__(self, raw: _abi.AppendTokensSpec):
        self._raw = raw
        self._paged = Bf16PagedBatchDecodeSpec(raw.paged)

    @classmethod
    def new(cls, tokens, batch_size, max_num_pages, num_query_heads, num_kv_heads,
            head_dim=HEAD_DIM, page_size=PAGE_SIZE):
        raw = _abi.AppendTokensSpec()
        _check(_abi.load().lb_append_tokens_spec_new(tokens, batch_size, max_num_pages,
                                                     num_query_heads, num_kv_heads, head_dim,
                                                     page_size, byref(raw)))
        return cls(raw)

    @classmethod
    def new_extended(cls, tokens, batch_size, max_num_pages, num_query_heads, num_kv_heads,
                     head_dim=HEAD_DIM, page_size=PAGE_SIZE):
        raw = _abi.AppendTokensSpec()
        _check(_abi.load().lb_append_tokens_spec_new_extended(
            tokens, batch_size, max_num_pages, num_query_heads, num_kv_heads, head_dim, page_size,
            byref(raw)))
        return cls(raw)

    def tokens(self): return self._raw.tokens
    def paged(self): return self._paged
    def batch_size(self): return self._paged.batch_size()
    def max_num_pages(self): return self._paged.max_num_pages()
    def num_query_heads(self): return self._paged.num_query_heads()
    def num_kv_heads(self): return self._paged.num_kv_heads()
    def query_numel(self): return self.tokens() * self.num_query_heads() * HEAD_DIM
    def key_numel(self): return self.tokens() * self.num_kv_heads() * HEAD_DIM
    def value_numel(self): return self.key_numel()
    def query_output_numel(self): return self.query_numel()
    def kv_pages_numel(self): return self._paged.kv_pages_numel()

    def validate_metadata(self, batch_indices, positions, page_indptr, page_indices,
                          last_page_len):
        """Returns the physical (page, offset) slot of every token."""
        _, bp, bl = _i32(batch_indices)
        _, pp, pl = _i32(positions)
        _, ipp, ipl = _i32(page_indptr)
        _, ixp, ixl = _i32(page_indices)
        _, lap, lal = _i32(last_page_len)
        slots = np.zeros((self.tokens(), 2), dtype=np.int64)
        _check(_abi.load().lb_append_tokens_spec_validate_metadata(
            byref(self._raw), bp, bl, pp, pl, ipp, ipl, ixp, ixl, lap, lal,
            slots.ctypes.data_as(ctypes.POINTER(c_int64))))
        return [tuple(int(v) for v in row) for row in slots]


def split_partition_range(length: int, partitions: int, partition: int):
    """Bf16SingleDecodeSplitKSpec::partition_token_range (single_decode/mod.rs:171-185)."""
    start, end = c_size_t(), c_size_t()
    ok = _abi.load().lb_split_partition_range(length, partitions, partition, byref(start),
                                              byref(end))
    return (start.value, end.value) if ok else None


def paged_split_workspace_numel(spec: Bf16PagedBatchDecodeSpec, partitions: int) -> int:
    out = c_size_t()
    _check(_abi.load().lb_paged_split_workspace_numel(byref(spec._raw), partitions, byref(out)))
    return out.value


def paged_split_state_offset(spec, partitions, request, query_head, partition):
    offset = _abi.load().lb_paged_split_state_offset(byref(spec._raw), partitions, request,
                                                     query_head, partition)
    return None if offset < 0 else offset


# ---- command runtime ---------------------------------------------------------------------------------


@dataclass(frozen=True)
class DeviceSpan:
    """A caller-owned device allocation: pointer, element count, element type."""
    ptr: int
    numel: int
    dtype: int


def _describe(buffer):
    if isinstance(buffer, DeviceSpan):
        return buffer.dtype, buffer.ptr, buffer.numel
    import torch
    dtypes = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int32: I32,
              torch.uint8: U8}
    if buffer.dtype not in dtypes:
        raise TypeError(f"unsupported element type {buffer.dtype}")
    if not buffer.is_contiguous():
        raise ValueError("bindings take contiguous device buffers")
    return dtypes[buffer.dtype], buffer.data_ptr(), buffer.numel()


class _Handle:
    access = ACCESS_READ

    def __init__(self, raw: _abi.Handle):
        self._raw = raw

    def slot(self): return self._raw.slot
    def set_id(self): return self._raw.set_id


class Read(_Handle):
    access = ACCESS_READ


class Write(_Handle):
    access = ACCESS_WRITE


class ReadWrite(_Handle):
    """command/binding.rs:306-327."""
    access = ACCESS_READ_WRITE

    def read(self) -> Read:
        return Read(_abi.load().lb_handle_read(self._raw))

    def write(self) -> Write:
        return Write(_abi.load().lb_handle_write(self._raw))


def _null_handle():
    return _abi.Handle()


class CheckedBindings:
    """command/binding.rs:16-134."""

    def __init__(self, ptr):
        self._ptr = ptr
        self._buffers = {}

    def __del__(self):
        _dispose(self, "lb_bindings_destroy")

    def _release(self):
        ptr, self._ptr = self._ptr, None
        return ptr

    def capacity(self): return _abi.load().lb_bindings_capacity(self._ptr)
    def __len__(self): return _abi.load().lb_bindings_len(self._ptr)

    def bind_read(self, buffer) -> Read:
        dtype, ptr, numel = _describe(buffer)
        raw = _abi.Handle()
        _check(_abi.load().lb_bind_read(self._ptr, dtype, c_void_p(ptr), numel, byref(raw)))
        self._buffers[raw.slot] = buffer
        return Read(raw)

    def bind_read_write(self, buffer) -> ReadWrite:
        dtype, ptr, numel = _describe(buffer)
        raw = _abi.Handle()
        _check(_abi.load().lb_bind_read_write(self._ptr, dtype, c_void_p(ptr), numel, byref(raw)))
        self._buffers[raw.slot] = buffer
        return ReadWrite(raw)

    def take_read_write(self, handle: ReadWrite):
        ptr, numel = c_void_p(), c_size_t()
        _check(_abi.load().lb_take_read_write(self._ptr, handle._raw, byref(ptr), byref(numel)))
        return self._buffers.pop(handle._raw.slot)


class CommandQueue:
    """command/submission.rs:18-117.  `stream` is a torch.cuda.Stream or a raw stream handle."""

    def __init__(self, stream, max_commands: int):
        self._stream_owner = stream
        handle = getattr(stream, "cuda_stream", stream)
        out = c_void_p()
        _check(_abi.load().lb_queue_create(c_void_p(handle), max_commands, byref(out)))
        self._ptr = out.value

    def __del__(self):
        _dispose(self, "lb_queue_destroy")

    def stream(self): return self._stream_owner
    def max_commands(self): return _abi.load().lb_queue_max_commands(self._ptr)
    def is_poisoned(self): return bool(_abi.load().lb_queue_is_poisoned(self._ptr))

    def bindings(self, capacity: int) -> CheckedBindings:
        out = c_void_p()
        _check(_abi.load().lb_queue_bindings(self._ptr, capacity, byref(out)))
        return CheckedBindings(out.value)

    def begin(self, bindings: CheckedBindings) -> "CommandScope":
        buffers = bindings._buffers
        out = c_void_p()
        status = _abi.load().lb_queue_begin(self._ptr, bindings._ptr, byref(out))
        if status != _abi_status("LB_OBJECT_IN_USE"):
            bindings._release()  # moved, on success and on contract failures alike
        _check(status)
        return CommandScope(self, out.value, buffers)


def _abi_status(name: str) -> int:
    return {"LB_OBJECT_IN_USE": 501}[name]


class CommandScope:
    """command/submission.rs:119-329."""

    def __init__(self, queue, ptr, buffers):
        self._queue, self._ptr, self._buffers = queue, ptr, buffers

    def __del__(self):
        _dispose(self, "lb_scope_abandon")

    def submitted_commands(self): return _abi.load().lb_scope_submitted(self._ptr)

    def finish(self) -> "CommandCompletion":
        out = c_void_p()
        ptr, self._ptr = self._ptr, None
        _check(_abi.load().lb_scope_finish(ptr, byref(out)))
        return CommandCompletion(self._queue, out.value, self._buffers)


class CommandCompletion:
    """command/completion.rs:6-141."""

    def __init__(self, queue, ptr, buffers):
        self._queue, self._ptr, self._buffers = queue, ptr, buffers

    def __del__(self):
        _dispose(self, "lb_completion_abandon")

    def submitted(self): return _abi.load().lb_completion_submitted(self._ptr)

    def is_complete(self) -> bool:
        done = c_int()
        _check(_abi.load().lb_completion_is_complete(self._ptr, byref(done)))
        return bool(done.value)

    def wait(self) -> CheckedBindings:
        out = c_void_p()
        ptr, self._ptr = self._ptr, None
        _check(_abi.load().lb_completion_wait(ptr, byref(out)))
        bindings = CheckedBindings(out.value)
        bindings._buffers = self._buffers
        return bindings


# ---- decode provider -----------------------------------------------------------------------------------


class Bf16PagedBatchDecodeAlgorithm:
    ClusterSplit = 3
    Direct = 0
    SplitK = 1
    Balanced = 2


@dataclass
class Bf16PagedBatchDecodeArgs:
    """decode.rs:1451-1487 plus the split-K workspace operand (:1420-1449)."""
    query: Read
    key_pages: Read
    value_pages: Read
    page_indptr: Read
    page_indices: Read
    last_page_len: Read
    output: Write
    lse: Write
    workspace: Optional[ReadWrite] = None


@dataclass
class StateMergeArgs:
    """states F32 [rows, partitions, 130]; output BF16 [rows, 128]; lse F32 [rows] (base 2)."""
    states: Read
    output: Write
    lse: Write


class StateMergePlan:
    def __init__(self, ptr, rows, partitions):
        self._ptr, self._rows, self._partitions = ptr, rows, partitions

    def __del__(self):
        _dispose(self, "lb_state_merge_plan_destroy")

    def rows(self): return self._rows
    def partitions(self): return self._partitions
    def states_numel(self): return self._rows * self._partitions * PARTIAL_STATE_WIDTH

    def enqueue_into(self, scope: "CommandScope", args: StateMergeArgs):
        raw = _abi.StateMergeArgs(states=args.states._raw, output=args.output._raw,
                                  lse=args.lse._raw)
        _check(_abi.load().lb_state_merge_enqueue(self._ptr, scope._ptr, byref(raw)))


class DecodeProvider:
    """decode.rs:1001-1104."""

    def __init__(self, ptr, device):
        self._ptr, self._device = ptr, device

    @classmethod
    def load(cls, device: int = 0) -> "DecodeProvider":
        out = c_void_p()
        _check(_abi.load().lb_decode_provider_load(device, byref(out)))
        return cls(out.value, device)

    def __del__(self):
        _dispose(self, "lb_decode_provider_destroy")

    def device_status(self) -> int:
        out = c_int32()
        _check(_abi.load().lb_decode_provider_device_status(self._ptr, byref(out)))
        return out.value

    def plan_state_merge(self, rows: int, partitions: int) -> "StateMergePlan":
        """The split-K merge as an operator over caller-provided states (no reference
        counterpart; listed as planned in the reference's docs/flashinfer-parity.md:38)."""
        out = c_void_p()
        _check(_abi.load().lb_state_merge_plan_create(self._ptr, rows, partitions, byref(out)))
        return StateMergePlan(out.value, rows, partitions)

    def plan_bf16_paged_batch(self, spec: Bf16PagedBatchDecodeSpec, partitions: int = 0,
                              heads_per_cta: int = 0, balanced: int = 0,
                              balanced_ctas: int = 0, indices_capacity: bool = False,
                              wait_limit_us: int = 0, test_skip_page: int = 0,
                              cluster: bool = False,
                              merge_in_kernel: int = 0,
                              max_stages: int = 0,
                              producer_warps: int = 0) -> "Bf16PagedBatchDecodePlan":
        """partitions: 0 heuristic, 1 direct, N split-K; balanced (with partitions 0): 0
        heuristic, 1 force the balanced algorithm, 2 never use it.  indices_capacity: the bound
        page_indices may be longer than the table in use (page_indptr[batch] <= len), which
        lets one fixed-address Graph serve steps with different total page counts.
        wait_limit_us: limit of the kernels' bounded waits (0 = about two seconds);
        test_skip_page: tests of the give-up path only.  merge_in_kernel (static split-K): 1 the
        last CTA of an item merges it (one command), 0 or 2 a second command does.  max_stages:
        cap on the stages of the page ring (0 = the plan decides)."""
        options = _abi.DecodeOptions(partitions=partitions, heads_per_cta=heads_per_cta,
                                     balanced=balanced, balanced_ctas=balanced_ctas,
                                     indices_capacity=1 if indices_capacity else 0,
                                     wait_limit_us=wait_limit_us, test_skip_page=test_skip_page,
                                     cluster=1 if cluster else 0,
                                     merge_in_kernel=merge_in_kernel, max_stages=max_stages,
                                     producer_warps=producer_warps)
        out = c_void_p()
        _check(_abi.load().lb_paged_decode_plan_create(self._ptr, byref(spec._raw),
                                                       byref(options), byref(out)))
        return Bf16PagedBatchDecodePlan(out.value)


def choose_paged_decode(spec, sm_count: int, partitions: int = 0, heads_per_cta: int = 0,
                        balanced: int = 0, merge_in_kernel: int = 0):
    """The plan-time heuristic as a pure function (no device needed)."""
    options = _abi.DecodeOptions(partitions=partitions, heads_per_cta=heads_per_cta,
                                 balanced=balanced, merge_in_kernel=merge_in_kernel)
    info = _abi.DecodePlanInfo()
    _check(_abi.load().lb_paged_decode_choose(byref(spec._raw), sm_count, byref(options),
                                              byref(info)))
    return info


class Bf16PagedBatchDecodePlan:
    """decode.rs:1181-1297; immutable."""

    def __init__(self, ptr):
        self._ptr = ptr
        self._spec = _abi.PagedSpec()
        self._info = _abi.DecodePlanInfo()
        _check(_abi.load().lb_paged_decode_plan_info_get(ptr, byref(self._spec),
                                                         byref(self._info)))

    def __del__(self):
        _dispose(self, "lb_paged_decode_plan_destroy")

    def spec(self): return Bf16PagedBatchDecodeSpec(self._spec)
    def algorithm(self): return self._info.algorithm
    def partitions(self): return self._info.partitions
    def info(self): return self._info
    def commands(self): return self._info.commands
    def merged_in_kernel(self): return bool(self._info.merged_in_kernel)
    def workspace_required_numel(self): return self._info.workspace_numel
    def workspace_required_bytes(self): return self._info.workspace_bytes

    def enqueue_into(self, scope: CommandScope, args: Bf16PagedBatchDecodeArgs):
        raw = _abi.DecodeArgs(
            query=args.query._raw, key_pages=args.key_pages._raw,
            value_pages=args.value_pages._raw, page_indptr=args.page_indptr._raw,
            page_indices=args.page_indices._raw, last_page_len=args.last_page_len._raw,
            output=args.output._raw, lse=args.lse._raw,
            workspace=args.workspace._raw if args.workspace is not None else _null_handle())
        _check(_abi.load().lb_paged_decode_enqueue(self._ptr, scope._ptr, byref(raw)))

    def enqueue_gathered_into(self, scope: CommandScope, args: Bf16PagedBatchDecodeArgs,
                              dest_rows: Read, group: "PeerGroup", output: "PeerBuffer",
                              lse: "PeerBuffer", total_requests: int,
                              gathered_query_heads: int = 0, head_offset: int = 0,
                              defer_wait: bool = False):
        """lb_paged_decode_enqueue_gathered: args.output / args.lse are the bound local copies of
        the peer buffers `output` / `lse`; every finished row goes to every rank's copy.
        defer_wait: a later gathering command of the same step publishes the epoch and waits."""
        decode = _abi.DecodeArgs(
            query=args.query._raw, key_pages=args.key_pages._raw,
            value_pages=args.value_pages._raw, page_indptr=args.page_indptr._raw,
            page_indices=args.page_indices._raw, last_page_len=args.last_page_len._raw,
            output=args.output._raw, lse=args.lse._raw,
            workspace=args.workspace._raw if args.workspace is not None else _null_handle())
        raw = _abi.DecodeGatherArgs(decode=decode, dest_rows=dest_rows._raw)
        layout = _abi.GatherLayout(
            total_requests=total_requests,
            gathered_query_heads=gathered_query_heads or self._spec.num_query_heads,
            head_offset=head_offset, defer_wait=1 if defer_wait else 0)
        _check(_abi.load().lb_paged_decode_enqueue_gathered(
            self._ptr, scope._ptr, byref(raw), byref(layout), group._ptr, output._ptr, lse._ptr))


# ---- output rows across GPUs ------------------------------------------------------------------------


class PeerGroup:
    """The ranks of one job, one process per GPU (lb_peer_group).  Creating a group, a peer buffer
    and enqueueing a gathering command are collective."""

    ID_BYTES = 128

    @staticmethod
    def unique_id() -> bytes:
        raw = (ctypes.c_uint8 * PeerGroup.ID_BYTES)()
        _check(_abi.load().lb_peer_group_unique_id(raw))
        return bytes(raw)

    def __init__(self, device: int, world: int, rank: int, unique_id: bytes):
        raw = (ctypes.c_uint8 * PeerGroup.ID_BYTES).from_buffer_copy(unique_id)
        out = c_void_p()
        _check(_abi.load().lb_peer_group_create(device, world, rank, raw, byref(out)))
        self._ptr = out.value
        self._buffers = []

    @classmethod
    def from_torch_distributed(cls, device: int) -> "PeerGroup":
        """Joins the ranks of the default torch.distributed group (the id travels by broadcast)."""
        import torch.distributed as dist
        world, rank = dist.get_world_size(), dist.get_rank()
        box = [cls.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return cls(device, world, rank, box[0])

    def rank(self): return _abi.load().lb_peer_group_rank(self._ptr)
    def world(self): return _abi.load().lb_peer_group_world(self._ptr)

    def buffer(self, numel: int, dtype: int) -> "PeerBuffer":
        return PeerBuffer(self, numel, dtype)

    def close(self):
        """After a host barrier: no rank may still store into this rank's buffers."""
        for buffer in self._buffers:
            buffer.close()
        self._buffers = []
        if self._ptr:
            _abi.load().lb_peer_group_destroy(self._ptr)
            self._ptr = None


class PeerBuffer:
    """Device memory of the same size on every rank, each copy mapped on every other rank
    (lb_peer_buffer).  `span` binds the local copy; `tensor()` views it as a torch tensor."""

    _ELEMENT_BYTES = {F32: 4, F16: 2, BF16: 2, I32: 4, U8: 1}

    def __init__(self, group: PeerGroup, numel: int, dtype: int):
        out = c_void_p()
        _check(_abi.load().lb_peer_buffer_create(group._ptr, numel * self._ELEMENT_BYTES[dtype],
                                                 byref(out)))
        self._ptr = out.value
        self.numel, self.dtype = numel, dtype
        self.span = DeviceSpan(_abi.load().lb_peer_buffer_local(self._ptr), numel, dtype)
        group._buffers.append(self)

    def tensor(self, device):
        """A torch view of the local copy (the library owns the memory; keep this object alive)."""
        import torch
        kinds = {F32: ("<f4", torch.float32), I32: ("<i4", torch.int32), U8: ("|u1", torch.uint8),
                 BF16: ("<i2", torch.bfloat16), F16: ("<f2", torch.float16)}
        typestr, dtype = kinds[self.dtype]

        class _Holder:
            __cuda_array_interface__ = {"shape": (self.numel,), "typestr": typestr,
                                        "data": (self.span.ptr, False), "version": 3}
        view = torch.as_tensor(_Holder(), device=device)
        return view.view(dtype) if view.dtype != dtype else view

    def close(self):
        if self._ptr:
            _abi.load().lb_peer_buffer_destroy(self._ptr)
            self._ptr = None


@dataclass
class OutputGatherArgs:
    local: Read
    gathered: Write


class OutputGatherPlan:
    """The all-gather of per-rank rows as one command of the scope (lb_output_gather_*)."""

    def __init__(self, group: PeerGroup, dtype: int, rows_per_rank: Sequence[int], row_numel: int):
        rows = (c_size_t * len(rows_per_rank))(*rows_per_rank)
        out = c_void_p()
        _check(_abi.load().lb_output_gather_plan_create(group._ptr, dtype, rows, row_numel,
                                                        byref(out)))
        self._ptr = out.value
        self._group = group

    def __del__(self):
        _dispose(self, "lb_output_gather_plan_destroy")

    def enqueue_into(self, scope: CommandScope, args: OutputGatherArgs):
        raw = _abi.OutputGatherArgs(local=args.local._raw, gathered=args.gathered._raw)
        _check(_abi.load().lb_output_gather_enqueue(self._ptr, scope._ptr, byref(raw)))


def paged_decode_split_noalloc(spec: Bf16PagedBatchDecodeSpec, partitions: int, stream, query,
                               key_pages, value_pages, page_indptr, page_indices, last_page_len,
                               output, lse):
    """Split-K paged decode without a caller workspace (lb_paged_decode_split_noalloc).

    For hosts that cannot allocate device memory: the partial states live in a fixed array inside
    the library (at most `paged_decode_split_noalloc_max_states()` states).  Arguments are CUDA
    tensors (or DeviceSpan) used as raw pointers; the call enqueues on `stream` and returns.
    Calls that overlap on the GPU race on the shared array."""
    def pointer(buffer):
        return c_void_p(_describe(buffer)[1])

    # raw pointers carry no length across the C ABI; this wrapper knows the tensors, so it makes
    # the length and type checks lb_paged_decode_enqueue makes before anything is launched
    batch = spec.batch_size()
    expected = (("Q", query, BF16, spec.query_numel()),
                ("K_pages", key_pages, BF16, spec.kv_pages_numel()),
                ("V_pages", value_pages, BF16, spec.kv_pages_numel()),
                ("page_indptr", page_indptr, I32, batch + 1),
                ("last_page_len", last_page_len, I32, batch),
                ("O", output, BF16, spec.output_numel()),
                ("LSE", lse, F32, spec.lse_numel()))
    limit = paged_decode_split_noalloc_max_states()
    fits = partitions >= 2 and batch * spec.num_query_heads() * partitions <= limit
    for operand, buffer, dtype, numel in expected:
        actual_dtype, _, actual = _describe(buffer)
        if actual_dtype != dtype:
            raise TypeError(f"{operand}: element type {actual_dtype}, expected {dtype}")
        # a request the static array cannot hold is refused by the library itself, whatever the
        # buffers are
        if fits and actual != numel:
            info = _abi.ErrorInfo(status=200, name=b"LengthMismatch", operand=operand.encode(),
                                  a=numel, b=actual,
                                  message=f"{operand} length mismatch: expected {numel}, "
                                          f"got {actual}".encode())
            raise EnqueueError(info)
    if _describe(page_indices)[0] != I32:
        raise TypeError("page_indices: expected I32")
    handle = getattr(stream, "cuda_stream", stream)
    indices_ptr = ctypes.cast(pointer(page_indices), ctypes.POINTER(c_int32))
    _check(_abi.load().lb_paged_decode_split_noalloc(
        byref(spec._raw), partitions, c_void_p(handle), pointer(query), pointer(key_pages),
        pointer(value_pages), ctypes.cast(pointer(page_indptr), ctypes.POINTER(c_int32)),
        indices_ptr, _describe(page_indices)[2],
        ctypes.cast(pointer(last_page_len), ctypes.POINTER(c_int32)), pointer(output),
        pointer(lse)))


def paged_decode_split_noalloc_status(device: int = 0) -> int:
    """Reads and clears the status word of the no-workspace entry point on `device`: non-zero when
    a CTA of one of its calls gave up on a bounded wait since the last read."""
    status = c_int32(0)
    _check(_abi.load().lb_paged_decode_split_noalloc_status(device, byref(status)))
    return status.value


def paged_decode_split_noalloc_max_states() -> int:
    return _abi.load().lb_paged_decode_split_noalloc_max_states()


# ---- RoPE + append provider -------------------------------------------------------------------------------


@dataclass
class Bf16RopePagedKvAppendArgs:
    """rope/mod.rs:963-1010."""
    query: Read
    key: Read
    value: Read
    page_indptr: Read
    page_indices: Read
    last_page_len: Read
    query_output: Write
    key_pages: Write
    value_pages: Write


@dataclass
class Bf16RopePagedKvAppendTokensArgs:
    """rope/mod.rs:1012-1077."""
    query: Read
    key: Read
    value: Read
    batch_indices: Read
    positions: Read
    page_indptr: Read
    page_indices: Read
    last_page_len: Read
    query_output: Write
    key_pages: Write
    value_pages: Write
    workspace: Optional[ReadWrite] = None  # I32, extended plans only


class Bf16RopePosIdsSpec:
    """Standard NeoX split-half RoPE over contiguous NHD Q and K
    (crates/loom-infer/src/rope/mod.rs:9-108)."""

    def __init__(self, raw: _abi.RopePosIdsSpec):
        self._raw = raw

    @classmethod
    def new(cls, tokens, query_heads, key_heads, head_dim=HEAD_DIM, rotary_dim=HEAD_DIM,
            rope_scale=1.0, rope_theta=10000.0):
        raw = _abi.RopePosIdsSpec()
        _check(_abi.load().lb_rope_pos_ids_spec_new(tokens, query_heads, key_heads, head_dim,
                                                    rotary_dim, rope_scale, rope_theta, byref(raw)))
        return cls(raw)

    def tokens(self): return self._raw.tokens
    def query_heads(self): return self._raw.query_heads
    def key_heads(self): return self._raw.key_heads
    def head_dim(self): return self._raw.head_dim
    def rotary_dim(self): return self._raw.rotary_dim
    def rope_scale(self): return self._raw.rope_scale
    def rope_theta(self): return self._raw.rope_theta
    def query_numel(self): return _abi.load().lb_rope_pos_ids_spec_query_numel(byref(self._raw))
    def key_numel(self): return _abi.load().lb_rope_pos_ids_spec_key_numel(byref(self._raw))
    def position_numel(self): return self._raw.tokens


@dataclass
class Bf16RopePosIdsArgs:
    """crates/loom-infer-cuda/src/rope/mod.rs (Bf16RopePosIdsArgs::new)."""
    query: Read
    key: Read
    position_ids: Read
    query_output: Write
    key_output: Write


class Bf16RopePosIdsPlan:
    """rope/mod.rs:694-742."""

    def __init__(self, ptr, spec):
        self._ptr, self._spec = ptr, spec

    def __del__(self):
        _dispose(self, "lb_rope_pos_ids_plan_destroy")

    def spec(self): return self._spec

    def enqueue_into(self, scope: "CommandScope", args: Bf16RopePosIdsArgs):
        raw = _abi.RopePosIdsArgs(query=args.query._raw, key=args.key._raw,
                                  position_ids=args.position_ids._raw,
                                  query_output=args.query_output._raw,
                                  key_output=args.key_output._raw)
        _check(_abi.load().lb_rope_pos_ids_enqueue(self._ptr, scope._ptr, byref(raw)))


class RopeProvider:
    """rope/mod.rs:579-683."""

    def __init__(self, ptr):
        self._ptr = ptr

    def device_status(self) -> int:
        """Reads and clears the provider's device status word (written by the checked build of the
        library only: 0x1000 | site when a computed index fell outside its operand)."""
        status = c_int32(0)
        _check(_abi.load().lb_rope_provider_device_status(self._ptr, byref(status)))
        return status.value

    def plan_bf16_pos_ids(self, spec: Bf16RopePosIdsSpec) -> Bf16RopePosIdsPlan:
        out = c_void_p()
        _check(_abi.load().lb_rope_pos_ids_plan_create(self._ptr, byref(spec._raw), byref(out)))
        return Bf16RopePosIdsPlan(out.value, spec)

    @classmethod
    def load(cls, device: int = 0) -> "RopeProvider":
        out = c_void_p()
        _check(_abi.load().lb_rope_provider_load(device, byref(out)))
        return cls(out.value)

    def __del__(self):
        _dispose(self, "lb_rope_provider_destroy")

    def plan_bf16_paged_append(self, spec: Bf16RopePagedKvAppendSpec,
                               indices_capacity: bool = False):
        """indices_capacity: see DecodeProvider.plan_bf16_paged_batch."""
        out = c_void_p()
        options = _abi.AppendOptions(indices_capacity=1 if indices_capacity else 0)
        _check(_abi.load().lb_rope_append_plan_create_with(self._ptr, byref(spec.paged()._raw),
                                                           byref(options), byref(out)))
        return Bf16RopePagedKvAppendPlan(out.value, spec)

    def plan_bf16_paged_append_tokens(self, spec: Bf16RopePagedKvAppendTokensSpec,
                                      indices_capacity: bool = False, one_command: bool = False):
        """one_command (extended specs of up to 2048 tokens): validation and scatter in one kernel
        whose token CTAs wait for the validators, instead of two commands."""
        out = c_void_p()
        options = _abi.AppendOptions(indices_capacity=1 if indices_capacity else 0,
                                     one_command=1 if one_command else 0)
        _check(_abi.load().lb_rope_append_tokens_plan_create_with(
            self._ptr, byref(spec._raw), byref(options), byref(out)))
        return Bf16RopePagedKvAppendTokensPlan(out.value, spec)


class _AppendPlan:
    def __init__(self, ptr, spec):
        self._ptr, self._spec = ptr, spec
        self._info = _abi.AppendPlanInfo()
        _check(_abi.load().lb_rope_append_plan_info_get(ptr, byref(self._info)))

    def __del__(self):
        _dispose(self, "lb_rope_append_plan_destroy")

    def spec(self): return self._spec
    def info(self): return self._info
    def commands(self): return self._info.commands
    def workspace_required_numel(self): return self._info.workspace_numel


class Bf16RopePagedKvAppendPlan(_AppendPlan):
    """rope/mod.rs:745-831."""

    def enqueue_into(self, scope: CommandScope, args: Bf16RopePagedKvAppendArgs):
        raw = _abi.AppendArgs(
            query=args.query._raw, key=args.key._raw, value=args.value._raw,
            batch_indices=_null_handle(), positions=_null_handle(),
            page_indptr=args.page_indptr._raw, page_indices=args.page_indices._raw,
            last_page_len=args.last_page_len._raw, query_output=args.query_output._raw,
            key_pages=args.key_pages._raw, value_pages=args.value_pages._raw)
        _check(_abi.load().lb_rope_append_enqueue(self._ptr, scope._ptr, byref(raw)))


class Bf16RopePagedKvAppendTokensPlan(_AppendPlan):
    """rope/mod.rs:833-934."""

    def enqueue_into(self, scope: CommandScope, args: Bf16RopePagedKvAppendTokensArgs):
        raw = _abi.AppendArgs(
            query=args.query._raw, key=args.key._raw, value=args.value._raw,
            batch_indices=args.batch_indices._raw, positions=args.positions._raw,
            page_indptr=args.page_indptr._raw, page_indices=args.page_indices._raw,
            last_page_len=args.last_page_len._raw, query_output=args.query_output._raw,
            key_pages=args.key_pages._raw, value_pages=args.value_pages._raw,
            workspace=args.workspace._raw if args.workspace is not None else _null_handle())
        _check(_abi.load().lb_rope_append_enqueue(self._ptr, scope._ptr, byref(raw)))


# ---- fixed-address CUDA Graph -------------------------------------------------------------------------------


class GraphQueue:
    """graph/mod.rs:27-71: capture-only queue with a private stream."""

    def __init__(self, device: int, max_commands: int):
        out = c_void_p()
        _check(_abi.load().lb_graph_queue_create(device, max_commands, byref(out)))
        self._ptr = out.value

    def __del__(self):
        _dispose(self, "lb_graph_queue_destroy")

    def bindings(self, capacity: int) -> CheckedBindings:
        out = c_void_p()
        _check(_abi.load().lb_graph_queue_bindings(self._ptr, capacity, byref(out)))
        return CheckedBindings(out.value)

    def capture(self, bindings: CheckedBindings,
                record: Callable[[CommandScope], None]) -> "CapturedGraph":
        """Consumes the queue and the bindings.  `record` enqueues plans into the scope; an
        exception it raises aborts the capture and is re-raised."""
        buffers = bindings._buffers
        raised = []

        def trampoline(scope_ptr, _user):
            scope = CommandScope(None, scope_ptr, buffers)
            try:
                record(scope)
                return 0
            except LoomError as error:
                raised.append(error)
                return error.status
            except Exception as error:  # noqa: BLE001 - reported to the caller below
                raised.append(error)
                return 500
            finally:
                scope._ptr = None  # the library owns the scope during capture

        callback = _abi.RECORD_FN(trampoline)
        out = c_void_p()
        queue_ptr, self._ptr = self._ptr, None
        # no finaliser runs while the stream is capturing: one that frees device memory (an old
        # provider, a tensor) in this thread would invalidate the capture
        collecting = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            status = _abi.load().lb_graph_capture(queue_ptr, bindings._release(), callback, None,
                                                  byref(out))
        finally:
            if collecting:
                gc.enable()
        if raised:
            raise raised[0]
        _check(status)
        return CapturedGraph(out.value, buffers)


class CapturedGraph:
    """graph/mod.rs:165-215."""

    def __init__(self, ptr, buffers):
        self._ptr, self._buffers = ptr, buffers

    def __del__(self):
        _dispose(self, "lb_captured_graph_destroy")

    def commands(self): return _abi.load().lb_captured_graph_commands(self._ptr)

    def instantiate(self) -> "GraphExec":
        out = c_void_p()
        ptr, self._ptr = self._ptr, None
        _check(_abi.load().lb_captured_graph_instantiate(ptr, byref(out)))
        return GraphExec(out.value, self._buffers)


class GraphExec:
    """graph/mod.rs:217-382."""

    def __init__(self, ptr, buffers):
        self._ptr, self._buffers = ptr, buffers

    def __del__(self):
        _dispose(self, "lb_graph_exec_destroy")

    def commands(self): return _abi.load().lb_graph_exec_commands(self._ptr)
    def launches(self): return _abi.load().lb_graph_exec_launches(self._ptr)

    def launch(self) -> "GraphLaunchCompletion":
        out = c_void_p()
        _check(_abi.load().lb_graph_exec_launch(self._ptr, byref(out)))
        return GraphLaunchCompletion(out.value, self)

    def measure_launch_ms(self) -> float:
        ms = c_float()
        _check(_abi.load().lb_graph_exec_measure_launch_ms(self._ptr, byref(ms)))
        return ms.value

    def into_bindings(self) -> CheckedBindings:
        out = c_void_p()
        ptr, self._ptr = self._ptr, None
        _check(_abi.load().lb_graph_exec_into_bindings(ptr, byref(out)))
        bindings = CheckedBindings(out.value)
        bindings._buffers = self._buffers
        return bindings


class GraphLaunchCompletion:
    """graph/mod.rs:384-463."""

    def __init__(self, ptr, exec_):
        self._ptr, self._exec = ptr, exec_

    def __del__(self):
        _dispose(self, "lb_graph_completion_abandon")

    def launch_index(self): return _abi.load().lb_graph_completion_launch_index(self._ptr)

    def is_complete(self) -> bool:
        done = c_int()
        _check(_abi.load().lb_graph_completion_is_complete(self._ptr, byref(done)))
        return bool(done.value)

    def wait(self):
        ptr, self._ptr = self._ptr, None
        _check(_abi.load().lb_graph_completion_wait(ptr))
