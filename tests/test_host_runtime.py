"""Host logic without a GPU: the C ABI loads and exports every declared symbol, the contract
layer matches the reference's CPU-side tests, the plan heuristic is a pure function, and the
command / graph ownership and poisoning state machine runs against the in-process fake driver
(no kernel ever runs under the fake).

Cases follow crates/loom-infer/src/attention/paged_decode/tests.rs, .../paged_append/tests.rs,
crates/loom-infer-cuda/src/command/resolve.rs:1095-1125 and the preflight parts of
crates/loom-infer-validation/src/gates/{paged_batch_decode,single_decode,rope}.rs.
"""
import ctypes
import gc
import os
import re

import pytest

import loom_kernels_b200 as lk
from loom_kernels_b200 import _abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
D = lk.DeviceSpan
CUDA_ERROR_LAUNCH_FAILURE = 719


@pytest.fixture()
def fake():
    lib = _abi.load()
    lib.lb_test_use_fake_driver(1, 148)
    yield lib
    gc.collect()  # objects made under the fake hold fake handles: release them under the fake
    lib.lb_test_use_fake_driver(0, 0)


def test_library_exports_every_symbol_the_header_declares():
    header = open(os.path.join(ROOT, "include", "loom_b200.h")).read()
    declared = set(re.findall(r"\b(lb_[a-z0-9_]+)\s*\(", header))
    declared -= {"lb_record_fn", "lb_status"}  # the callback typedef
    lib = _abi.load()
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing
    assert declared == set(_abi.SIGNATURES), declared ^ set(_abi.SIGNATURES)
    assert b"sm_100a" in lib.lb_build_info()


def test_spec_contract():
    spec = lk.Bf16PagedBatchDecodeSpec.new(3, 7, 8, 2)
    assert (spec.batch_size(), spec.max_num_pages(), spec.gqa_group_size()) == (3, 7, 4)
    assert [spec.kv_head_for_query_head(h) for h in (0, 3, 4, 7, 8)] == [0, 0, 1, 1, None]
    assert spec.query_numel() == 3 * 8 * 128 and spec.kv_pages_numel() == 7 * 16 * 2 * 128
    assert spec.lse_numel() == 24 and spec.page_indptr_numel() == 4
    assert abs(spec.softmax_scale() - 128 ** -0.5) < 1e-8  # F32 1/sqrt(128)
    for dims in [(0, 1, 1, 1, 128, 16), (1, 1, 1, 1, 0, 16), (1, 1, 1, 1, 128, 0)]:
        with pytest.raises(lk.ContractError) as e:
            lk.Bf16PagedBatchDecodeSpec.new(*dims)
        assert e.value.variant == "ZeroDimension"
    for dims, variant, payload in [((1, 1, 1, 1, 64, 16), "UnsupportedHeadDimension", (128, 64)),
                                   ((1, 1, 1, 1, 128, 8), "UnsupportedPageSize", (16, 8)),
                                   ((1, 1, 6, 4, 128, 16), "InvalidHeadMapping", (6, 4))]:
        with pytest.raises(lk.ContractError) as e:
            lk.Bf16PagedBatchDecodeSpec.new(*dims)
        assert (e.value.variant, e.value.payload[:2]) == (variant, payload)
    with pytest.raises(lk.ContractError) as e:
        lk.Bf16PagedBatchDecodeSpec.new(2 ** 64 - 1, 1, 1, 1)
    assert e.value.variant == "ElementCountOverflow"


def test_page_table_view_and_errors():
    spec = lk.Bf16PagedBatchDecodeSpec.new(3, 8, 4, 2)
    table = spec.validate_page_table([0, 2, 3, 6], [5, 1, 7, 2, 0, 6], [3, 16, 1])
    assert [table.request_kv_len(r) for r in range(4)] == [19, 16, 33, None]
    assert table.request_page_range(2) == (3, 6) and table.request_page_range(3) is None
    assert table.physical_page_for_token(0, 18) == (1, 2)
    assert table.physical_page_for_token(0, 19) is None
    assert table.physical_page_for_token(2, 32) == (6, 0)
    spec = lk.Bf16PagedBatchDecodeSpec.new(2, 4, 4, 2)
    cases = [
        (([0, 1], [0, 1], [16, 16]), "LengthMismatch", "page_indptr", (3, 2)),
        (([0, 1, 2], [0, 1], [16]), "LengthMismatch", "last_page_len", (2, 1)),
        (([1, 2, 3], [0, 1, 2], [16, 16]), "InvalidPageIndptrStart", "", (1,)),
        (([0, 2, 1], [0], [16, 16]), "NonMonotonicPageIndptr", "", (1, 2, 1)),
        (([0, 0, 1], [0], [16, 16]), "EmptyPagedRequest", "", (0,)),
        (([0, 1, 2], [0, 1], [16, 17]), "InvalidLastPageLength", "", (1, 17, 16)),
        (([0, 1, 2], [0], [16, 16]), "LengthMismatch", "page_indices", (2, 1)),
        (([0, 1, 2], [0, 4], [16, 16]), "PageIndexOutOfRange", "", (1, 4, 4)),
    ]
    for args, variant, operand, payload in cases:
        with pytest.raises(lk.ContractError) as e:
            spec.validate_page_table(*args)
        assert (e.value.variant, e.value.operand, e.value.payload[:len(payload)]) == \
            (variant, operand, payload)
    assert "page indptr must start at zero, got 1" in str(
        pytest.raises(lk.ContractError, spec.validate_page_table, [1, 2, 3], [0, 1, 2],
                      [16, 16]).value)


def test_append_contract():
    spec = lk.Bf16RopePagedKvAppendSpec.new(2, 2, 2, 1)
    with pytest.raises(lk.ContractError) as e:
        spec.validate_page_table([0, 1, 2], [1, 1], [4, 4])
    assert (e.value.variant, e.value.payload) == ("DuplicatePageAppendSlot", (0, 1, 1, 3))
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new(6, 3, 8, 4, 2)
    slots = spec.validate_metadata([2, 0, 1, 0, 2, 1], [17, 3, 20, 16, 16, 19], [0, 2, 4, 6],
                                   [7, 3, 2, 6, 3, 1], [5, 8, 4])
    assert slots == [(1, 1), (7, 3), (6, 4), (3, 0), (1, 0), (6, 3)]
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new(2, 2, 4, 2, 1)
    table = ([0, 2, 4], [3, 1, 3, 2], [4, 4])
    for batch_indices, positions, variant, payload in [
            ([0, 2], [1, 17], "AppendBatchIndexOutOfRange", (1, 2, 2, 0)),
            ([0, 1], [1, 20], "AppendPositionOutOfRange", (1, 1, 20, 20)),
            ([0, 1], [2, 2], "DuplicatePageAppendTokenSlot", (0, 1, 3, 2))]:
        with pytest.raises(lk.ContractError) as e:
            spec.validate_metadata(batch_indices, positions, *table)
        assert (e.value.variant, e.value.payload) == (variant, payload)
    with pytest.raises(lk.ContractError) as e:
        lk.Bf16RopePagedKvAppendTokensSpec.new(65, 1, 1, 1, 1)
    assert (e.value.variant, e.value.payload[:2]) == ("UnsupportedAppendTokenCount", (64, 65))
    assert lk.Bf16RopePagedKvAppendTokensSpec.new_extended(1040, 32, 8192, 32, 8).tokens() == 1040


def test_split_contract_pieces():
    assert [lk.split_partition_range(10, 4, p) for p in range(5)] == \
        [(0, 3), (3, 6), (6, 8), (8, 10), None]
    spec = lk.Bf16PagedBatchDecodeSpec.new(8, 20000, 64, 8)
    assert lk.paged_split_workspace_numel(spec, 16) == 8 * 64 * 16 * 130
    assert lk.paged_split_state_offset(spec, 16, 0, 0, 3) == 3 * 130
    assert lk.paged_split_state_offset(spec, 16, 1, 2, 0) == ((64 + 2) * 16) * 130
    assert lk.paged_split_state_offset(spec, 16, 8, 0, 0) is None
    with pytest.raises(lk.ContractError) as e:
        lk.paged_split_workspace_numel(spec, 0)
    assert e.value.variant == "InvalidPartitionCount"


def test_plan_heuristic_is_fixed_by_spec_and_device():
    c3 = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(64, 20000, 32, 8), 148,
                                partitions=1)
    assert (c3.partitions, c3.algorithm, c3.commands, c3.workspace_numel) == (1, 0, 1, 0)
    assert c3.grid == 64 * (8 // c3.heads_per_cta) and c3.block == 288
    # left to itself the plan cuts a batch smaller than the device by pages, one CTA per SM
    auto = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(64, 20000, 32, 8), 148)
    assert (auto.algorithm, auto.commands, auto.grid, auto.heads_per_cta) == (2, 2, 148, 8)
    assert auto.merged_in_kernel == 0 and auto.merge_grid == 512
    assert auto.workspace_numel == 148 * 2 * 8 * 4 * 130 + 64 + 8
    # on request the cut items are merged in the decode kernel: one command, the same workspace
    one = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(64, 20000, 32, 8), 148,
                                 merge_in_kernel=1)
    assert (one.algorithm, one.commands, one.merged_in_kernel, one.merge_grid) == (2, 1, 1, 0)
    assert one.workspace_numel == auto.workspace_numel
    # few requests on many workers: dozens of states per item, a CTA of the merge kernel each
    few = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(32, 65536, 32, 1), 148)
    assert (few.algorithm, few.commands, few.merged_in_kernel, few.merge_grid) == (2, 2, 0, 1024)
    many = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(4096, 65536, 32, 8), 148)
    assert (many.algorithm, many.commands) == (0, 1)  # thousands of requests tile the device
    c4 = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(8, 20000, 64, 8), 148,
                                partitions=16)
    assert (c4.partitions, c4.algorithm, c4.commands, c4.merged_in_kernel) == (16, 1, 2, 0)
    assert c4.workspace_numel == 8 * 64 * 16 * 130 and c4.merge_grid == 8 * 64 // 4
    # on request the last CTA of every item merges it: one command, the workspace stays
    one = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(8, 20000, 64, 8), 148,
                                 partitions=16, merge_in_kernel=1)
    assert (one.commands, one.merged_in_kernel, one.merge_grid) == (1, 1, 0)
    assert one.workspace_numel == c4.workspace_numel
    with pytest.raises(lk.PlanError):  # more items than a queue has counting words
        lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(40000, 2000000, 8, 8), 148,
                               partitions=2, heads_per_cta=8, merge_in_kernel=1)
    with pytest.raises(lk.PlanError):  # nothing to merge
        lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(64, 20000, 32, 8), 148,
                               partitions=1, merge_in_kernel=1)
    c1 = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(1, 256, 32, 32), 148, balanced=2)
    assert c1.partitions > 1 and c1.grid >= 64  # one request cannot fill 148 SMs unsplit
    mqa = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(256, 65536, 32, 1), 148)
    assert mqa.q_tiles == 2 and mqa.heads_per_cta == 1  # group 32 = two 16-row MMA tiles
    wide = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(2, 64, 160, 1), 148)
    assert (wide.q_tiles, wide.q_blocks) == (8, 2)
    with pytest.raises(lk.PlanError):
        lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(2, 64, 8, 2), 148, heads_per_cta=8)
    # same inputs, same plan
    again = lk.choose_paged_decode(lk.Bf16PagedBatchDecodeSpec.new(64, 20000, 32, 8), 148)
    assert (again.heads_per_cta, again.grid, again.stages) == (auto.heads_per_cta, auto.grid, auto.stages)


# ---- command runtime against the fake driver ---------------------------------------------------


def decode_setup(queue, spec, capacity=9, short=None, device_bit=0):
    b = queue.bindings(capacity)
    base = 0x10000000 | (device_bit << 40)
    sizes = dict(query=spec.query_numel(), key_pages=spec.kv_pages_numel(),
                 value_pages=spec.kv_pages_numel(), page_indptr=spec.batch_size() + 1,
                 page_indices=8, last_page_len=spec.batch_size())
    if short:
        sizes[short] -= 1
    h = {}
    for i, (name, numel) in enumerate(sizes.items()):
        dtype = _abi.I32 if "page_" in name or name == "last_page_len" else _abi.BF16
        h[name] = b.bind_read(D(base + i * 0x1000000, numel, dtype))
    out = b.bind_read_write(D(base + 0x7000000, spec.output_numel(), _abi.BF16))
    lse = b.bind_read_write(D(base + 0x8000000, spec.lse_numel(), _abi.F32))
    return b, h, out, lse


def test_queue_and_binding_errors(fake):
    with pytest.raises(lk.CommandError) as e:
        lk.CommandQueue(0x100, 0)
    assert e.value.variant == "ZeroCommandCapacity"
    queue = lk.CommandQueue(0x100, 1)
    assert queue.max_commands() == 1
    with pytest.raises(lk.CommandError) as e:
        queue.bindings(0)
    assert e.value.variant == "ZeroBindingCapacity"
    b = queue.bindings(1)
    assert (b.capacity(), len(b)) == (1, 0)
    h = b.bind_read(D(0x1000, 4, _abi.F32))
    with pytest.raises(lk.CommandError) as e:
        b.bind_read(D(0x2000, 4, _abi.F32))
    assert (e.value.variant, e.value.payload[0]) == ("BindingCapacityExceeded", 1)
    with pytest.raises(lk.CommandError) as e:  # a buffer of device 1 on a device-0 queue
        queue.bindings(1).bind_read(D((1 << 40) | 0x1000, 4, _abi.F32))
    assert (e.value.variant, e.value.payload[:2]) == ("BufferContextMismatch", (1, 0))
    with pytest.raises(lk.CommandError) as e:
        b.take_read_write(lk.ReadWrite(h._raw))
    assert e.value.variant == "BindingIsReadOnly"
    other = lk.CommandQueue(0x200, 1)
    with pytest.raises(lk.CommandError) as e:
        other.begin(queue.bindings(1))
    assert e.value.variant == "BindingsQueueMismatch"


def test_decode_enqueue_preflight_and_resolution(fake):
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 8, 16, 4)
    provider = lk.DecodeProvider.load(0)
    plan = provider.plan_bf16_paged_batch(spec, partitions=1)
    queue = lk.CommandQueue(0x100, 2)

    def args(h, out, lse, **override):
        fields = dict(h, output=out.write(), lse=lse.write())
        fields.update(override)
        return lk.Bf16PagedBatchDecodeArgs(**fields)

    # every short operand is named, and nothing is submitted (paged_batch_decode.rs:150-222)
    for operand, name in [("query", "Q"), ("key_pages", "K_pages"), ("value_pages", "V_pages"),
                          ("page_indptr", "page_indptr"), ("last_page_len", "last_page_len")]:
        b, h, out, lse = decode_setup(queue, spec, short=operand)
        scope = queue.begin(b)
        with pytest.raises(lk.EnqueueError) as e:
            plan.enqueue_into(scope, args(h, out, lse))
        assert (e.value.variant, e.value.operand) == ("LengthMismatch", name)
        completion = scope.finish()
        assert completion.submitted() == 0 and completion.is_complete()
        completion.wait()
    assert fake.lb_test_launch_count() == 0

    b, h, out, lse = decode_setup(queue, spec, capacity=10)
    frozen = b.bind_read(D(0x19000000, spec.output_numel(), _abi.BF16))
    scope = queue.begin(b)
    with pytest.raises(lk.CommandError) as e:  # alias check: one slot for two operands
        plan.enqueue_into(scope, args(h, out, lse, value_pages=h["key_pages"]))
    assert e.value.variant == "DuplicateBindingSlot"
    with pytest.raises(lk.CommandError) as e:  # a read-only binding as the output
        plan.enqueue_into(scope, args(h, out, lse, output=lk.Write(frozen._raw)))
    assert e.value.variant == "BindingIsReadOnly"
    with pytest.raises(lk.CommandError) as e:  # element type
        plan.enqueue_into(scope, args(h, out, lse, page_indptr=h["query"], query=h["page_indptr"]))
    assert e.value.variant == "BindingTypeMismatch"
    foreign = queue.bindings(1).bind_read(D(0x9000, 4, _abi.BF16))
    with pytest.raises(lk.CommandError) as e:
        plan.enqueue_into(scope, args(h, out, lse, query=foreign))
    assert e.value.variant == "BindingSetMismatch"
    plan.enqueue_into(scope, args(h, out, lse))
    plan.enqueue_into(scope, args(h, out, lse))
    with pytest.raises(lk.CommandError) as e:
        plan.enqueue_into(scope, args(h, out, lse))
    assert (e.value.variant, e.value.payload[0]) == ("CommandCapacityExceeded", 2)
    completion = scope.finish()
    assert completion.submitted() == 2
    b = completion.wait()
    assert b.take_read_write(out).numel == spec.output_numel()
    with pytest.raises(lk.CommandError) as e:
        b.take_read_write(out)
    assert e.value.variant == "BindingSlotVacant"

    # misaligned base: the 16-byte rule of these kernels, reported like the reference's 4-byte one
    b = queue.bindings(9)
    h2 = dict(h)
    names = ["query", "key_pages", "value_pages", "page_indptr", "page_indices", "last_page_len"]
    sizes = [spec.query_numel(), spec.kv_pages_numel(), spec.kv_pages_numel(), 5, 8, 4]
    for i, (name, numel) in enumerate(zip(names, sizes)):
        dtype = _abi.I32 if i >= 3 else _abi.BF16
        h2[name] = b.bind_read(D(0x10000000 + i * 0x1000000 + (2 if name == "key_pages" else 0),
                                 numel, dtype))
    out = b.bind_read_write(D(0x17000000, spec.output_numel(), _abi.BF16))
    lse = b.bind_read_write(D(0x18000000, spec.lse_numel(), _abi.F32))
    scope = queue.begin(b)
    with pytest.raises(lk.EnqueueError) as e:
        plan.enqueue_into(scope, args(h2, out, lse))
    assert (e.value.variant, e.value.operand, e.value.payload[1]) == ("MisalignedBuffer", "K_pages", 16)
    scope.finish().wait()


def test_split_plan_reserves_both_commands_and_checks_workspace(fake):
    # single_decode.rs:416-513 shape: capacity for two commands before any launch
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 64, 16, 4)
    provider = lk.DecodeProvider.load(0)
    plan = provider.plan_bf16_paged_batch(spec, partitions=3)
    assert plan.commands() == 2 and plan.workspace_required_numel() == 4 * 16 * 3 * 130
    for max_commands, workspace_numel, variant in [(1, 4 * 16 * 3 * 130, "CommandCapacityExceeded"),
                                                   (2, 4 * 16 * 3 * 130 - 1, "LengthMismatch")]:
        queue = lk.CommandQueue(0x100, max_commands)
        b, h, out, lse = decode_setup(queue, spec, capacity=9)
        ws = b.bind_read_write(D(0x30000000, workspace_numel, _abi.F32))
        scope = queue.begin(b)
        with pytest.raises(lk.LoomError) as e:
            plan.enqueue_into(scope, lk.Bf16PagedBatchDecodeArgs(output=out.write(),
                                                                 lse=lse.write(), workspace=ws, **h))
        assert e.value.variant == variant
        assert scope.finish().submitted() == 0
    queue = lk.CommandQueue(0x100, 2)
    b, h, out, lse = decode_setup(queue, spec, capacity=9)
    ws = b.bind_read_write(D(0x30000000, 4 * 16 * 3 * 130, _abi.F32))
    scope = queue.begin(b)
    before = fake.lb_test_launch_count()
    plan.enqueue_into(scope, lk.Bf16PagedBatchDecodeArgs(output=out.write(), lse=lse.write(),
                                                         workspace=ws, **h))
    assert fake.lb_test_launch_count() - before == 2
    assert scope.finish().submitted() == 2
    # merged by the last CTA of every item: one command, same workspace
    fused = provider.plan_bf16_paged_batch(spec, partitions=3, merge_in_kernel=1)
    assert fused.commands() == 1 and fused.merged_in_kernel()
    assert fused.workspace_required_numel() == 4 * 16 * 3 * 130
    queue = lk.CommandQueue(0x100, 1)
    b, h, out, lse = decode_setup(queue, spec, capacity=9)
    ws = b.bind_read_write(D(0x30000000, 4 * 16 * 3 * 130, _abi.F32))
    scope = queue.begin(b)
    before = fake.lb_test_launch_count()
    fused.enqueue_into(scope, lk.Bf16PagedBatchDecodeArgs(output=out.write(), lse=lse.write(),
                                                          workspace=ws, **h))
    assert fake.lb_test_launch_count() - before == 1
    assert scope.finish().submitted() == 1


def test_launch_failure_poisons_scope_and_queue(fake):
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 8, 16, 4)
    plan = lk.DecodeProvider.load(0).plan_bf16_paged_batch(spec)
    queue = lk.CommandQueue(0x100, 4)
    b, h, out, lse = decode_setup(queue, spec)
    scope = queue.begin(b)
    a = lk.Bf16PagedBatchDecodeArgs(output=out.write(), lse=lse.write(), **h)
    plan.enqueue_into(scope, a)
    fake.lb_test_fake_fail(b"launch", 1, CUDA_ERROR_LAUNCH_FAILURE)
    with pytest.raises(lk.CommandError) as e:
        plan.enqueue_into(scope, a)
    assert (e.value.variant, e.value.payload[0]) == ("Driver", CUDA_ERROR_LAUNCH_FAILURE)
    with pytest.raises(lk.CommandError) as e:
        plan.enqueue_into(scope, a)
    assert e.value.variant == "ScopePoisoned"
    completion = scope.finish()
    assert completion.submitted() == 2  # the failed launch still counts as possibly submitted
    with pytest.raises(lk.CommandError):
        completion.is_complete()
    with pytest.raises(lk.CommandError) as e:
        completion.wait()
    assert e.value.payload[0] == CUDA_ERROR_LAUNCH_FAILURE
    assert queue.is_poisoned()
    with pytest.raises(lk.CommandError) as e:
        queue.begin(queue.bindings(1))
    assert e.value.variant == "QueuePoisoned"


def test_completion_event_failure_poisons_the_queue(fake):
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 8, 16, 4)
    plan = lk.DecodeProvider.load(0).plan_bf16_paged_batch(spec)
    queue = lk.CommandQueue(0x100, 2)
    b, h, out, lse = decode_setup(queue, spec)
    scope = queue.begin(b)
    plan.enqueue_into(scope, lk.Bf16PagedBatchDecodeArgs(output=out.write(), lse=lse.write(), **h))
    completion = scope.finish()
    fake.lb_test_fake_fail(b"event_sync", 1, 700)
    with pytest.raises(lk.CommandError):
        completion.wait()
    assert queue.is_poisoned()


def test_one_live_scope_per_queue_and_abandon_settles(fake):
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 8, 16, 4)
    plan = lk.DecodeProvider.load(0).plan_bf16_paged_batch(spec)
    queue = lk.CommandQueue(0x100, 2)
    b, h, out, lse = decode_setup(queue, spec)
    scope = queue.begin(b)
    second = queue.bindings(1)
    with pytest.raises(lk.LoomError) as e:
        queue.begin(second)
    assert e.value.variant == "ObjectInUse"
    plan.enqueue_into(scope, lk.Bf16PagedBatchDecodeArgs(output=out.write(), lse=lse.write(), **h))
    del scope  # dropping an unfinished scope synchronises and frees the queue
    scope = queue.begin(second)
    completion = scope.finish()
    del completion  # dropping a completion settles it
    assert not queue.is_poisoned()
    queue.begin(queue.bindings(1)).finish().wait()


def test_rope_append_enqueue_preflight(fake):
    provider = lk.RopeProvider.load(0)
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new(6, 3, 8, 16, 4)
    plan = provider.plan_bf16_paged_append_tokens(spec)
    assert plan.info().commands == 1 and plan.info().grid == 6
    queue = lk.CommandQueue(0x100, 1)
    names = ["query", "key", "value", "batch_indices", "positions", "page_indptr", "page_indices",
             "last_page_len"]
    sizes = [6 * 16 * 128, 6 * 4 * 128, 6 * 4 * 128, 6, 6, 4, 5, 3]

    def setup(short=None):
        b = queue.bindings(11)
        h = {}
        for i, (name, numel) in enumerate(zip(names, sizes)):
            dtype = _abi.BF16 if i < 3 else _abi.I32
            h[name] = b.bind_read(D(0x20000000 + i * 0x1000000, numel - (name == short), dtype))
        q = b.bind_read_write(D(0x2a000000, 6 * 16 * 128, _abi.BF16))
        k = b.bind_read_write(D(0x2b000000, spec.kv_pages_numel() - (short == "key_pages"), _abi.BF16))
        v = b.bind_read_write(D(0x2c000000, spec.kv_pages_numel(), _abi.BF16))
        return b, lk.Bf16RopePagedKvAppendTokensArgs(query_output=q.write(), key_pages=k.write(),
                                                     value_pages=v.write(), **h)

    for short in ["query", "key", "value", "batch_indices", "positions", "page_indptr",
                  "last_page_len", "key_pages"]:
        b, a = setup(short)
        scope = queue.begin(b)
        with pytest.raises(lk.EnqueueError) as e:
            plan.enqueue_into(scope, a)
        assert (e.value.variant, e.value.operand) == ("LengthMismatch", short)
        assert scope.finish().submitted() == 0
    b, a = setup()
    scope = queue.begin(b)
    plan.enqueue_into(scope, a)
    with pytest.raises(lk.CommandError) as e:
        plan.enqueue_into(scope, a)
    assert (e.value.variant, e.value.payload[0]) == ("CommandCapacityExceeded", 1)
    assert scope.finish().submitted() == 1
    with pytest.raises(lk.ContractError):
        provider.plan_bf16_paged_append_tokens(lk.Bf16RopePagedKvAppendTokensSpec.new(65, 1, 4, 1, 1))


def test_extended_append_as_one_command_or_two(fake):
    """The any-total append: two commands (validate, scatter) by default, one on request; both
    need the workspace, and the one-command form fits a queue of one command."""
    provider = lk.RopeProvider.load(0)
    spec = lk.Bf16RopePagedKvAppendTokensSpec.new_extended(100, 4, 96, 16, 4)
    sizes = [100 * 16 * 128, 100 * 4 * 128, 100 * 4 * 128, 100, 100, 5, 40, 4]
    names = ["query", "key", "value", "batch_indices", "positions", "page_indptr", "page_indices",
             "last_page_len"]
    for one_command, commands in ((False, 2), (True, 1)):
        plan = provider.plan_bf16_paged_append_tokens(spec, one_command=one_command)
        assert plan.info().commands == commands and plan.workspace_required_numel() == 32 + 200
        queue = lk.CommandQueue(0x100, commands)
        b = queue.bindings(12)
        h = {}
        for i, (name, numel) in enumerate(zip(names, sizes)):
            h[name] = b.bind_read(D(0x20000000 + i * 0x1000000, numel,
                                    _abi.BF16 if i < 3 else _abi.I32))
        q = b.bind_read_write(D(0x2a000000, 100 * 16 * 128, _abi.BF16))
        k = b.bind_read_write(D(0x2b000000, spec.kv_pages_numel(), _abi.BF16))
        v = b.bind_read_write(D(0x2c000000, spec.kv_pages_numel(), _abi.BF16))
        ws = b.bind_read_write(D(0x2d000000, 32 + 200, _abi.I32))
        args = lk.Bf16RopePagedKvAppendTokensArgs(query_output=q.write(), key_pages=k.write(),
                                                  value_pages=v.write(), workspace=ws, **h)
        scope = queue.begin(b)
        before = fake.lb_test_launch_count()
        plan.enqueue_into(scope, args)
        assert fake.lb_test_launch_count() - before == commands
        with pytest.raises(lk.CommandError) as e:  # the queue is full
            plan.enqueue_into(scope, args)
        assert e.value.variant == "CommandCapacityExceeded"
        assert scope.finish().submitted() == commands


def test_rope_pos_ids_contract_and_preflight(fake):
    """Bf16RopePosIdsSpec::new (crates/loom-infer/src/rope/mod.rs:21-62), plan_bf16_pos_ids
    (crates/loom-infer-cuda/src/rope/mod.rs:592-626) and the enqueue preflight (:698-742)."""
    for args, variant in [((0, 16, 4), "ZeroDimension"), ((5, 0, 4), "ZeroDimension"),
                          ((5, 16, 4, 128, 0), "InvalidRotaryDimension"),
                          ((5, 16, 4, 128, 63), "InvalidRotaryDimension"),
                          ((5, 16, 4, 128, 130), "InvalidRotaryDimension"),
                          ((5, 16, 4, 128, 128, 0.0), "InvalidRopeScale"),
                          ((5, 16, 4, 128, 128, float("inf")), "InvalidRopeScale"),
                          ((5, 16, 4, 128, 128, 1.0, 1.0), "InvalidRopeTheta"),
                          ((5, 16, 4, 128, 128, 1.0, float("nan")), "InvalidRopeTheta"),
                          ((2 ** 62, 16, 4), "ElementCountOverflow")]:
        with pytest.raises(lk.ContractError) as e:
            lk.Bf16RopePosIdsSpec.new(*args)
        assert e.value.variant == variant, args
    spec = lk.Bf16RopePosIdsSpec.new(5, 16, 4, 128, 128, 1.0, 10000.0)
    assert (spec.query_numel(), spec.key_numel(), spec.position_numel()) == (10240, 2560, 5)
    provider = lk.RopeProvider.load(0)
    with pytest.raises(lk.LoomError) as e:  # partial rotary dimension: rejected before submission
        provider.plan_bf16_pos_ids(lk.Bf16RopePosIdsSpec.new(5, 16, 4, 128, 64))
    assert (e.value.variant, e.value.payload[:2]) == ("UnsupportedRotaryDimension", (128, 64))
    with pytest.raises(lk.LoomError) as e:
        provider.plan_bf16_pos_ids(lk.Bf16RopePosIdsSpec.new(5, 16, 4, 64, 64))
    assert (e.value.variant, e.value.payload[:2]) == ("UnsupportedHeadDimension", (128, 64))
    plan = provider.plan_bf16_pos_ids(spec)
    queue = lk.CommandQueue(0x100, 1)
    names = ["query", "key", "position_ids", "query_output", "key_output"]
    sizes = [10240, 2560, 5, 10240, 2560]

    def setup(short=None):
        b = queue.bindings(5)
        h = []
        for i, (name, numel) in enumerate(zip(names, sizes)):
            span = D(0x30000000 + i * 0x1000000, numel - (name == short),
                     _abi.I32 if name == "position_ids" else _abi.BF16)
            h.append(b.bind_read(span) if i < 3 else b.bind_read_write(span).write())
        return b, lk.Bf16RopePosIdsArgs(*h)

    for short in names:
        b, a = setup(short)
        scope = queue.begin(b)
        with pytest.raises(lk.EnqueueError) as e:
            plan.enqueue_into(scope, a)
        assert (e.value.variant, e.value.operand) == ("LengthMismatch", short)
        assert scope.finish().submitted() == 0
    b, a = setup()
    scope = queue.begin(b)
    plan.enqueue_into(scope, a)
    assert scope.finish().submitted() == 1


# ---- graph state machine against the fake driver --------------------------------------------------


def graph_setup(spec, max_commands=2):
    gq = lk.GraphQueue(0, max_commands)
    b = gq.bindings(9)
    base = 0x10000000
    sizes = [spec.query_numel(), spec.kv_pages_numel(), spec.kv_pages_numel(),
             spec.batch_size() + 1, 8, spec.batch_size()]
    reads = [b.bind_read(D(base + i * 0x1000000, n, _abi.BF16 if i < 3 else _abi.I32))
             for i, n in enumerate(sizes)]
    out = b.bind_read_write(D(base + 0x7000000, spec.output_numel(), _abi.BF16))
    lse = b.bind_read_write(D(base + 0x8000000, spec.lse_numel(), _abi.F32))
    return gq, b, lk.Bf16PagedBatchDecodeArgs(*reads, out.write(), lse.write()), out


def test_graph_capture_replay_and_ownership(fake):
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 8, 16, 4)
    plan = lk.DecodeProvider.load(0).plan_bf16_paged_batch(spec)
    gq, b, a, out = graph_setup(spec)
    captured = gq.capture(b, lambda scope: plan.enqueue_into(scope, a))
    assert captured.commands() == 1
    del plan  # external owners may go away before replay (graph/mod.rs docs, rope.rs:780-789)
    exec_ = captured.instantiate()
    assert (exec_.commands(), exec_.launches()) == (1, 0)
    completion = exec_.launch()
    assert completion.launch_index() == 1 and completion.is_complete()
    with pytest.raises(lk.GraphError) as e:  # one replay in flight
        exec_.launch()
    assert e.value.variant == "ReplayInFlight"
    completion.wait()
    second = exec_.launch()
    del second  # dropping the completion settles the replay too
    assert exec_.launches() == 2
    assert exec_.measure_launch_ms() > 0 and exec_.launches() == 3
    bindings = exec_.into_bindings()
    assert bindings.take_read_write(out).numel == spec.output_numel()


def test_graph_capture_errors(fake):
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 8, 16, 4)
    plan = lk.DecodeProvider.load(0).plan_bf16_paged_batch(spec)
    gq, b, a, _ = graph_setup(spec)
    with pytest.raises(lk.GraphError) as e:
        gq.capture(b, lambda scope: None)
    assert e.value.variant == "EmptyCapture"
    gq, b, a, _ = graph_setup(spec)

    def failing(scope):
        plan.enqueue_into(scope, a)
        raise ValueError("record closure failed")

    with pytest.raises(ValueError):
        gq.capture(b, failing)
    gq, b, a, _ = graph_setup(spec, max_commands=1)

    def too_many(scope):
        plan.enqueue_into(scope, a)
        plan.enqueue_into(scope, a)

    with pytest.raises(lk.CommandError) as e:
        gq.capture(b, too_many)
    assert e.value.variant == "CommandCapacityExceeded"
    gq, b, a, _ = graph_setup(spec)
    fake.lb_test_fake_fail(b"capture_begin", 1, 900)
    with pytest.raises(lk.GraphError) as e:
        gq.capture(b, lambda scope: plan.enqueue_into(scope, a))
    assert (e.value.variant, e.value.operand) == ("GraphDriver", "capture begin")


def test_graph_replay_failure_poisons_the_executable(fake):
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 8, 16, 4)
    plan = lk.DecodeProvider.load(0).plan_bf16_paged_batch(spec)
    gq, b, a, _ = graph_setup(spec)
    exec_ = gq.capture(b, lambda scope: plan.enqueue_into(scope, a)).instantiate()
    fake.lb_test_fake_fail(b"graph_launch", 1, CUDA_ERROR_LAUNCH_FAILURE)
    with pytest.raises(lk.GraphError) as e:
        exec_.launch()
    assert (e.value.variant, e.value.operand, e.value.payload[0]) == \
        ("GraphDriver", "launch", CUDA_ERROR_LAUNCH_FAILURE)
    with pytest.raises(lk.GraphError) as e:
        exec_.launch()
    assert e.value.variant == "ExecutionPoisoned"
    gq, b, a, _ = graph_setup(spec)
    exec_ = gq.capture(b, lambda scope: plan.enqueue_into(scope, a)).instantiate()
    completion = exec_.launch()
    fake.lb_test_fake_fail(b"event_sync", 1, 700)
    with pytest.raises(lk.GraphError):
        completion.wait()
    with pytest.raises(lk.GraphError) as e:
        exec_.launch()
    assert e.value.variant == "ExecutionPoisoned"


def test_unsupported_device_and_missing_gpu_fail_loudly():
    # without the fake there is no device here: the provider must refuse, not fall back
    lib = _abi.load()
    lib.lb_test_use_fake_driver(0, 0)
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(lk.LoomError):
        lk.DecodeProvider.load(0)
    with pytest.raises(lk.LoomError):
        lk.RopeProvider.load(0)


def test_state_merge_plan_and_preflight(fake):
    provider = lk.DecodeProvider.load(0)
    for rows, partitions, variant in [(0, 4, "ZeroDimension"), (4, 0, "ZeroDimension"),
                                      (4, 65536, "InvalidPartitionCount"),
                                      (2 ** 31, 2, "StateCountOutOfRange")]:
        with pytest.raises(lk.LoomError) as e:
            provider.plan_state_merge(rows, partitions)
        assert e.value.variant == variant, (rows, partitions)
    plan = provider.plan_state_merge(6, 3)
    assert plan.states_numel() == 6 * 3 * 130
    queue = lk.CommandQueue(0x100, 1)
    for short, operand in [("states", "states"), ("output", "O"), ("lse", "LSE")]:
        b = queue.bindings(3)
        states = b.bind_read(D(0x40000000, plan.states_numel() - (short == "states"), _abi.F32))
        out = b.bind_read_write(D(0x41000000, 6 * 128 - (short == "output"), _abi.BF16))
        lse = b.bind_read_write(D(0x42000000, 6 - (short == "lse"), _abi.F32))
        scope = queue.begin(b)
        with pytest.raises(lk.EnqueueError) as e:
            plan.enqueue_into(scope, lk.StateMergeArgs(states, out.write(), lse.write()))
        assert (e.value.variant, e.value.operand) == ("LengthMismatch", operand)
        assert scope.finish().submitted() == 0
    b = queue.bindings(3)
    states = b.bind_read(D(0x40000000, plan.states_numel(), _abi.F32))
    out = b.bind_read_write(D(0x41000000, 6 * 128, _abi.BF16))
    lse = b.bind_read_write(D(0x42000000, 6, _abi.F32))
    scope = queue.begin(b)
    plan.enqueue_into(scope, lk.StateMergeArgs(states, out.write(), lse.write()))
    assert scope.finish().submitted() == 1


def test_indices_capacity_option_is_a_plan_property(fake):
    """The option only changes the device guard; plan shape and enqueue preflight are the same,
    and a value other than 0 or 1 is refused at plan time."""
    spec = lk.Bf16PagedBatchDecodeSpec.new(4, 96, 16, 4)
    decode, rope = lk.DecodeProvider.load(0), lk.RopeProvider.load(0)
    plain = decode.plan_bf16_paged_batch(spec, partitions=2)
    relaxed = decode.plan_bf16_paged_batch(spec, partitions=2, indices_capacity=True)
    assert (plain.commands(), plain.workspace_required_numel()) == \
        (relaxed.commands(), relaxed.workspace_required_numel())
    append_spec = lk.Bf16RopePagedKvAppendSpec.new(4, 96, 16, 4)
    assert rope.plan_bf16_paged_append(append_spec, indices_capacity=True).commands() == 1
    tokens_spec = lk.Bf16RopePagedKvAppendTokensSpec.new_extended(100, 4, 96, 16, 4)
    extended = rope.plan_bf16_paged_append_tokens(tokens_spec, indices_capacity=True)
    assert (extended.commands(), extended.workspace_required_numel()) == (2, 32 + 200)
    extended = rope.plan_bf16_paged_append_tokens(tokens_spec, indices_capacity=True,
                                                  one_command=True)
    assert (extended.commands(), extended.workspace_required_numel()) == (1, 32 + 200)
    with pytest.raises(lk.LoomError):  # a call too large for its whole grid to be resident
        rope.plan_bf16_paged_append_tokens(
            lk.Bf16RopePagedKvAppendTokensSpec.new_extended(4000, 4, 4096, 16, 4), one_command=True)
    lib = _abi.load()
    options = _abi.DecodeOptions(indices_capacity=2)
    out = ctypes.c_void_p()
    assert lib.lb_paged_decode_plan_create(decode._ptr, ctypes.byref(spec._raw),
                                           ctypes.byref(options), ctypes.byref(out)) != 0
    append_options = _abi.AppendOptions(indices_capacity=7)
    assert lib.lb_rope_append_plan_create_with(rope._ptr, ctypes.byref(spec._raw),
                                               ctypes.byref(append_options),
                                               ctypes.byref(out)) != 0


def test_noalloc_entry_under_the_fake_driver_caches_nothing(fake):
    """The no-workspace split-K entry resolves its static array once per GPU on the real driver.
    Under the fake there is no device to resolve it on, so a call must leave the per-GPU set-up
    untouched (a later real call still has to do it), while its checks and its two launches run as
    on a device."""
    lib = _abi.load()
    spec = lk.Bf16PagedBatchDecodeSpec.new(2, 40, 16, 4)
    stream = 0x1000  # fake stream of device 0
    q = D(0x40000000, spec.query_numel(), _abi.BF16)
    pool = spec.kv_pages_numel()
    k, v = D(0x41000000, pool, _abi.BF16), D(0x42000000, pool, _abi.BF16)
    indptr, indices, last = (D(0x43000000, 3, _abi.I32), D(0x43100000, 40, _abi.I32),
                             D(0x43200000, 2, _abi.I32))
    out, lse = D(0x44000000, spec.output_numel(), _abi.BF16), D(0x45000000, 32, _abi.F32)
    before = lib.lb_test_launch_count()
    lk.paged_decode_split_noalloc(spec, 4, stream, q, k, v, indptr, indices, last, out, lse)
    assert lib.lb_test_launch_count() == before + 2  # partial states, then the merge
    assert lib.lb_test_noalloc_is_set_up(0) == 0
    assert lk.paged_decode_split_noalloc_status(0) == 0
    # operand checks that need no device: lengths (in the wrapper), owner GPU, memory kind
    with pytest.raises(lk.EnqueueError) as e:
        lk.paged_decode_split_noalloc(spec, 4, stream, q, k, v, indptr, indices, last,
                                      D(0x44000000, 16, _abi.BF16), lse)
    assert (e.value.variant, e.value.operand, e.value.payload[:2]) == \
        ("LengthMismatch", "O", (spec.output_numel(), 16))
    other_gpu = D(0x41000000 | (1 << 40), pool, _abi.BF16)
    with pytest.raises(lk.CommandError) as e:
        lk.paged_decode_split_noalloc(spec, 4, stream, q, other_gpu, v, indptr, indices, last, out,
                                      lse)
    assert (e.value.variant, e.value.payload[:2]) == ("BufferContextMismatch", (1, 0))
    host_memory = D(0x45000000 | (1 << 41), 32, _abi.F32)
    with pytest.raises(lk.LoomError):
        lk.paged_decode_split_noalloc(spec, 4, stream, q, k, v, indptr, indices, last, out,
                                      host_memory)
    assert lib.lb_test_launch_count() == before + 2
    assert lib.lb_test_noalloc_is_set_up(0) == 0


def test_gathering_commands_under_the_fake_driver(fake):
    """Bookkeeping of the two ways to leave output rows gathered on every rank: the library
    all-gather recorded as one external command (a failure poisons the queue, as the reference's
    record_failed_external_submission), and the decode whose own kernels store the rows into the
    peers' buffers (same command count as the plain enqueue, operands checked before any launch)."""
    lib = _abi.load()
    group = lk.PeerGroup(0, 2, 1, lk.PeerGroup.unique_id())
    assert (group.rank(), group.world()) == (1, 2)
    spec = lk.Bf16PagedBatchDecodeSpec.new(3, 40, 16, 4)
    provider = lk.DecodeProvider.load(0)
    queue = lk.CommandQueue(0x1000, 8)
    total = 6  # requests of the gathered result
    g_out, g_lse = group.buffer(total * 16 * 128, _abi.BF16), group.buffer(total * 16, _abi.F32)

    def bind(b, plan):
        reads = [b.bind_read(D(0x40000000 + i * 0x1000000, n, t)) for i, (n, t) in enumerate([
            (spec.query_numel(), _abi.BF16), (spec.kv_pages_numel(), _abi.BF16),
            (spec.kv_pages_numel(), _abi.BF16), (4, _abi.I32), (40, _abi.I32), (3, _abi.I32)])]
        ws = (b.bind_read_write(D(0x48000000, plan.workspace_required_numel(), _abi.F32))
              if plan.workspace_required_numel() else None)
        return reads, ws

    for options, commands in (({"partitions": 1}, 1), ({"partitions": 4}, 2),
                              ({"partitions": 4, "merge_in_kernel": 1}, 1), ({"balanced": 1}, 2)):
        plan = provider.plan_bf16_paged_batch(spec, **options)
        b = queue.bindings(12)
        reads, ws = bind(b, plan)
        out, lse = b.bind_read_write(g_out.span), b.bind_read_write(g_lse.span)
        rows = b.bind_read(D(0x49000000, 3, _abi.I32))
        short_rows = b.bind_read(D(0x49100000, 2, _abi.I32))
        scope = queue.begin(b)
        args = lk.Bf16PagedBatchDecodeArgs(*reads, out.write(), lse.write(), ws)
        with pytest.raises(lk.EnqueueError) as e:
            plan.enqueue_gathered_into(scope, args, short_rows, group, g_out, g_lse, total)
        assert (e.value.variant, e.value.operand) == ("LengthMismatch", "dest_rows")
        with pytest.raises(lk.EnqueueError) as e:  # the layout says 7 requests, the buffer holds 6
            plan.enqueue_gathered_into(scope, args, rows, group, g_out, g_lse, total + 1)
        assert (e.value.variant, e.value.operand) == ("LengthMismatch", "O")
        with pytest.raises(lk.ContractError) as e:  # 16 heads at offset 8 of 16 gathered heads
            plan.enqueue_gathered_into(scope, args, rows, group, g_out, g_lse, total, 16, 8)
        assert e.value.variant == "InvalidHeadMapping"
        with pytest.raises(lk.LoomError):  # the bound output is not the peer buffer's local copy
            plan.enqueue_gathered_into(scope, args, rows, group, g_lse, g_lse, total)
        assert scope.submitted_commands() == 0
        plan.enqueue_gathered_into(scope, args, rows, group, g_out, g_lse, total)
        assert scope.submitted_commands() == commands
        scope.finish().wait()

    # the all-gather as a command: rows differ per rank (2 and 4)
    gather = lk.OutputGatherPlan(group, _abi.BF16, [2, 4], 16 * 128)
    b = queue.bindings(3)
    local = b.bind_read(D(0x4a000000, 4 * 16 * 128, _abi.BF16))
    short = b.bind_read(D(0x4a800000, 2 * 16 * 128, _abi.BF16))
    gathered = b.bind_read_write(D(0x4b000000, 6 * 16 * 128, _abi.BF16))
    scope = queue.begin(b)
    with pytest.raises(lk.EnqueueError) as e:
        gather.enqueue_into(scope, lk.OutputGatherArgs(short, gathered.write()))
    assert (e.value.variant, e.value.operand) == ("LengthMismatch", "local")
    gather.enqueue_into(scope, lk.OutputGatherArgs(local, gathered.write()))
    gather.enqueue_into(scope, lk.OutputGatherArgs(local, gathered.write()))
    assert scope.submitted_commands() == 2
    lib.lb_test_fake_fail(b"external", 1, 5)  # the library call fails: ncclInvalidUsage
    with pytest.raises(lk.CommandError) as e:
        gather.enqueue_into(scope, lk.OutputGatherArgs(local, gathered.write()))
    assert (e.value.variant, e.value.operand, e.value.payload[0]) == ("External", "nccl", 5)
    assert scope.submitted_commands() == 3 and queue.is_poisoned()
    with pytest.raises(lk.CommandError) as e:
        gather.enqueue_into(scope, lk.OutputGatherArgs(local, gathered.write()))
    assert e.value.variant in ("ScopePoisoned", "QueuePoisoned")
    del scope
    group.close()


def test_queue_destroyed_before_its_scope_is_deferred(fake):
    """A queue destroyed while its scope (or completion) is alive goes only when that borrower has
    settled: the borrower keeps a pointer to it.  (Found by the AddressSanitizer build when a
    garbage collector finalised a queue before its scope.)"""
    lib = _abi.load()
    queue, bindings, scope, completion = (ctypes.c_void_p() for _ in range(4))
    assert lib.lb_queue_create(ctypes.c_void_p(0x1000), 2, ctypes.byref(queue)) == 0
    assert lib.lb_queue_bindings(queue, 1, ctypes.byref(bindings)) == 0
    assert lib.lb_queue_begin(queue, bindings, ctypes.byref(scope)) == 0
    lib.lb_queue_destroy(queue)          # deferred: the scope still points at the queue
    assert lib.lb_scope_submitted(scope) == 0
    assert lib.lb_scope_finish(scope, ctypes.byref(completion)) == 0
    lib.lb_completion_abandon(completion)  # settles, and the queue goes with it
