"""Paged causal prefill without a GPU: the contract layer against the reference's CPU-side tests
(crates/loom-infer/src/attention/paged_prefill/tests.rs), the plan's launch shape as a pure
function, and the enqueue preflight against the in-process fake driver (the cases of
crates/loom-infer-validation/src/gates/paged_prefill.rs:161-236,316-380)."""
import gc

import pytest

import loom_kernels_b200 as lk
from loom_kernels_b200 import _abi

D = lk.DeviceSpan


@pytest.fixture()
def fake():
    lib = _abi.load()
    lib.lb_test_use_fake_driver(1, 148)
    yield lib
    gc.collect()
    lib.lb_test_use_fake_driver(0, 0)


def test_metadata_maps_bottom_right_causal_pages():
    """tests.rs:3-25."""
    spec = lk.Bf16PagedPrefillSpec.new(2, 3, 6, 4, 2)
    m = spec.validate_metadata([0, 2, 3], [0, 2, 4], [4, 1, 5, 2], [3, 16])
    assert m.spec() == spec
    assert [m.request_query_range(r) for r in range(3)] == [(0, 2), (2, 3), None]
    assert [m.request_page_range(r) for r in range(2)] == [(0, 2), (2, 4)]
    assert [m.request_kv_len(r) for r in range(2)] == [19, 32]
    assert [m.causal_kv_end(0, i) for i in range(3)] == [18, 19, None]
    assert m.physical_page_for_token(0, 0) == (4, 0)
    assert m.physical_page_for_token(0, 16) == (1, 0)
    assert m.physical_page_for_token(0, 18) == (1, 2)
    assert m.physical_page_for_token(0, 19) is None
    assert (spec.query_numel(), spec.kv_pages_numel(), spec.lse_numel()) == \
        (3 * 4 * 128, 6 * 16 * 2 * 128, 12)
    assert [spec.kv_head_for_query_head(h) for h in (0, 1, 2, 3, 4)] == [0, 0, 1, 1, None]


def test_metadata_rejects_malformed_query_and_page_tables():
    """tests.rs:129-201, same order and payloads."""
    spec = lk.Bf16PagedPrefillSpec.new(2, 3, 4, 4, 2)
    cases = [
        (([0, 3], [0, 1, 2], [0, 1], [16, 16]), "LengthMismatch", "qo_indptr", (3, 2)),
        (([1, 2, 4], [0, 1, 2], [0, 1], [16, 16]), "InvalidIndptrStart", "qo_indptr", (1,)),
        (([0, 2, 1], [0, 1, 2], [0, 1], [16, 16]), "NonMonotonicIndptr", "qo_indptr", (1, 2, 1)),
        (([0, 2, 3], [1, 2, 3], [0, 1, 2], [16, 16]), "InvalidPageIndptrStart", "", (1,)),
        (([0, 2, 3], [0, 2, 1], [0], [16, 16]), "NonMonotonicPageIndptr", "", (1, 2, 1)),
        (([0, 2, 3], [0, 0, 1], [0], [16, 16]), "EmptyPagedRequest", "", (0,)),
        (([0, 2, 3], [0, 1, 2], [0, 1], [16, 0]), "InvalidLastPageLength", "", (1, 0, 16)),
        (([0, 2, 3], [0, 1, 2], [0, 4], [16, 16]), "PageIndexOutOfRange", "", (1, 4, 4)),
        (([0, 2, 3], [0, 1, 2], [0, 1], [1, 16]), "RaggedQueryLongerThanKv", "", (0, 2, 1)),
    ]
    for args, variant, operand, payload in cases:
        with pytest.raises(lk.ContractError) as e:
            spec.validate_metadata(*args)
        assert (e.value.variant, e.value.operand, e.value.payload[:len(payload)]) == \
            (variant, operand, payload)
    with pytest.raises(lk.ContractError) as e:
        spec.validate_metadata([0, 0, 3], [0, 1, 2], [0, 1], [16, 16])
    assert (e.value.variant, e.value.operand, e.value.payload[0]) == \
        ("EmptyRaggedRequest", "qo_indptr", 0)
    assert "qo_indptr request 0 has zero length" in str(e.value)
    with pytest.raises(lk.ContractError) as e:
        spec.validate_metadata([0, 2, 3], [0, 1, 2], [0, 1], [1, 16])
    assert "ragged prefill request 0 has query length 2 greater than KV length 1" in str(e.value)


def test_spec_requires_exact_contracts():
    """tests.rs:203-243."""
    for shape in [(0, 1, 1, 1, 1, 128, 16), (1, 0, 1, 1, 1, 128, 16), (1, 1, 0, 1, 1, 128, 16),
                  (1, 1, 1, 0, 1, 128, 16), (1, 1, 1, 1, 0, 128, 16), (1, 1, 1, 1, 1, 0, 16),
                  (1, 1, 1, 1, 1, 128, 0)]:
        with pytest.raises(lk.ContractError) as e:
            lk.Bf16PagedPrefillSpec.new(*shape)
        assert e.value.variant == "ZeroDimension"
    for shape, variant, payload in [((1, 1, 1, 1, 1, 64, 16), "UnsupportedHeadDimension", (128, 64)),
                                    ((1, 1, 1, 1, 1, 128, 8), "UnsupportedPageSize", (16, 8)),
                                    ((1, 1, 1, 6, 4, 128, 16), "InvalidHeadMapping", (6, 4))]:
        with pytest.raises(lk.ContractError) as e:
            lk.Bf16PagedPrefillSpec.new(*shape)
        assert (e.value.variant, e.value.payload[:2]) == (variant, payload)
    for shape in [(1, 2 ** 31, 1, 1, 1, 128, 16), (1, 1, 2 ** 64 - 1, 1, 1, 128, 16)]:
        with pytest.raises(lk.ContractError) as e:
            lk.Bf16PagedPrefillSpec.new(*shape)
        assert e.value.variant == "ElementCountOverflow"
    assert abs(lk.Bf16PagedPrefillSpec.new(1, 1, 1, 1, 1).softmax_scale() - 128 ** -0.5) < 1e-8


def test_launch_shape_is_fixed_by_spec_and_device():
    # a short call: 16-row tiles, eight pages in flight per CTA, one partly filled tile per request
    short = lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(2, 96, 96, 16, 4), 148)
    assert (short.q_tiles, short.pages_per_stage, short.rows_per_cta, short.commands) == (1, 8, 16, 1)
    assert short.tiles == 96 * 4 // 16 + 2 and short.grid == short.tiles * 4 and short.block == 288
    # a long prompt: the tensor-core kernel, 128-row tiles and 64-token blocks
    prompt = lk.Bf16PagedPrefillSpec.new(1, 8192, 600, 32, 8)
    tiled = lk.choose_paged_prefill(prompt, 148)
    assert tiled.algorithm == lk.Bf16PagedPrefillAlgorithm.Tiled
    assert (tiled.rows_per_cta, tiled.pages_per_stage, tiled.block, tiled.commands) == (128, 4, 192, 1)
    assert tiled.tiles == 8192 * 4 // 128 + 1 and tiled.grid == tiled.tiles * 8
    assert 2 * (tiled.shared_bytes + 1024) <= 233472  # two CTAs share an SM
    # the same prompt forced onto the token-parallel kernel: every loaded page used by 128 rows
    long = lk.choose_paged_prefill(prompt, 148, algorithm=1)
    assert long.algorithm == lk.Bf16PagedPrefillAlgorithm.TokenParallel
    assert (long.q_tiles, long.pages_per_stage, long.rows_per_cta) == (8, 1, 128)
    assert long.tiles == 8192 * 4 // 128 + 1 and long.grid == long.tiles * 8
    forced = lk.choose_paged_prefill(prompt, 148, q_tiles=2)
    assert (forced.algorithm, forced.q_tiles, forced.pages_per_stage) == (0, 2, 4)
    assert lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(2, 96, 96, 16, 4), 148,
                                   algorithm=2).algorithm == 1  # the caller may force it
    with pytest.raises(lk.PlanError):
        lk.choose_paged_prefill(prompt, 148, algorithm=3)
    for info in (short, long, forced):
        # the ring holds whole stages and, with several page slots, the states they merge through
        ring = info.stages * info.pages_per_stage * 8192
        assert info.shared_bytes >= ring + 1024 and info.shared_bytes <= 232448
        assert info.pages_per_stage == 1 or ring >= 8 * 68 * 32 * 4
    with pytest.raises(lk.PlanError) as e:
        lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(1, 8, 8, 4, 4), 148, q_tiles=3)
    assert e.value.variant == "Launch"
    # same inputs, same plan
    again = lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(2, 96, 96, 16, 4), 148)
    assert bytes(again) == bytes(short)


def prefill_setup(queue, spec, short=None, capacity=9):
    base = 0x20000000
    sizes = dict(query=(spec.query_numel(), _abi.BF16), key_pages=(spec.kv_pages_numel(), _abi.BF16),
                 value_pages=(spec.kv_pages_numel(), _abi.BF16),
                 qo_indptr=(spec.indptr_numel(), _abi.I32),
                 page_indptr=(spec.indptr_numel(), _abi.I32),
                 page_indices=(spec.batch_size(), _abi.I32),
                 last_page_len=(spec.last_page_len_numel(), _abi.I32))
    b = queue.bindings(capacity)
    h = {}
    for i, (name, (numel, dtype)) in enumerate(sizes.items()):
        if name == short:
            numel -= 1
        h[name] = b.bind_read(D(base + i * 0x1000000, numel, dtype))
    out = b.bind_read_write(D(base + 0x7000000, spec.output_numel() - (short == "output"),
                              _abi.BF16))
    lse = b.bind_read_write(D(base + 0x8000000, spec.lse_numel() - (short == "lse"), _abi.F32))
    return b, h, out, lse


def test_enqueue_preflight(fake):
    spec = lk.Bf16PagedPrefillSpec.new(2, 2, 2, 4, 2)
    provider = lk.PrefillProvider.load(0)
    plan = provider.plan_bf16_paged(spec)
    assert plan.spec() == spec and plan.commands() == 1
    assert plan.algorithm() == lk.Bf16PagedPrefillAlgorithm.TokenParallel
    queue = lk.CommandQueue(0x100, 1)

    def args(h, out, lse, **override):
        fields = dict(h, output=out.write(), lse=lse.write())
        fields.update(override)
        return lk.Bf16PagedPrefillArgs(**fields)

    # gates/paged_prefill.rs:161-236: a short qo_indptr fails before submission; so does every
    # other operand, by name (prefill.rs:2475-2499)
    for operand, name in [("qo_indptr", "qo_indptr"), ("query", "Q"), ("key_pages", "K_pages"),
                          ("value_pages", "V_pages"), ("page_indptr", "page_indptr"),
                          ("last_page_len", "last_page_len"), ("output", "O"), ("lse", "LSE")]:
        b, h, out, lse = prefill_setup(queue, spec, short=operand)
        scope = queue.begin(b)
        with pytest.raises(lk.EnqueueError) as e:
            plan.enqueue_into(scope, args(h, out, lse))
        assert (e.value.variant, e.value.operand) == ("LengthMismatch", name)
        if operand == "qo_indptr":
            assert e.value.payload[:2] == (spec.indptr_numel(), spec.indptr_numel() - 1)
        completion = scope.finish()
        assert completion.submitted() == 0
        completion.wait()
    b, h, out, lse = prefill_setup(queue, spec, short="page_indices")
    scope = queue.begin(b)
    with pytest.raises(lk.EnqueueError) as e:
        plan.enqueue_into(scope, args(h, out, lse))
    assert (e.value.variant, e.value.payload[:2]) == ("PageIndicesTooShort", (2, 1))
    scope.finish().wait()
    assert fake.lb_test_launch_count() == 0

    # gates/paged_prefill.rs:316-380: one binding for two operands
    b, h, out, lse = prefill_setup(queue, spec)
    scope = queue.begin(b)
    with pytest.raises(lk.CommandError) as e:
        plan.enqueue_into(scope, args(h, out, lse, key_pages=h["value_pages"]))
    assert e.value.variant == "DuplicateBindingSlot"
    with pytest.raises(lk.CommandError) as e:
        plan.enqueue_into(scope, args(h, out, lse, qo_indptr=h["query"], query=h["qo_indptr"]))
    assert e.value.variant == "BindingTypeMismatch"
    plan.enqueue_into(scope, args(h, out, lse))
    with pytest.raises(lk.CommandError) as e:
        plan.enqueue_into(scope, args(h, out, lse))
    assert (e.value.variant, e.value.payload[0]) == ("CommandCapacityExceeded", 1)
    completion = scope.finish()
    assert completion.submitted() == 1 and fake.lb_test_launch_count() == 1
    completion.wait()

    # a misaligned pool is named with the alignment this kernel needs
    b = queue.bindings(9)
    h = dict(query=b.bind_read(D(0x30000000, spec.query_numel(), _abi.BF16)),
             key_pages=b.bind_read(D(0x31000002, spec.kv_pages_numel(), _abi.BF16)),
             value_pages=b.bind_read(D(0x32000000, spec.kv_pages_numel(), _abi.BF16)),
             qo_indptr=b.bind_read(D(0x33000000, 3, _abi.I32)),
             page_indptr=b.bind_read(D(0x34000000, 3, _abi.I32)),
             page_indices=b.bind_read(D(0x35000000, 2, _abi.I32)),
             last_page_len=b.bind_read(D(0x36000000, 2, _abi.I32)))
    out = b.bind_read_write(D(0x37000000, spec.output_numel(), _abi.BF16))
    lse = b.bind_read_write(D(0x38000000, spec.lse_numel(), _abi.F32))
    scope = queue.begin(b)
    with pytest.raises(lk.EnqueueError) as e:
        plan.enqueue_into(scope, args(h, out, lse))
    assert (e.value.variant, e.value.operand, e.value.payload[:2]) == \
        ("MisalignedBuffer", "K_pages", (0x31000002, 16))
    scope.finish().wait()


def test_plan_errors(fake):
    provider = lk.PrefillProvider.load(0)
    with pytest.raises(lk.PlanError) as e:  # prefill.rs:2293-2299
        provider.plan_bf16_paged(lk.Bf16PagedPrefillSpec.new(1, 2 ** 31 - 1, 1, 4, 1))
    assert e.value.variant == "StateCountOutOfRange"
    with pytest.raises(lk.PlanError):
        provider.plan_bf16_paged(lk.Bf16PagedPrefillSpec.new(1, 8, 8, 4, 4), q_tiles=5)


def test_split_plan_shape():
    """A chunk of new tokens over a long cache has few 128-row tiles: the tiled plan shares the
    64-token KV blocks of every tile out to several CTAs and adds a merge command."""
    chunk = lk.Bf16PagedPrefillSpec.new(1, 128, 1024, 32, 8)  # 4 tiles x 8 KV heads, 16 K tokens
    auto = lk.choose_paged_prefill(chunk, 148, algorithm=2)
    assert auto.algorithm == lk.Bf16PagedPrefillAlgorithm.Tiled
    # 32 whole tiles for 296 slots: nine chunks fill them in one wave
    assert (auto.partitions, auto.commands, auto.min_chunk_blocks) == (9, 2, 16)
    assert auto.grid == auto.tiles * 8 * 9 and auto.tiles == 128 * 4 // 128 + 1
    assert auto.workspace_numel == 128 * 32 * 9 * 130
    assert (auto.merge_grid, auto.merge_block) == (128 * 32 // 4, 128)
    assert bytes(lk.choose_paged_prefill(chunk, 148)) == bytes(auto)  # also the plan-time choice
    # eight whole tiles: at most sixteen chunks
    assert lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(1, 32, 1024, 32, 8),
                                   148).partitions == 16
    # little KV room in the pool: never fewer than 1024 tokens per chunk
    small = lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(1, 128, 200, 32, 8), 148)
    assert (small.algorithm, small.partitions, small.commands) == (1, 3, 2)
    assert small.workspace_numel == 128 * 32 * 3 * 130
    tiny = lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(1, 128, 40, 32, 8), 148,
                                   algorithm=2)
    assert (tiny.partitions, tiny.commands, tiny.workspace_numel, tiny.merge_grid) == (1, 1, 0, 0)
    # many short requests: every request has a tile of its own, nothing to share out
    assert lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(32, 512, 32 * 128, 32, 8),
                                   148).partitions == 1
    # by itself: the token-parallel kernel for few rows or next to no KV
    for dims in ((1, 128, 12, 32, 8), (1, 64, 128, 32, 8), (2, 96, 130, 16, 4)):
        assert lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(*dims), 148).algorithm == 0
    assert lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(1, 128, 40, 32, 8),
                                   148).algorithm == 1
    # 128 whole tiles: two chunks each
    wide = lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(1, 512, 1024, 32, 8), 148)
    assert (wide.algorithm, wide.partitions) == (1, 2)
    # a long prompt fills the device by itself
    prompt = lk.choose_paged_prefill(lk.Bf16PagedPrefillSpec.new(1, 8192, 600, 32, 8), 148)
    assert (prompt.partitions, prompt.commands) == (1, 1)
    # the caller's count wins, and implies the tiled kernel
    forced = lk.choose_paged_prefill(chunk, 148, partitions=5)
    assert (forced.algorithm, forced.partitions, forced.grid) == (1, 5, forced.tiles * 8 * 5)
    assert forced.min_chunk_blocks == 1
    assert lk.choose_paged_prefill(chunk, 148, algorithm=2, partitions=1).commands == 1
    with pytest.raises(lk.ContractError) as e:
        lk.choose_paged_prefill(chunk, 148, partitions=65)
    assert e.value.variant == "InvalidPartitionCount"
    with pytest.raises(lk.PlanError):
        lk.choose_paged_prefill(chunk, 148, algorithm=1, partitions=2)
    with pytest.raises(lk.PlanError):  # a token-parallel tile shape and a chunk count
        lk.choose_paged_prefill(chunk, 148, q_tiles=2, partitions=2)
    assert lk.choose_paged_prefill(chunk, 148, algorithm=1).partitions == 1


def test_split_plan_reserves_both_commands_and_checks_workspace(fake):
    spec = lk.Bf16PagedPrefillSpec.new(2, 2, 2, 4, 2)
    plan = lk.PrefillProvider.load(0).plan_bf16_paged(spec, partitions=3)
    numel = 2 * 4 * 3 * 130
    assert plan.commands() == 2 and plan.partitions() == 3
    assert plan.workspace_required_numel() == numel and plan.workspace_required_bytes() == numel * 4
    for max_commands, workspace_numel, variant in [(1, numel, "CommandCapacityExceeded"),
                                                   (2, numel - 1, "LengthMismatch")]:
        queue = lk.CommandQueue(0x100, max_commands)
        b, h, out, lse = prefill_setup(queue, spec, capacity=10)
        ws = b.bind_read_write(D(0x40000000, workspace_numel, _abi.F32))
        scope = queue.begin(b)
        with pytest.raises(lk.LoomError) as e:
            plan.enqueue_into(scope, lk.Bf16PagedPrefillArgs(output=out.write(), lse=lse.write(),
                                                             workspace=ws, **h))
        assert e.value.variant == variant
        assert scope.finish().submitted() == 0
    queue = lk.CommandQueue(0x100, 2)
    b, h, out, lse = prefill_setup(queue, spec, capacity=10)
    scope = queue.begin(b)
    with pytest.raises(lk.LoomError):  # a split plan needs its workspace
        plan.enqueue_into(scope, lk.Bf16PagedPrefillArgs(output=out.write(), lse=lse.write(), **h))
    assert scope.finish().submitted() == 0
    b, h, out, lse = prefill_setup(queue, spec, capacity=10)
    ws = b.bind_read_write(D(0x40000000, numel, _abi.F32))
    scope = queue.begin(b)
    before = fake.lb_test_launch_count()
    plan.enqueue_into(scope, lk.Bf16PagedPrefillArgs(output=out.write(), lse=lse.write(),
                                                     workspace=ws, **h))
    assert fake.lb_test_launch_count() - before == 2
    assert scope.finish().submitted() == 2
