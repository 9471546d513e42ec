// Status names, thread-local error detail, and the reference's Display text per variant.
// Variant names and wording follow crates/loom-infer/src/error.rs:111-272,
// crates/loom-infer-cuda/src/command/mod.rs:66-107, attention/decode.rs:1499-1551 and
// graph/mod.rs:687-721.
#include <cstdio>
#include <cstring>

#include "runtime.hpp"

namespace lb {
namespace {

thread_local lb_error_info g_last_error;

struct Entry {
    lb_status status;
    const char *name;
};

const Entry kNames[] = {
    {LB_OK, "Ok"},
    {LB_ZERO_DIMENSION, "ZeroDimension"},
    {LB_ELEMENT_COUNT_OVERFLOW, "ElementCountOverflow"},
    {LB_INVALID_EPSILON, "InvalidEpsilon"},
    {LB_UNSUPPORTED_HEAD_DIMENSION, "UnsupportedHeadDimension"},
    {LB_UNSUPPORTED_PAGE_SIZE, "UnsupportedPageSize"},
    {LB_INVALID_HEAD_MAPPING, "InvalidHeadMapping"},
    {LB_INVALID_PARTITION_COUNT, "InvalidPartitionCount"},
    {LB_INVALID_INDPTR_START, "InvalidIndptrStart"},
    {LB_NON_MONOTONIC_INDPTR, "NonMonotonicIndptr"},
    {LB_EMPTY_RAGGED_REQUEST, "EmptyRaggedRequest"},
    {LB_RAGGED_QUERY_LONGER_THAN_KV, "RaggedQueryLongerThanKv"},
    {LB_INVALID_PAGE_INDPTR_START, "InvalidPageIndptrStart"},
    {LB_NON_MONOTONIC_PAGE_INDPTR, "NonMonotonicPageIndptr"},
    {LB_EMPTY_PAGED_REQUEST, "EmptyPagedRequest"},
    {LB_PAGE_INDEX_OUT_OF_RANGE, "PageIndexOutOfRange"},
    {LB_INVALID_LAST_PAGE_LENGTH, "InvalidLastPageLength"},
    {LB_INVALID_ROTARY_DIMENSION, "InvalidRotaryDimension"},
    {LB_INVALID_ROPE_SCALE, "InvalidRopeScale"},
    {LB_INVALID_ROPE_THETA, "InvalidRopeTheta"},
    {LB_NEGATIVE_POSITION_ID, "NegativePositionId"},
    {LB_UNSUPPORTED_APPEND_TOKEN_COUNT, "UnsupportedAppendTokenCount"},
    {LB_APPEND_BATCH_INDEX_OUT_OF_RANGE, "AppendBatchIndexOutOfRange"},
    {LB_APPEND_POSITION_OUT_OF_RANGE, "AppendPositionOutOfRange"},
    {LB_DUPLICATE_PAGE_APPEND_SLOT, "DuplicatePageAppendSlot"},
    {LB_DUPLICATE_PAGE_APPEND_TOKEN_SLOT, "DuplicatePageAppendTokenSlot"},
    {LB_UNSUPPORTED_DTYPE, "UnsupportedDType"},
    {LB_LENGTH_MISMATCH, "LengthMismatch"},
    {LB_ZERO_COMMAND_CAPACITY, "ZeroCommandCapacity"},
    {LB_ZERO_BINDING_CAPACITY, "ZeroBindingCapacity"},
    {LB_IDENTIFIER_SPACE_EXHAUSTED, "IdentifierSpaceExhausted"},
    {LB_BINDINGS_QUEUE_MISMATCH, "BindingsQueueMismatch"},
    {LB_QUEUE_POISONED, "QueuePoisoned"},
    {LB_SCOPE_POISONED, "ScopePoisoned"},
    {LB_BINDING_CAPACITY_EXCEEDED, "BindingCapacityExceeded"},
    {LB_BUFFER_CONTEXT_MISMATCH, "BufferContextMismatch"},
    {LB_BINDING_SET_MISMATCH, "BindingSetMismatch"},
    {LB_BINDING_SLOT_OUT_OF_RANGE, "BindingSlotOutOfRange"},
    {LB_BINDING_IS_READ_ONLY, "BindingIsReadOnly"},
    {LB_BINDING_SLOT_VACANT, "BindingSlotVacant"},
    {LB_BINDING_TYPE_MISMATCH, "BindingTypeMismatch"},
    {LB_DUPLICATE_BINDING_SLOT, "DuplicateBindingSlot"},
    {LB_COMMAND_CAPACITY_EXCEEDED, "CommandCapacityExceeded"},
    {LB_EXTERNAL_COMMAND, "External"},
    {LB_DRIVER, "Driver"},
    {LB_ENQUEUE_LENGTH_MISMATCH, "LengthMismatch"},
    {LB_PAGE_INDICES_TOO_SHORT, "PageIndicesTooShort"},
    {LB_MISALIGNED_BUFFER, "MisalignedBuffer"},
    {LB_STATE_COUNT_OUT_OF_RANGE, "StateCountOutOfRange"},
    {LB_STATE_COUNT_OVERFLOW, "StateCountOverflow"},
    {LB_LAUNCH_CONTRACT, "Launch"},
    {LB_UNSUPPORTED_DEVICE, "UnsupportedDevice"},
    {LB_UNSUPPORTED_ROTARY_DIMENSION, "UnsupportedRotaryDimension"},
    {LB_GRAPH_DEFAULT_STREAM_UNSUPPORTED, "DefaultStreamUnsupported"},
    {LB_GRAPH_EMPTY_CAPTURE, "EmptyCapture"},
    {LB_GRAPH_CAPTURE_INVALIDATED, "CaptureInvalidated"},
    {LB_GRAPH_NULL_EXECUTABLE_HANDLE, "NullExecutableHandle"},
    {LB_GRAPH_EXECUTION_POISONED, "ExecutionPoisoned"},
    {LB_GRAPH_REPLAY_IN_FLIGHT, "ReplayInFlight"},
    {LB_GRAPH_LAUNCH_COUNT_EXHAUSTED, "LaunchCountExhausted"},
    {LB_GRAPH_TIMING_EVENT_CONTEXT_MISMATCH, "TimingEventContextMismatch"},
    {LB_GRAPH_DRIVER, "GraphDriver"},
    {LB_GRAPH_SETTLEMENT, "GraphSettlement"},
    {LB_GRAPH_CAPTURE_RECORD, "CaptureRecord"},
    {LB_INVALID_ARGUMENT, "InvalidArgument"},
    {LB_OBJECT_IN_USE, "ObjectInUse"},
    {LB_STATIC_SCRATCH_EXCEEDED, "StaticScratchExceeded"},
};

void format_message(lb_error_info &e) {
    const long long a = e.a, b = e.b, c = e.c, d = e.d;
    char *m = e.message;
    const size_t n = sizeof(e.message);
    switch (e.status) {
    case LB_ZERO_DIMENSION: snprintf(m, n, "tensor dimensions must be nonzero"); break;
    case LB_ELEMENT_COUNT_OVERFLOW: snprintf(m, n, "tensor element count overflowed"); break;
    case LB_UNSUPPORTED_HEAD_DIMENSION:
        snprintf(m, n, "unsupported attention head dimension: expected %lld, got %lld", a, b);
        break;
    case LB_UNSUPPORTED_PAGE_SIZE:
        snprintf(m, n, "unsupported KV page size: expected %lld, got %lld", a, b);
        break;
    case LB_INVALID_HEAD_MAPPING:
        snprintf(m, n, "query heads must be divisible by KV heads: query=%lld, KV=%lld", a, b);
        break;
    case LB_INVALID_PARTITION_COUNT:
        snprintf(m, n, "attention partition count must be in 1..=%lld, got %lld", b, a);
        break;
    case LB_INVALID_INDPTR_START:
        snprintf(m, n, "%s must start at zero, got %lld", e.operand, a);
        break;
    case LB_NON_MONOTONIC_INDPTR:
        snprintf(m, n, "%s must be nondecreasing at request %lld, got %lld then %lld", e.operand,
                 a, b, c);
        break;
    case LB_EMPTY_RAGGED_REQUEST:
        snprintf(m, n, "%s request %lld has zero length", e.operand, a);
        break;
    case LB_RAGGED_QUERY_LONGER_THAN_KV:
        snprintf(m, n,
                 "ragged prefill request %lld has query length %lld greater than KV length %lld",
                 a, b, c);
        break;
    case LB_INVALID_PAGE_INDPTR_START:
        snprintf(m, n, "page indptr must start at zero, got %lld", a);
        break;
    case LB_NON_MONOTONIC_PAGE_INDPTR:
        snprintf(m, n, "page indptr must be nondecreasing at request %lld, got %lld then %lld", a,
                 b, c);
        break;
    case LB_EMPTY_PAGED_REQUEST:
        snprintf(m, n, "paged decode request %lld has no KV pages", a);
        break;
    case LB_PAGE_INDEX_OUT_OF_RANGE:
        snprintf(m, n, "page index at position %lld must be in 0..%lld, got %lld", a, c, b);
        break;
    case LB_INVALID_LAST_PAGE_LENGTH:
        snprintf(m, n, "last page length for request %lld must be in 1..=%lld, got %lld", a, c, b);
        break;
    case LB_UNSUPPORTED_APPEND_TOKEN_COUNT:
        snprintf(m, n, "explicit paged KV append supports at most %lld tokens, got %lld", a, b);
        break;
    case LB_APPEND_BATCH_INDEX_OUT_OF_RANGE:
        snprintf(m, n, "paged KV append batch index at token %lld must be in 0..%lld, got %lld", a,
                 c, b);
        break;
    case LB_APPEND_POSITION_OUT_OF_RANGE:
        snprintf(m, n,
                 "paged KV append position at token %lld for request %lld must be in 0..%lld, got "
                 "%lld",
                 a, b, d, c);
        break;
    case LB_DUPLICATE_PAGE_APPEND_SLOT:
        snprintf(m, n,
                 "paged KV append requests %lld and %lld target the same physical slot (%lld, "
                 "%lld)",
                 a, b, c, d);
        break;
    case LB_DUPLICATE_PAGE_APPEND_TOKEN_SLOT:
        snprintf(m, n,
                 "paged KV append tokens %lld and %lld target the same physical slot (%lld, %lld)",
                 a, b, c, d);
        break;
    case LB_LENGTH_MISMATCH:
    case LB_ENQUEUE_LENGTH_MISMATCH:
        snprintf(m, n, "%s length mismatch: expected %lld, got %lld", e.operand, a, b);
        break;
    case LB_ZERO_COMMAND_CAPACITY:
        snprintf(m, n, "command queues require capacity for at least one command");
        break;
    case LB_ZERO_BINDING_CAPACITY:
        snprintf(m, n, "checked bindings require capacity for at least one resource");
        break;
    case LB_IDENTIFIER_SPACE_EXHAUSTED:
        snprintf(m, n, "command queue identifier space is exhausted");
        break;
    case LB_BINDINGS_QUEUE_MISMATCH:
        snprintf(m, n, "the checked bindings were created by a different command queue");
        break;
    case LB_QUEUE_POISONED:
        snprintf(m, n, "the command queue is poisoned by an earlier completion failure");
        break;
    case LB_SCOPE_POISONED:
        snprintf(m, n, "the command scope is poisoned by an earlier submission failure");
        break;
    case LB_BINDING_CAPACITY_EXCEEDED:
        snprintf(m, n, "checked binding capacity %lld is exhausted", a);
        break;
    case LB_BUFFER_CONTEXT_MISMATCH:
        snprintf(m, n,
                 "buffer belongs to CUDA device %lld, but the queue stream belongs to device %lld",
                 a, b);
        break;
    case LB_BINDING_SET_MISMATCH:
        snprintf(m, n, "the resource handle belongs to a different checked binding set");
        break;
    case LB_BINDING_SLOT_OUT_OF_RANGE:
        snprintf(m, n, "binding slot %lld is out of range for %lld bindings", a, b);
        break;
    case LB_BINDING_IS_READ_ONLY: snprintf(m, n, "binding slot %lld is read-only", a); break;
    case LB_BINDING_SLOT_VACANT:
        snprintf(m, n, "binding slot %lld has already been removed", a);
        break;
    case LB_BINDING_TYPE_MISMATCH:
        snprintf(m, n, "binding slot %lld has a different element type than its resource handle",
                 a);
        break;
    case LB_DUPLICATE_BINDING_SLOT:
        snprintf(m, n, "one command cannot use the same binding slot for multiple operands");
        break;
    case LB_COMMAND_CAPACITY_EXCEEDED:
        snprintf(m, n, "command scope capacity %lld is exhausted", a);
        break;
    case LB_DRIVER: snprintf(m, n, "CUDA driver error %lld", a); break;
    case LB_PAGE_INDICES_TOO_SHORT:
        snprintf(m, n, "page_indices requires at least %lld entries, got %lld", a, b);
        break;
    case LB_MISALIGNED_BUFFER:
        snprintf(m, n, "packed paged batch decode requires %s to be %lld-byte aligned, got %#llx",
                 e.operand, b, (unsigned long long)a);
        break;
    case LB_STATE_COUNT_OUT_OF_RANGE:
        snprintf(m, n, "state count %lld exceeds the CUDA grid range", a);
        break;
    case LB_STATE_COUNT_OVERFLOW: snprintf(m, n, "state count overflowed"); break;
    case LB_LAUNCH_CONTRACT: snprintf(m, n, "launch contract violated (detail %lld)", a); break;
    case LB_UNSUPPORTED_DEVICE:
        snprintf(m, n, "kernels are built for sm_100a; device reports compute capability %lld.%lld",
                 a / 10, a % 10);
        break;
    case LB_UNSUPPORTED_ROTARY_DIMENSION:
        snprintf(m, n, "RoPE provider supports rotary dimension %lld, got %lld", a, b);
        break;
    case LB_GRAPH_DEFAULT_STREAM_UNSUPPORTED:
        snprintf(m, n, "CUDA Graph capture requires a non-default stream");
        break;
    case LB_GRAPH_EMPTY_CAPTURE: snprintf(m, n, "CUDA Graph capture recorded no commands"); break;
    case LB_GRAPH_CAPTURE_INVALIDATED:
        snprintf(m, n, "CUDA Graph capture was invalidated and returned no graph");
        break;
    case LB_GRAPH_NULL_EXECUTABLE_HANDLE:
        snprintf(m, n, "CUDA Graph instantiation returned a null executable handle");
        break;
    case LB_GRAPH_EXECUTION_POISONED:
        snprintf(m, n, "CUDA Graph execution is poisoned by an earlier replay failure");
        break;
    case LB_GRAPH_REPLAY_IN_FLIGHT:
        snprintf(m, n, "a CUDA Graph replay is already in flight");
        break;
    case LB_GRAPH_LAUNCH_COUNT_EXHAUSTED:
        snprintf(m, n, "CUDA Graph launch count is exhausted");
        break;
    case LB_GRAPH_TIMING_EVENT_CONTEXT_MISMATCH:
        snprintf(m, n, "CUDA Graph timing events belong to a different CUDA context");
        break;
    case LB_GRAPH_DRIVER:
        snprintf(m, n, "CUDA Graph %s failed: CUDA error %lld", e.operand, a);
        break;
    case LB_GRAPH_SETTLEMENT:
        snprintf(m, n,
                 "CUDA Graph %s failed: CUDA error %lld; fallback stream synchronization also "
                 "reported: CUDA error %lld",
                 e.operand, a, b);
        break;
    case LB_GRAPH_CAPTURE_RECORD:
        snprintf(m, n, "graph recording failed: status %lld", a);
        break;
    case LB_INVALID_ARGUMENT: snprintf(m, n, "invalid argument: %s", e.operand); break;
    case LB_OBJECT_IN_USE:
        snprintf(m, n, "the command queue already has a live scope or completion");
        break;
    case LB_STATIC_SCRATCH_EXCEEDED:
        snprintf(m, n,
                 "split-K states need %lld floats but the library's static device scratch holds "
                 "%lld; use a split plan with a caller-owned workspace",
                 a, b);
        break;
    default: snprintf(m, n, "%s", e.name); break;
    }
}

} // namespace

const char *status_name(lb_status status) {
    for (const Entry &entry : kNames)
        if (entry.status == status) return entry.name;
    return "Unknown";
}

lb_status fail(lb_status status, const char *operand, int64_t a, int64_t b, int64_t c, int64_t d) {
    lb_error_info &e = g_last_error;
    memset(&e, 0, sizeof(e));
    e.status = status;
    snprintf(e.name, sizeof(e.name), "%s", status_name(status));
    if (operand) snprintf(e.operand, sizeof(e.operand), "%s", operand);
    e.a = a; e.b = b; e.c = c; e.d = d;
    format_message(e);
    return status;
}

} // namespace lb

extern "C" {

const char *lb_status_name(lb_status status) { return lb::status_name(status); }

void lb_last_error(lb_error_info *out) {
    if (out) *out = lb::g_last_error;
}

const char *lb_build_info(void) { return "loom_b200 0.1 (CUDA C++, sm_100a)"; }

}
