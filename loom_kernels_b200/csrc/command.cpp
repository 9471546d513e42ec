// Command runtime: typed binding arena, stream-ordered scope, one completion fence, and the
// poison rules.  State machine of crates/loom-infer-cuda/src/command/{binding,submission,
// completion,resolve}.rs of the reference, with explicit flags where Rust relies on moves and
// borrows (a queue lends itself to one live scope or completion at a time).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <vector>

#include <cuda_runtime.h>

#include "runtime.hpp"

namespace lb {

namespace {
std::atomic<uint64_t> g_next_id{1};

[[noreturn]] void abort_after_bookkeeping_invariant() {
    fprintf(stderr, "loom_b200 detected an internal command-accounting violation after GPU "
                    "submission; aborting to preserve resource safety\n");
    abort();
}
} // namespace

uint64_t fresh_id() { return g_next_id.fetch_add(1, std::memory_order_relaxed); }

lb_status require_command_capacity(const Scope &scope, size_t additional) {
    if (scope.has_error) return fail(LB_SCOPE_POISONED);
    size_t required = scope.submitted + additional;
    if (required < scope.submitted) required = SIZE_MAX;
    if (required > scope.queue->max_commands)
        return fail(LB_COMMAND_CAPACITY_EXCEEDED, nullptr, (int64_t)scope.queue->max_commands);
    return LB_OK;
}

// validate_binding_request (command/resolve.rs:856-877) followed by the per-lease checks of
// ResolveElement::{read,write} (command/binding.rs:268-287).
lb_status resolve(Scope &scope, const OperandRequest *requests, size_t count, Operand *out) {
    const Bindings &bindings = *scope.bindings;
    for (size_t i = 0; i < count; ++i)
        if (requests[i].handle.set_id != bindings.set_id) return fail(LB_BINDING_SET_MISMATCH);
    for (size_t i = 0; i < count; ++i) {
        const uint32_t slot = requests[i].handle.slot;
        for (size_t j = 0; j < i; ++j)
            if (requests[j].handle.slot == slot) return fail(LB_DUPLICATE_BINDING_SLOT);
        if (slot >= bindings.leases.size())
            return fail(LB_BINDING_SLOT_OUT_OF_RANGE, nullptr, slot,
                        (int64_t)bindings.leases.size());
    }
    for (size_t i = 0; i < count; ++i) {
        const uint32_t slot = requests[i].handle.slot;
        const Lease &lease = bindings.leases[slot];
        if (lease.kind == Lease::Vacant) return fail(LB_BINDING_SLOT_VACANT, nullptr, slot);
        if (lease.dtype != requests[i].dtype || requests[i].handle.dtype != requests[i].dtype)
            return fail(LB_BINDING_TYPE_MISMATCH, nullptr, slot);
        if (requests[i].write &&
            (lease.kind != Lease::ReadWrite || requests[i].handle.access == LB_ACCESS_READ))
            return fail(LB_BINDING_IS_READ_ONLY, nullptr, slot);
        out[i].ptr = lease.ptr;
        out[i].numel = lease.numel;
    }
    return LB_OK;
}

void record_submission(Scope &scope) {
    Queue &queue = *scope.queue;
    if (queue.retained != scope.submitted || scope.submitted >= queue.max_commands)
        abort_after_bookkeeping_invariant();
    queue.retained += 1;
    scope.submitted += 1;
}

void record_failed_submission(Scope &scope, int cuda_error) {
    record_submission(scope);
    scope.queue->poisoned = true;
    scope.has_error = true;
    scope.submission_error = cuda_error;
}

lb_status submit_launch(Scope &scope, const std::function<int()> &launch) {
    const int error = driver().launch(scope.queue->device, launch);
    if (error == 0) {
        record_submission(scope);
        return LB_OK;
    }
    record_failed_submission(scope, error);
    return fail(LB_DRIVER, "launch", error);
}

lb_status submit_external(Scope &scope, const char *provider, const std::function<int()> &call) {
    const int error = driver().external(scope.queue->device, call);
    if (error == 0) {
        record_submission(scope);
        return LB_OK;
    }
    record_failed_submission(scope, error);
    return fail(LB_EXTERNAL_COMMAND, provider, error);
}

namespace {

bool valid_dtype(int dtype) { return dtype >= LB_F32 && dtype <= LB_U8; }

lb_status bind(Bindings *bindings, int dtype, void *ptr, size_t numel, Lease::Kind kind,
               lb_handle *out) {
    if (!bindings || !out) return fail(LB_INVALID_ARGUMENT, "bindings");
    if (!valid_dtype(dtype)) return fail(LB_UNSUPPORTED_DTYPE, nullptr, dtype);
    if (!ptr && numel != 0) return fail(LB_INVALID_ARGUMENT, "device_ptr");
    // check_buffer then reserve_slot, command/binding.rs:109-133
    if (ptr) {
        int device = 0;
        bool is_device = false;
        const int rc = driver().pointer_device(ptr, &device, &is_device);
        if (rc != 0 || !is_device) return fail(LB_INVALID_ARGUMENT, "device_ptr", rc);
        if (device != bindings->device)
            return fail(LB_BUFFER_CONTEXT_MISMATCH, nullptr, device, bindings->device);
    }
    if (bindings->leases.size() == bindings->capacity)
        return fail(LB_BINDING_CAPACITY_EXCEEDED, nullptr, (int64_t)bindings->capacity);
    Lease lease;
    lease.kind = kind;
    lease.dtype = (uint8_t)dtype;
    lease.ptr = ptr;
    lease.numel = numel;
    out->set_id = bindings->set_id;
    out->slot = (uint32_t)bindings->leases.size();
    out->dtype = (uint8_t)dtype;
    out->access = kind == Lease::Read ? LB_ACCESS_READ : LB_ACCESS_READ_WRITE;
    out->reserved = 0;
    bindings->leases.push_back(lease);
    return LB_OK;
}

// settle, command/completion.rs:90-123: returns 0 when everything completed, else the CUDA
// error to report.
int settle(Completion &completion) {
    Queue &queue = *completion.queue;
    if (completion.submitted == 0)
        return completion.has_submission_error ? completion.submission_error : 0;
    int reported = 0;
    if (completion.has_submission_error) reported = completion.submission_error;
    else if (completion.record_error) reported = completion.record_error;
    else if (completion.poll_error) reported = completion.poll_error;
    if (reported) {
        synchronize_stream_or_abort(queue.stream, queue.device);
        return reported;
    }
    const int event_error = driver().event_sync(queue.completion_event);
    if (event_error == 0) return 0;
    synchronize_stream_or_abort(queue.stream, queue.device);
    return event_error;
}

} // namespace
} // namespace lb

using namespace lb;

extern "C" {

lb_handle lb_handle_read(lb_handle h) {
    h.access = LB_ACCESS_READ;
    return h;
}
lb_handle lb_handle_write(lb_handle h) {
    if (h.access == LB_ACCESS_READ_WRITE) h.access = LB_ACCESS_WRITE;
    return h;
}

// The synchronisation words of queues come from a per-device list and go back to it: a queue
// leaves its words zero, so the next queue takes them as they are, and destroying a queue calls
// nothing that a stream capture running in the same thread would forbid (a garbage collector may
// finalise an old queue at any moment, a cudaFree there invalidated the capture).  The blocks
// live as long as the process.
static std::mutex g_words_mutex;
static std::map<int, std::vector<int32_t *>> g_free_words;

static int acquire_sync_words(int device, int32_t **out) {
    {
        std::lock_guard<std::mutex> lock(g_words_mutex);
        std::vector<int32_t *> &list = g_free_words[device];
        if (!list.empty()) {
            *out = list.back();
            list.pop_back();
            return 0;
        }
    }
    int32_t *words = nullptr;
    const int rc = driver().configure(device, [&]() -> int {
        int e = cudaMalloc((void **)&words, kQueueSyncWords * sizeof(int32_t));
        if (e) return e;
        if ((e = cudaMemset(words, 0, kQueueSyncWords * sizeof(int32_t)))) return e;
        return cudaDeviceSynchronize(); // the zeros are there before any stream uses them
    });
    *out = rc ? nullptr : words; // (the fake driver runs no set-up: no words, and no kernels)
    return rc;
}

static void release_sync_words(int device, int32_t *words) {
    std::lock_guard<std::mutex> lock(g_words_mutex);
    g_free_words[device].push_back(words);
}

lb_status lb_queue_create(void *stream, size_t max_commands, lb_queue **out) {
    if (!out) return fail(LB_INVALID_ARGUMENT, "out");
    *out = nullptr;
    if (max_commands == 0) return fail(LB_ZERO_COMMAND_CAPACITY);
    int device = 0;
    int rc = driver().stream_device(stream, &device);
    if (rc) return fail(LB_DRIVER, "stream_device", rc);
    void *event = nullptr;
    if ((rc = driver().event_create(device, false, &event))) return fail(LB_DRIVER, "event", rc);
    // (under the fake driver nothing is allocated: its launches run no kernel)
    int32_t *words = nullptr;
    if ((rc = acquire_sync_words(device, &words))) {
        driver().event_destroy(device, event);
        return fail(LB_DRIVER, "queue_words", rc);
    }
    lb_queue *queue = new lb_queue();
    queue->sync_words = words;
    queue->id = fresh_id();
    queue->stream = stream;
    queue->device = device;
    queue->completion_event = event;
    queue->max_commands = max_commands;
    *out = queue;
    return LB_OK;
}

// The borrower (scope or completion) of a queue has settled: the queue is free again, or, if
// its owner destroyed it meanwhile, goes now.
static void release_queue(lb_queue *queue) {
    queue->retained = 0;
    queue->busy = false;
    if (queue->orphaned) lb_queue_destroy(queue);
}

void lb_queue_destroy(lb_queue *queue) {
    if (!queue) return;
    // Rust's borrow of the queue by its scope / completion makes this order impossible there; a
    // C caller (or a garbage collector finalising a group of objects in no particular order) can
    // get it wrong, and the borrower still holds a pointer to the queue: destruction is deferred
    // until the borrower has settled.
    if (queue->busy) {
        queue->orphaned = true;
        return;
    }
    if (queue->retained != 0) {
        const int error = synchronize_stream_or_abort(queue->stream, queue->device);
        queue->retained = 0;
        if (error)
            fprintf(stderr, "loom_b200 command queue synchronized after a stream error during "
                            "drop: CUDA error %d\n", error);
    }
    driver().event_destroy(queue->device, queue->completion_event);
    // (a queue that met an error may leave counts behind: its words are not handed on)
    if (queue->sync_words && !queue->poisoned) release_sync_words(queue->device, queue->sync_words);
    if (queue->owns_stream) driver().stream_destroy(queue->device, queue->stream);
    delete queue;
}

void *lb_queue_stream(const lb_queue *queue) { return queue ? queue->stream : nullptr; }
size_t lb_queue_max_commands(const lb_queue *queue) { return queue ? queue->max_commands : 0; }
int lb_queue_is_poisoned(const lb_queue *queue) { return queue && queue->poisoned ? 1 : 0; }

lb_status lb_queue_bindings(lb_queue *queue, size_t capacity, lb_bindings **out) {
    if (!queue || !out) return fail(LB_INVALID_ARGUMENT, "queue");
    *out = nullptr;
    if (capacity == 0) return fail(LB_ZERO_BINDING_CAPACITY);
    lb_bindings *bindings = new lb_bindings();
    bindings->queue_id = queue->id;
    bindings->set_id = fresh_id();
    bindings->stream = queue->stream;
    bindings->device = queue->device;
    bindings->capacity = capacity;
    bindings->leases.reserve(capacity);
    *out = bindings;
    return LB_OK;
}

size_t lb_bindings_len(const lb_bindings *b) { return b ? b->leases.size() : 0; }
size_t lb_bindings_capacity(const lb_bindings *b) { return b ? b->capacity : 0; }
void lb_bindings_destroy(lb_bindings *b) { delete b; }

lb_status lb_bind_read(lb_bindings *b, int dtype, const void *ptr, size_t numel, lb_handle *out) {
    return bind(b, dtype, const_cast<void *>(ptr), numel, Lease::Read, out);
}
lb_status lb_bind_read_write(lb_bindings *b, int dtype, void *ptr, size_t numel, lb_handle *out) {
    return bind(b, dtype, ptr, numel, Lease::ReadWrite, out);
}

lb_status lb_take_read_write(lb_bindings *b, lb_handle handle, void **ptr, size_t *numel) {
    if (!b) return fail(LB_INVALID_ARGUMENT, "bindings");
    if (handle.set_id != b->set_id) return fail(LB_BINDING_SET_MISMATCH);
    if (handle.slot >= b->leases.size())
        return fail(LB_BINDING_SLOT_OUT_OF_RANGE, nullptr, handle.slot, (int64_t)b->leases.size());
    Lease &lease = b->leases[handle.slot];
    if (lease.kind == Lease::Vacant) return fail(LB_BINDING_SLOT_VACANT, nullptr, handle.slot);
    if (lease.dtype != handle.dtype) return fail(LB_BINDING_TYPE_MISMATCH, nullptr, handle.slot);
    if (lease.kind == Lease::Read) return fail(LB_BINDING_IS_READ_ONLY, nullptr, handle.slot);
    if (ptr) *ptr = lease.ptr;
    if (numel) *numel = lease.numel;
    lease = Lease();
    return LB_OK;
}

lb_status lb_queue_begin(lb_queue *queue, lb_bindings *bindings, lb_scope **out) {
    std::unique_ptr<lb_bindings> owned(bindings); // moved in, released on every error path
    if (!queue || !bindings || !out) return fail(LB_INVALID_ARGUMENT, "queue");
    *out = nullptr;
    if (queue->busy) {
        owned.release(); // the caller's misuse must not free a set it may still reference
        return fail(LB_OBJECT_IN_USE);
    }
    if (queue->poisoned) return fail(LB_QUEUE_POISONED);
    if (bindings->queue_id != queue->id || bindings->stream != queue->stream ||
        bindings->device != queue->device)
        return fail(LB_BINDINGS_QUEUE_MISMATCH);
    if (queue->retained != 0) {
        queue->poisoned = true;
        return fail(LB_QUEUE_POISONED);
    }
    lb_scope *scope = new lb_scope();
    scope->queue = queue;
    scope->bindings.reset(owned.release());
    scope->scope_id = fresh_id();
    queue->busy = true;
    *out = scope;
    return LB_OK;
}

size_t lb_scope_submitted(const lb_scope *scope) { return scope ? scope->submitted : 0; }

lb_status lb_scope_finish(lb_scope *scope, lb_completion **out) {
    if (!scope || !out) return fail(LB_INVALID_ARGUMENT, "scope");
    std::unique_ptr<lb_scope> owned(scope);
    Queue *queue = scope->queue;
    lb_completion *completion = new lb_completion();
    completion->queue = queue;
    completion->bindings = std::move(scope->bindings);
    completion->submitted = scope->submitted;
    completion->has_submission_error = scope->has_error;
    completion->submission_error = scope->submission_error;
    if (scope->submitted != 0 && !scope->has_error)
        completion->record_error = driver().event_record(queue->completion_event, queue->stream);
    *out = completion; // the queue stays borrowed by the completion
    return LB_OK;
}

void lb_scope_abandon(lb_scope *scope) {
    if (!scope) return;
    std::unique_ptr<lb_scope> owned(scope);
    Queue *queue = scope->queue;
    if (scope->submitted > 0) {
        const int sync_error = synchronize_stream_or_abort(queue->stream, queue->device);
        if (scope->has_error || sync_error) queue->poisoned = true;
    } else if (scope->has_error) {
        queue->poisoned = true;
    }
    release_queue(queue);
}

lb_status lb_completion_is_complete(lb_completion *completion, int *complete) {
    if (!completion || !complete) return fail(LB_INVALID_ARGUMENT, "completion");
    if (completion->has_submission_error) return fail(LB_DRIVER, "submission", completion->submission_error);
    if (completion->record_error) return fail(LB_DRIVER, "event_record", completion->record_error);
    if (completion->poll_error) return fail(LB_DRIVER, "event_query", completion->poll_error);
    if (completion->submitted == 0) {
        *complete = 1;
        return LB_OK;
    }
    bool done = false;
    const int error = driver().event_query(completion->queue->completion_event, &done);
    if (error) {
        completion->poll_error = error;
        return fail(LB_DRIVER, "event_query", error);
    }
    *complete = done ? 1 : 0;
    return LB_OK;
}

size_t lb_completion_submitted(const lb_completion *completion) {
    return completion ? completion->submitted : 0;
}

lb_status lb_completion_wait(lb_completion *completion, lb_bindings **out) {
    if (!completion) return fail(LB_INVALID_ARGUMENT, "completion");
    std::unique_ptr<lb_completion> owned(completion);
    if (out) *out = nullptr;
    Queue *queue = completion->queue;
    const int failure = settle(*completion);
    if (failure == 0) {
        lb_bindings *bindings = completion->bindings.release();
        if (out) *out = bindings;
        else delete bindings;
        release_queue(queue);
        return LB_OK;
    }
    queue->poisoned = true; // bindings are dropped with the completion
    release_queue(queue);
    return fail(LB_DRIVER, "completion", failure);
}

void lb_completion_abandon(lb_completion *completion) {
    if (!completion) return;
    std::unique_ptr<lb_completion> owned(completion);
    Queue *queue = completion->queue;
    if (settle(*completion) != 0) queue->poisoned = true;
    release_queue(queue);
}

}
