// Fixed-address CUDA Graph capture and replay.
//
// State machine of crates/loom-infer-cuda/src/graph/mod.rs of the reference: a capture-only
// queue with a private non-default stream, one non-empty checked command sequence per graph,
// an executable that owns the bindings until it is torn down, one replay in flight at a time,
// and poisoning after any driver failure.  No rebinding, node update or cross-stream launch.
#include <cstdio>
#include <cstdlib>

#include "runtime.hpp"

using namespace lb;

struct lb_graph_queue {
    lb_queue *queue = nullptr; // owns its private stream
};

struct lb_captured_graph {
    void *graph = nullptr;
    void *stream = nullptr;
    int device = 0;
    std::unique_ptr<lb_bindings> bindings;
    size_t commands = 0;
};

struct lb_graph_exec {
    void *exec = nullptr, *graph = nullptr, *stream = nullptr, *completion_event = nullptr;
    int device = 0;
    std::unique_ptr<lb_bindings> bindings;
    size_t commands = 0;
    uint64_t launches = 0;
    bool in_flight = false, poisoned = false, has_completion = false;
    int record_error = 0, poll_error = 0;
};

struct lb_graph_completion {
    lb_graph_exec *exec = nullptr;
    uint64_t launch_index = 0;
};

namespace {

[[noreturn]] void abort_cleanup(const char *resource, int error) {
    fprintf(stderr, "loom_b200 failed to destroy a CUDA %s: CUDA error %d; aborting before "
                    "releasing fixed bindings or retained resources\n", resource, error);
    abort();
}

void destroy_graph(int device, void *graph) {
    if (!graph) return;
    const int error = driver().graph_destroy(device, graph);
    if (error) abort_cleanup("graph", error);
}

void destroy_exec(int device, void *exec) {
    if (!exec) return;
    const int error = driver().graph_exec_destroy(device, exec);
    if (error) abort_cleanup("executable graph", error);
}

void release_private_stream(void *stream, int device) {
    if (stream) driver().stream_destroy(device, stream);
}

struct Settlement {
    int reported = 0, synchronization = 0;
};

// settle_in_flight, graph/mod.rs:341-368
Settlement settle_in_flight(lb_graph_exec &exec) {
    Settlement result;
    if (!exec.in_flight) return result;
    int reported = exec.record_error ? exec.record_error : exec.poll_error;
    if (!reported) reported = driver().event_sync(exec.completion_event);
    if (reported) {
        result.reported = reported;
        result.synchronization = synchronize_stream_or_abort(exec.stream, exec.device);
    }
    exec.in_flight = false;
    exec.record_error = 0;
    exec.poll_error = 0;
    return result;
}

lb_status settlement_error(const Settlement &s, const char *operation) {
    if (s.synchronization)
        return fail(LB_GRAPH_SETTLEMENT, operation, s.reported, s.synchronization);
    return fail(LB_GRAPH_DRIVER, operation, s.reported);
}

void teardown_exec(lb_graph_exec *exec) {
    Settlement s = settle_in_flight(*exec);
    if (s.reported) exec->poisoned = true;
    destroy_exec(exec->device, exec->exec);
    destroy_graph(exec->device, exec->graph);
    exec->exec = exec->graph = nullptr;
    if (exec->completion_event) driver().event_destroy(exec->device, exec->completion_event);
    exec->completion_event = nullptr;
}

} // namespace

extern "C" {

lb_status lb_graph_queue_create(int device, size_t max_commands, lb_graph_queue **out) {
    if (!out) return fail(LB_INVALID_ARGUMENT, "out");
    *out = nullptr;
    if (max_commands == 0) return fail(LB_ZERO_COMMAND_CAPACITY);
    void *stream = nullptr;
    const int error = driver().stream_create(device, &stream);
    if (error) return fail(LB_DRIVER, "stream_create", error);
    lb_queue *queue = nullptr;
    const lb_status rc = lb_queue_create(stream, max_commands, &queue);
    if (rc) {
        driver().stream_destroy(device, stream);
        return rc;
    }
    queue->owns_stream = true;
    lb_graph_queue *graph_queue = new lb_graph_queue();
    graph_queue->queue = queue;
    *out = graph_queue;
    return LB_OK;
}

void lb_graph_queue_destroy(lb_graph_queue *queue) {
    if (!queue) return;
    lb_queue_destroy(queue->queue);
    delete queue;
}

lb_status lb_graph_queue_bindings(lb_graph_queue *queue, size_t capacity, lb_bindings **out) {
    if (!queue) return fail(LB_INVALID_ARGUMENT, "queue");
    return lb_queue_bindings(queue->queue, capacity, out);
}

lb_status lb_graph_capture(lb_graph_queue *graph_queue, lb_bindings *bindings, lb_record_fn record,
                           void *user, lb_captured_graph **out) {
    std::unique_ptr<lb_bindings> owned_bindings(bindings);
    if (!graph_queue || !bindings || !record || !out) {
        if (graph_queue) lb_graph_queue_destroy(graph_queue);
        return fail(LB_INVALID_ARGUMENT, "capture");
    }
    *out = nullptr;
    // the queue is consumed: its private stream lives on in the captured graph, or dies here
    lb_queue *queue = graph_queue->queue;
    delete graph_queue;
    struct QueueGuard {
        lb_queue *queue;
        bool keep_stream = false;
        ~QueueGuard() {
            if (keep_stream) queue->owns_stream = false;
            lb_queue_destroy(queue);
        }
    } guard{queue};

    // input readiness: one context synchronisation before capture (graph/mod.rs:62-68)
    if (int error = driver().device_sync(queue->device)) {
        fprintf(stderr, "loom_b200 cannot establish CUDA Graph input readiness: CUDA error %d; "
                        "aborting before releasing caller-supplied allocations\n", error);
        abort();
    }
    if (queue->stream == nullptr) return fail(LB_GRAPH_DEFAULT_STREAM_UNSUPPORTED);

    lb_scope *scope = nullptr;
    lb_status rc = lb_queue_begin(queue, owned_bindings.release(), &scope);
    if (rc) return rc;
    if (int error = driver().capture_begin(queue->device, queue->stream)) {
        lb_scope_abandon(scope);
        return fail(LB_GRAPH_DRIVER, "capture begin", error);
    }
    scope->capturing = true;
    const lb_status record_status = record(scope, user);
    lb_error_info record_error;
    if (record_status) lb_last_error(&record_error);

    void *graph = nullptr;
    const int end_error = driver().capture_end(queue->device, queue->stream, &graph);
    if (end_error) {
        bool still_capturing = true;
        if (driver().capture_status(queue->stream, &still_capturing) != 0 || still_capturing) {
            fprintf(stderr, "loom_b200 cannot prove CUDA Graph capture ended after CUDA error %d; "
                            "aborting to preserve buffer and stream safety\n", end_error);
            abort();
        }
    }
    // captured launches never ran: nothing is retained on the stream
    const size_t submitted = scope->submitted;
    const bool scope_error = scope->has_error;
    const int scope_cuda_error = scope->submission_error;
    std::unique_ptr<lb_bindings> captured_bindings = std::move(scope->bindings);
    queue->retained = 0;
    queue->busy = false;
    delete scope;

    if (record_status) {
        destroy_graph(queue->device, graph);
        if (end_error) return fail(LB_GRAPH_DRIVER, "capture end", end_error);
        return fail(LB_GRAPH_CAPTURE_RECORD, record_error.name, record_status);
    }
    if (end_error) return fail(LB_GRAPH_DRIVER, "capture end", end_error);
    if (!graph) return fail(LB_GRAPH_CAPTURE_INVALIDATED);
    if (scope_error) {
        destroy_graph(queue->device, graph);
        return fail(LB_DRIVER, "capture", scope_cuda_error);
    }
    if (submitted == 0) {
        destroy_graph(queue->device, graph);
        return fail(LB_GRAPH_EMPTY_CAPTURE);
    }
    lb_captured_graph *captured = new lb_captured_graph();
    captured->graph = graph;
    captured->stream = queue->stream;
    captured->device = queue->device;
    captured->bindings = std::move(captured_bindings);
    captured->commands = submitted;
    guard.keep_stream = true;
    *out = captured;
    return LB_OK;
}

size_t lb_captured_graph_commands(const lb_captured_graph *graph) {
    return graph ? graph->commands : 0;
}

void lb_captured_graph_destroy(lb_captured_graph *graph) {
    if (!graph) return;
    destroy_graph(graph->device, graph->graph);
    release_private_stream(graph->stream, graph->device);
    delete graph;
}

lb_status lb_captured_graph_instantiate(lb_captured_graph *graph, lb_graph_exec **out) {
    if (!graph || !out) return fail(LB_INVALID_ARGUMENT, "graph");
    std::unique_ptr<lb_captured_graph> owned(graph);
    *out = nullptr;
    void *event = nullptr;
    int error = driver().event_create(graph->device, false, &event);
    if (error) {
        destroy_graph(graph->device, graph->graph);
        release_private_stream(graph->stream, graph->device);
        return fail(LB_GRAPH_DRIVER, "completion event creation", error);
    }
    void *exec_handle = nullptr;
    error = driver().graph_instantiate(graph->device, graph->graph, &exec_handle);
    if (error || !exec_handle) {
        driver().event_destroy(graph->device, event);
        destroy_graph(graph->device, graph->graph);
        release_private_stream(graph->stream, graph->device);
        if (error) return fail(LB_GRAPH_DRIVER, "instantiate", error);
        return fail(LB_GRAPH_NULL_EXECUTABLE_HANDLE);
    }
    lb_graph_exec *exec = new lb_graph_exec();
    exec->exec = exec_handle;
    exec->graph = graph->graph;
    exec->stream = graph->stream;
    exec->device = graph->device;
    exec->completion_event = event;
    exec->bindings = std::move(graph->bindings);
    exec->commands = graph->commands;
    *out = exec;
    return LB_OK;
}

size_t lb_graph_exec_commands(const lb_graph_exec *exec) { return exec ? exec->commands : 0; }
uint64_t lb_graph_exec_launches(const lb_graph_exec *exec) { return exec ? exec->launches : 0; }

lb_status lb_graph_exec_launch(lb_graph_exec *exec, lb_graph_completion **out) {
    if (!exec || !out) return fail(LB_INVALID_ARGUMENT, "exec");
    *out = nullptr;
    if (exec->poisoned) return fail(LB_GRAPH_EXECUTION_POISONED);
    if (exec->in_flight || exec->has_completion) return fail(LB_GRAPH_REPLAY_IN_FLIGHT);
    if (exec->launches == UINT64_MAX) return fail(LB_GRAPH_LAUNCH_COUNT_EXHAUSTED);
    // every raw launch attempt counts as possibly submitted (graph/mod.rs:265-268)
    exec->in_flight = true;
    exec->record_error = 0;
    exec->poll_error = 0;
    const int error = driver().graph_launch(exec->device, exec->exec, exec->stream);
    if (error) {
        Settlement s;
        s.reported = error;
        s.synchronization = synchronize_stream_or_abort(exec->stream, exec->device);
        exec->in_flight = false;
        exec->poisoned = true;
        return settlement_error(s, "launch");
    }
    exec->launches += 1;
    exec->record_error = driver().event_record(exec->completion_event, exec->stream);
    lb_graph_completion *completion = new lb_graph_completion();
    completion->exec = exec;
    completion->launch_index = exec->launches;
    exec->has_completion = true;
    *out = completion;
    return LB_OK;
}

uint64_t lb_graph_completion_launch_index(const lb_graph_completion *completion) {
    return completion ? completion->launch_index : 0;
}

lb_status lb_graph_completion_is_complete(lb_graph_completion *completion, int *complete) {
    if (!completion || !complete) return fail(LB_INVALID_ARGUMENT, "completion");
    lb_graph_exec *exec = completion->exec;
    if (exec->record_error)
        return fail(LB_GRAPH_DRIVER, "completion event record", exec->record_error);
    if (exec->poll_error) return fail(LB_GRAPH_DRIVER, "completion event query", exec->poll_error);
    bool done = false;
    const int error = driver().event_query(exec->completion_event, &done);
    if (error) {
        exec->poll_error = error;
        return fail(LB_GRAPH_DRIVER, "completion event query", error);
    }
    *complete = done ? 1 : 0;
    return LB_OK;
}

lb_status lb_graph_completion_wait(lb_graph_completion *completion) {
    if (!completion) return fail(LB_INVALID_ARGUMENT, "completion");
    std::unique_ptr<lb_graph_completion> owned(completion);
    lb_graph_exec *exec = completion->exec;
    exec->has_completion = false;
    const Settlement s = settle_in_flight(*exec);
    if (!s.reported) return LB_OK;
    exec->poisoned = true;
    return settlement_error(s, "completion");
}

void lb_graph_completion_abandon(lb_graph_completion *completion) {
    if (!completion) return;
    std::unique_ptr<lb_graph_completion> owned(completion);
    lb_graph_exec *exec = completion->exec;
    exec->has_completion = false;
    if (settle_in_flight(*exec).reported) exec->poisoned = true;
}

lb_status lb_graph_exec_measure_launch_ms(lb_graph_exec *exec, float *milliseconds) {
    if (!exec || !milliseconds) return fail(LB_INVALID_ARGUMENT, "exec");
    void *start = nullptr, *end = nullptr;
    int error = driver().event_create(exec->device, true, &start);
    if (!error) error = driver().event_create(exec->device, true, &end);
    if (error) {
        if (start) driver().event_destroy(exec->device, start);
        return fail(LB_GRAPH_DRIVER, "timing event creation", error);
    }
    lb_status rc = LB_OK;
    if ((error = driver().event_record(start, exec->stream))) {
        rc = fail(LB_GRAPH_DRIVER, "timing start event record", error);
    } else {
        lb_graph_completion *completion = nullptr;
        rc = lb_graph_exec_launch(exec, &completion);
        if (rc == LB_OK) {
            error = driver().event_record(end, exec->stream);
            if (error) {
                lb_graph_completion_abandon(completion);
                rc = fail(LB_GRAPH_DRIVER, "timing end event record", error);
            } else if ((rc = lb_graph_completion_wait(completion)) == LB_OK) {
                // the end event was recorded after the completion event on the same stream
                if ((error = driver().event_sync(end)) ||
                    (error = driver().event_elapsed_ms(start, end, milliseconds)))
                    rc = fail(LB_GRAPH_DRIVER, "timing event elapsed query", error);
            }
        }
    }
    driver().event_destroy(exec->device, start);
    driver().event_destroy(exec->device, end);
    return rc;
}

lb_status lb_graph_exec_into_bindings(lb_graph_exec *exec, lb_bindings **out) {
    if (!exec) return fail(LB_INVALID_ARGUMENT, "exec");
    std::unique_ptr<lb_graph_exec> owned(exec);
    if (out) *out = nullptr;
    const Settlement s = settle_in_flight(*exec);
    if (s.reported) {
        exec->poisoned = true;
        teardown_exec(exec);
        release_private_stream(exec->stream, exec->device);
        return settlement_error(s, "completion");
    }
    teardown_exec(exec);
    release_private_stream(exec->stream, exec->device);
    lb_bindings *bindings = exec->bindings.release();
    if (out) *out = bindings;
    else delete bindings;
    return LB_OK;
}

void lb_graph_exec_destroy(lb_graph_exec *exec) {
    if (!exec) return;
    teardown_exec(exec);
    release_private_stream(exec->stream, exec->device);
    delete exec;
}

}
