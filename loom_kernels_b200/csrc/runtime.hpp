// Internal C++ host layer behind the C ABI: error reporting, the CUDA driver seam, and the
// command / graph object model.  Mirrors the ownership rules of the reference's
// crates/loom-infer-cuda/src/command/* and graph/mod.rs with explicit states where Rust uses
// moves and borrows.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "loom_b200.h"

// The opaque C handle types are these structs.
struct lb_lease { // command/binding.rs:176-188 (Access + Lease)
    enum Kind : uint8_t { Vacant = 0, Read = 1, ReadWrite = 2 };
    Kind kind = Vacant;
    uint8_t dtype = 0;
    void *ptr = nullptr;
    size_t numel = 0;
};

struct lb_bindings { // CheckedBindings
    uint64_t queue_id = 0, set_id = 0;
    void *stream = nullptr;
    int device = 0;
    size_t capacity = 0;
    std::vector<lb_lease> leases;
};

struct lb_queue { // CommandQueue
    uint64_t id = 0;
    void *stream = nullptr;
    int device = 0;
    void *completion_event = nullptr;
    size_t max_commands = 0;
    size_t retained = 0; // retained_resources.len()
    bool poisoned = false;
    bool busy = false; // a scope or completion borrowed from this queue is alive
    bool orphaned = false; // lb_queue_destroy came while busy: the borrower destroys the queue
    bool owns_stream = false;
    // kQueueSyncWords device words, zero whenever no command of this queue is running: kernels
    // that count their CTAs (a split merged by its last CTA) use them and leave them zero.  The
    // queue's stream orders its commands, so no two kernels use the words at the same time.
    int32_t *sync_words = nullptr;
};
constexpr size_t kQueueSyncWords = 16384;

struct lb_scope { // CommandScope
    lb_queue *queue = nullptr;
    std::unique_ptr<lb_bindings> bindings;
    uint64_t scope_id = 0;
    size_t submitted = 0;
    bool has_error = false;
    int submission_error = 0; // CUDA error code of the failed submission
    bool capturing = false;
};

struct lb_completion { // CommandCompletion
    lb_queue *queue = nullptr;
    std::unique_ptr<lb_bindings> bindings;
    size_t submitted = 0;
    bool has_submission_error = false;
    int submission_error = 0;
    int record_error = 0, poll_error = 0;
};

namespace lb {

// ---- errors ---------------------------------------------------------------------------------

// Records the thread-local error detail and returns `status` so call sites can `return fail(...)`.
lb_status fail(lb_status status, const char *operand = nullptr, int64_t a = 0, int64_t b = 0,
               int64_t c = 0, int64_t d = 0);
const char *status_name(lb_status status);

// ---- driver seam ----------------------------------------------------------------------------

// Everything the runtime asks of CUDA goes through this table, so the host state machine can be
// driven by an in-process fake on machines without a GPU.  All calls return a CUDA error code
// (0 = success).
struct Driver {
    virtual ~Driver() = default;
    virtual int device_count(int *count) = 0;
    virtual int device_props(int device, int *sm_count, int *cc_major, int *cc_minor,
                             size_t *smem_optin, size_t *l2_bytes) = 0;
    virtual int stream_device(void *stream, int *device) = 0;
    virtual int pointer_device(const void *ptr, int *device, bool *is_device_memory) = 0;
    virtual int stream_create(int device, void **stream) = 0;
    virtual int stream_destroy(int device, void *stream) = 0;
    virtual int stream_sync(void *stream) = 0;
    virtual int device_sync(int device) = 0;
    virtual int event_create(int device, bool timing, void **event) = 0;
    virtual int event_destroy(int device, void *event) = 0;
    virtual int event_record(void *event, void *stream) = 0;
    virtual int event_query(void *event, bool *complete) = 0;
    virtual int event_sync(void *event) = 0;
    virtual int event_elapsed_ms(void *start, void *end, float *ms) = 0;
    // Runs a set-up closure (attribute / symbol / allocation calls) with `device` current.
    virtual int configure(int device, const std::function<int()> &setup) = 0;
    // Runs `launch` (a closure that calls one <<<>>> wrapper and returns its error code).
    virtual int launch(int device, const std::function<int()> &launch) = 0;
    // Runs a library call that enqueues work on the command's stream (a collective of the
    // communication library); the closure returns that library's own result code, 0 = success.
    virtual int external(int device, const std::function<int()> &call) = 0;
    // SM clock of the device in kHz (turns a wait limit in microseconds into cycles).
    virtual int device_clock_khz(int device, int *khz) = 0;
    virtual int capture_begin(int device, void *stream) = 0;
    virtual int capture_end(int device, void *stream, void **graph) = 0;
    virtual int capture_status(void *stream, bool *capturing) = 0;
    virtual int graph_instantiate(int device, void *graph, void **exec) = 0;
    virtual int graph_launch(int device, void *exec, void *stream) = 0;
    virtual int graph_destroy(int device, void *graph) = 0;
    virtual int graph_exec_destroy(int device, void *exec) = 0;
    // Encodes a rank-3 bf16 tiled tensor map with 128-byte swizzle into 128 bytes at `map`.
    // strides_bytes holds the strides of dimensions 1 and 2 (dimension 0 is contiguous).
    virtual int encode_tensor_map_3d(int device, void *map, const void *base,
                                     const uint64_t dims[3], const uint64_t strides_bytes[2],
                                     const uint32_t box[3]) = 0;
    virtual bool is_fake() const = 0;
    virtual uint64_t launch_count() const = 0;
};

Driver &driver();
void use_fake_driver(bool enable, int sm_count);
void fake_fail(const char *what, int n, int cuda_error);

// stream sync, then context sync, else abort  (command/completion.rs:165-182)
int synchronize_stream_or_abort(void *stream, int device);

// ---- command runtime ------------------------------------------------------------------------

using Lease = ::lb_lease;
using Bindings = ::lb_bindings;
using Queue = ::lb_queue;
using Scope = ::lb_scope;
using Completion = ::lb_completion;

struct Operand { // one resolved operand of a command
    void *ptr;
    size_t numel;
};

struct OperandRequest {
    lb_handle handle;
    uint8_t dtype;
    bool write;
};

// require_command_capacity, command/submission.rs:163-180
lb_status require_command_capacity(const Scope &scope, size_t additional);
// prepare_command + resolve_* , command/submission.rs:153-161 and command/resolve.rs:843-885
lb_status resolve(Scope &scope, const OperandRequest *requests, size_t count, Operand *out);
// record_cuda_submission / record_failed_cuda_submission, command/submission.rs:212-238
void record_submission(Scope &scope);
void record_failed_submission(Scope &scope, int cuda_error);
// Runs one kernel launch for a command that passed every preflight check and records it.
lb_status submit_launch(Scope &scope, const std::function<int()> &launch);
// record_external_submission / record_failed_external_submission, command/submission.rs:240-272:
// a library call that enqueued work on the queue's stream counts as one command; its failure
// poisons scope and queue (ExternalCommand, a = the library's result code).
lb_status submit_external(Scope &scope, const char *provider, const std::function<int()> &call);

uint64_t fresh_id();

// ---- contract helpers shared by the providers --------------------------------------------------

struct DecodeChoice {
    uint32_t algorithm; // LB_DECODE_DIRECT / LB_DECODE_SPLIT_K / LB_DECODE_BALANCED
    uint32_t partitions, heads_per_cta, q_tiles, q_blocks, pages_per_stage, stages, warps;
    uint32_t grid, block, shared_bytes, merge_grid, merge_block;
    size_t workspace_numel;
    uint32_t producer_warps;   // balanced plans: warps that issue the page copies
    uint32_t merge_four_warps; // balanced plans: the merge kernel's form (many states per item)
    uint32_t merged_in_kernel; // split-K as one command: the last CTA of an item merges it
};
lb_status choose_decode(const lb_paged_spec &spec, uint32_t sm_count, size_t smem_optin,
                        const lb_paged_decode_options *options, DecodeChoice *out);

} // namespace lb
