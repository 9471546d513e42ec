/*
 * loom_b200 -- C ABI of the B200 (sm_100a) provider for the Loom Infer paged-decode path.
 *
 * The ABI mirrors, one to one, the Rust surface an engine uses for this path in the reference
 * (paths below are relative to the reference project root):
 *
 *     validated spec -> immutable plan -> checked typed bindings -> one caller-owned
 *     stream -> one completion fence            (docs/design/loom-infer-architecture.md)
 *
 * Conventions
 *   - every function returns an lb_status (0 = LB_OK) and writes results through out-params;
 *     nothing throws across the boundary;
 *   - every non-zero status is a reference error variant, by name (lb_status_name);
 *     the variant's payload is read with lb_last_error (thread-local);
 *   - "moved" parameters are consumed by the call whether it succeeds or not, exactly where
 *     the Rust API takes `self` / an owned value;
 *   - no internal locking: one thread drives one queue; graph objects are thread-affine
 *     (crates/loom-infer-cuda/src/graph/mod.rs:29,173,234);
 *   - device buffers stay caller-allocated; a buffer bound read-write belongs to the binding
 *     set until lb_completion_wait / lb_graph_exec_into_bindings hands the set back.
 */
#ifndef LOOM_B200_H
#define LOOM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t lb_status;

/* ---- status codes ------------------------------------------------------------------------ */
enum {
    LB_OK = 0,
    /* ContractError, crates/loom-infer/src/error.rs:6-109 (same order) */
    LB_ZERO_DIMENSION = 1,
    LB_ELEMENT_COUNT_OVERFLOW,
    LB_INVALID_EPSILON,
    LB_UNSUPPORTED_HEAD_DIMENSION,       /* a=expected b=actual */
    LB_UNSUPPORTED_PAGE_SIZE,            /* a=expected b=actual */
    LB_INVALID_HEAD_MAPPING,             /* a=query_heads b=kv_heads */
    LB_INVALID_PARTITION_COUNT,          /* a=partitions b=kv_len (pages for the paged split) */
    LB_INVALID_INDPTR_START,             /* operand=buffer a=actual */
    LB_NON_MONOTONIC_INDPTR,             /* operand=buffer a=request b=start c=end */
    LB_EMPTY_RAGGED_REQUEST,             /* operand=buffer a=request */
    LB_RAGGED_QUERY_LONGER_THAN_KV,      /* a=request b=query_len c=kv_len */
    LB_INVALID_PAGE_INDPTR_START,        /* a=actual */
    LB_NON_MONOTONIC_PAGE_INDPTR,        /* a=request b=start c=end */
    LB_EMPTY_PAGED_REQUEST,              /* a=request */
    LB_PAGE_INDEX_OUT_OF_RANGE,          /* a=position b=index c=max_num_pages */
    LB_INVALID_LAST_PAGE_LENGTH,         /* a=request b=length c=page_size */
    LB_INVALID_ROTARY_DIMENSION,
    LB_INVALID_ROPE_SCALE,
    LB_INVALID_ROPE_THETA,
    LB_NEGATIVE_POSITION_ID,
    LB_UNSUPPORTED_APPEND_TOKEN_COUNT,   /* a=maximum b=actual */
    LB_APPEND_BATCH_INDEX_OUT_OF_RANGE,  /* a=token b=index c=batch_size */
    LB_APPEND_POSITION_OUT_OF_RANGE,     /* a=token b=request c=position d=kv_len */
    LB_DUPLICATE_PAGE_APPEND_SLOT,       /* a=first_request b=second_request c=page d=offset */
    LB_DUPLICATE_PAGE_APPEND_TOKEN_SLOT, /* a=first_token b=second_token c=page d=offset */
    LB_UNSUPPORTED_DTYPE,
    LB_LENGTH_MISMATCH,                  /* operand=buffer a=expected b=actual */

    /* CommandError, crates/loom-infer-cuda/src/command/mod.rs:66-107 */
    LB_ZERO_COMMAND_CAPACITY = 100,
    LB_ZERO_BINDING_CAPACITY,
    LB_IDENTIFIER_SPACE_EXHAUSTED,
    LB_BINDINGS_QUEUE_MISMATCH,
    LB_QUEUE_POISONED,
    LB_SCOPE_POISONED,
    LB_BINDING_CAPACITY_EXCEEDED,        /* a=capacity */
    LB_BUFFER_CONTEXT_MISMATCH,          /* a=buffer_device b=stream_device */
    LB_BINDING_SET_MISMATCH,
    LB_BINDING_SLOT_OUT_OF_RANGE,        /* a=slot b=bindings */
    LB_BINDING_IS_READ_ONLY,             /* a=slot */
    LB_BINDING_SLOT_VACANT,              /* a=slot */
    LB_BINDING_TYPE_MISMATCH,            /* a=slot */
    LB_DUPLICATE_BINDING_SLOT,
    LB_COMMAND_CAPACITY_EXCEEDED,        /* a=capacity */
    LB_EXTERNAL_COMMAND,
    LB_DRIVER,                           /* a=CUDA error code */

    /* {PagedBatchDecode,Rope}EnqueueError, crates/loom-infer-cuda/src/attention/decode.rs:1529-1551,
     * crates/loom-infer-cuda/src/rope/mod.rs (RopeEnqueueError) */
    LB_ENQUEUE_LENGTH_MISMATCH = 200,    /* operand a=expected b=actual */
    LB_PAGE_INDICES_TOO_SHORT,           /* a=minimum b=actual */
    LB_MISALIGNED_BUFFER,                /* operand a=address b=alignment */

    /* {PagedBatchDecode,Rope}PlanError, decode.rs:1499-1505, rope/mod.rs (RopePlanError) */
    LB_STATE_COUNT_OUT_OF_RANGE = 300,   /* a=states */
    LB_STATE_COUNT_OVERFLOW,
    LB_LAUNCH_CONTRACT,                  /* device or launch shape unusable; a=detail code */
    LB_UNSUPPORTED_DEVICE,               /* a=compute capability major*10+minor */
    LB_UNSUPPORTED_ROTARY_DIMENSION,     /* RopePlanError; a=expected b=actual */

    /* GraphError, crates/loom-infer-cuda/src/graph/mod.rs:687-721; CaptureError :136-143 */
    LB_GRAPH_DEFAULT_STREAM_UNSUPPORTED = 400,
    LB_GRAPH_EMPTY_CAPTURE,
    LB_GRAPH_CAPTURE_INVALIDATED,
    LB_GRAPH_NULL_EXECUTABLE_HANDLE,
    LB_GRAPH_EXECUTION_POISONED,
    LB_GRAPH_REPLAY_IN_FLIGHT,
    LB_GRAPH_LAUNCH_COUNT_EXHAUSTED,
    LB_GRAPH_TIMING_EVENT_CONTEXT_MISMATCH,
    LB_GRAPH_DRIVER,                     /* operand=operation a=CUDA error code */
    LB_GRAPH_SETTLEMENT,                 /* operand=operation a=error b=synchronization error */
    LB_GRAPH_CAPTURE_RECORD,             /* the record callback failed; a=its status */

    /* misuse the Rust borrow checker rules out at compile time */
    LB_INVALID_ARGUMENT = 500,           /* null pointer, dead object, not a device pointer */
    LB_OBJECT_IN_USE,                    /* queue already has a live scope / completion */
    LB_STATIC_SCRATCH_EXCEEDED           /* a=floats needed b=floats the static scratch holds */
};

typedef struct lb_error_info {
    lb_status status;
    char name[48];    /* variant name, e.g. "LengthMismatch" */
    char operand[32]; /* buffer / operand / operation name where the variant has one */
    int64_t a, b, c, d;
    char message[256]; /* the reference's Display text for the variant */
} lb_error_info;

const char *lb_status_name(lb_status status);
/* Details of the last non-zero status returned on this thread. */
void lb_last_error(lb_error_info *out);
/* Library version and the compute architecture the kernels were built for. */
const char *lb_build_info(void);

/* ---- contract: specs and host-side metadata validation ------------------------------------ */

/* Bf16PagedBatchDecodeSpec, crates/loom-infer/src/attention/paged_decode/mod.rs:17-149 */
typedef struct lb_paged_spec {
    size_t batch_size, max_num_pages, num_query_heads, num_kv_heads;
    float softmax_scale; /* 1/sqrt(128) */
} lb_paged_spec;

#define LB_HEAD_DIM 128u
#define LB_PAGE_SIZE 16u
#define LB_PARTIAL_STATE_WIDTH 130u      /* single_decode/mod.rs:13 */
#define LB_APPEND_MAX_TOKENS 64u         /* paged_append/mod.rs:12 */

/* Bf16PagedBatchDecodeSpec::new, paged_decode/mod.rs:28-82 */
lb_status lb_paged_spec_new(size_t batch_size, size_t max_num_pages, size_t num_query_heads,
                            size_t num_kv_heads, size_t head_dim, size_t page_size,
                            lb_paged_spec *out);
/* numel accessors, paged_decode/mod.rs:112-149 */
size_t lb_paged_spec_query_numel(const lb_paged_spec *spec);
size_t lb_paged_spec_kv_pages_numel(const lb_paged_spec *spec);
size_t lb_paged_spec_lse_numel(const lb_paged_spec *spec);
size_t lb_paged_spec_gqa_group_size(const lb_paged_spec *spec);
/* kv_head_for_query_head, :143-149; returns -1 for None */
int64_t lb_paged_spec_kv_head_for_query_head(const lb_paged_spec *spec, size_t query_head);
/* validate_page_table, :152-213 (host copies of the metadata) */
lb_status lb_paged_spec_validate_page_table(const lb_paged_spec *spec, const int32_t *page_indptr,
                                            size_t page_indptr_len, const int32_t *page_indices,
                                            size_t page_indices_len, const int32_t *last_page_len,
                                            size_t last_page_len_len);
/* Bf16PagedBatchDecodePageTable::request_kv_len / physical_page_for_token, :252-278.
 * The table must have passed validate_page_table.  Return 0 (None) or 1 (Some). */
int lb_page_table_request_kv_len(const lb_paged_spec *spec, const int32_t *page_indptr,
                                 const int32_t *last_page_len, size_t request, size_t *kv_len);
int lb_page_table_physical_page_for_token(const lb_paged_spec *spec, const int32_t *page_indptr,
                                          const int32_t *page_indices,
                                          const int32_t *last_page_len, size_t request,
                                          size_t logical_token, size_t *physical_page,
                                          size_t *page_offset);

/* Bf16RopePagedKvAppendSpec::validate_page_table (duplicate final slots),
 * crates/loom-infer/src/attention/paged_append/mod.rs:95-131 */
lb_status lb_append_spec_validate_page_table(const lb_paged_spec *spec, const int32_t *page_indptr,
                                             size_t page_indptr_len, const int32_t *page_indices,
                                             size_t page_indices_len,
                                             const int32_t *last_page_len,
                                             size_t last_page_len_len);

/* Bf16RopePagedKvAppendTokensSpec, paged_append/mod.rs:136-241 */
typedef struct lb_append_tokens_spec {
    lb_paged_spec paged;
    size_t tokens;
    size_t max_tokens; /* LB_APPEND_MAX_TOKENS for the contract; 0 = extended (no total cap) */
} lb_append_tokens_spec;

/* Bf16RopePagedKvAppendTokensSpec::new, :144-177 */
lb_status lb_append_tokens_spec_new(size_t tokens, size_t batch_size, size_t max_num_pages,
                                    size_t num_query_heads, size_t num_kv_heads, size_t head_dim,
                                    size_t page_size, lb_append_tokens_spec *out);
/* Extension (no reference counterpart): the same contract without the 64-token total cap, up
 * to lb_append_extended_max_tokens() tokens; same all-or-nothing device guard.  A plan made
 * from such a spec is two commands (validate once, then rotate and scatter) and needs an I32
 * workspace of lb_rope_append_plan_info.workspace_numel elements bound read-write. */
lb_status lb_append_tokens_spec_new_extended(size_t tokens, size_t batch_size,
                                             size_t max_num_pages, size_t num_query_heads,
                                             size_t num_kv_heads, size_t head_dim,
                                             size_t page_size, lb_append_tokens_spec *out);
size_t lb_append_extended_max_tokens(void);
/* validate_metadata, :244-317; slots_out (nullable) receives tokens x (page, offset) */
lb_status lb_append_tokens_spec_validate_metadata(
    const lb_append_tokens_spec *spec, const int32_t *batch_indices, size_t batch_indices_len,
    const int32_t *positions, size_t positions_len, const int32_t *page_indptr,
    size_t page_indptr_len, const int32_t *page_indices, size_t page_indices_len,
    const int32_t *last_page_len, size_t last_page_len_len, int64_t *slots_out);

/* Split-K contract pieces, crates/loom-infer/src/attention/single_decode/mod.rs:125-194,
 * applied per request to the PAGE count (the reference has no paged split-K, so chunks are
 * whole pages and the workspace gains a leading request dimension).
 * partition_token_range :171-185 -> page range; returns 0 (None) / 1 (Some). */
int lb_split_partition_range(size_t length, size_t partitions, size_t partition, size_t *start,
                             size_t *end);
/* workspace_numel :163-165 with a leading request dimension: batch*qh*partitions*130 */
lb_status lb_paged_split_workspace_numel(const lb_paged_spec *spec, size_t partitions,
                                         size_t *numel);
/* partial_state_offset :187-193 with the request dimension; returns -1 for None */
int64_t lb_paged_split_state_offset(const lb_paged_spec *spec, size_t partitions, size_t request,
                                    size_t query_head, size_t partition);

/* ---- command runtime ---------------------------------------------------------------------- */

typedef struct lb_queue lb_queue;           /* CommandQueue,      command/submission.rs:18-117 */
typedef struct lb_bindings lb_bindings;     /* CheckedBindings,   command/binding.rs:16-134 */
typedef struct lb_scope lb_scope;           /* CommandScope,      command/submission.rs:119-329 */
typedef struct lb_completion lb_completion; /* CommandCompletion, command/completion.rs:6-141 */

/* BindingElement types, command/binding.rs:181-187 */
enum { LB_F32 = 0, LB_F16 = 1, LB_BF16 = 2, LB_I32 = 3, LB_U8 = 4 };
enum { LB_ACCESS_READ = 0, LB_ACCESS_WRITE = 1, LB_ACCESS_READ_WRITE = 2 };

/* Read<T> / Write<T> / ReadWrite<T>, command/binding.rs:297-336.  Plain value; copyable. */
typedef struct lb_handle {
    uint64_t set_id;
    uint32_t slot;
    uint8_t dtype;
    uint8_t access;
    uint16_t reserved;
} lb_handle;

/* ReadWrite::read / ReadWrite::write, binding.rs:313-327 */
lb_handle lb_handle_read(lb_handle read_write);
lb_handle lb_handle_write(lb_handle read_write);

/* CommandQueue::new, submission.rs:31-46.  `stream` is a cudaStream_t / CUstream owned by
 * the caller; it must outlive the queue.
 * Beyond the reference: a queue also owns 64 KB of device words that are zero whenever none of
 * its commands is running.  Kernels that count their own CTAs (plans made with merge_in_kernel,
 * one_command) use them and leave them zero; the queue's stream is what keeps two such kernels
 * apart, so commands of one queue must not be made to overlap by any other means, and a Graph
 * uses the words of the queue it was captured on.  A queue that was poisoned does not hand its
 * words on. */
lb_status lb_queue_create(void *stream, size_t max_commands, lb_queue **out);
/* Drop for CommandQueue, submission.rs:102-117 (synchronises retained work first).  While a scope
 * or completion of the queue is alive the destruction is deferred until it has settled (in Rust the
 * borrow makes that order impossible). */
void lb_queue_destroy(lb_queue *queue);
void *lb_queue_stream(const lb_queue *queue);
size_t lb_queue_max_commands(const lb_queue *queue);
int lb_queue_is_poisoned(const lb_queue *queue);
/* CommandQueue::bindings, submission.rs:58-70 */
lb_status lb_queue_bindings(lb_queue *queue, size_t capacity, lb_bindings **out);
/* CommandQueue::begin, submission.rs:73-99; `bindings` is moved. */
lb_status lb_queue_begin(lb_queue *queue, lb_bindings *bindings, lb_scope **out);

size_t lb_bindings_len(const lb_bindings *bindings);
size_t lb_bindings_capacity(const lb_bindings *bindings);
void lb_bindings_destroy(lb_bindings *bindings);
/* bind_read / bind_read_write, binding.rs:38-87.  On failure the caller keeps the buffer. */
lb_status lb_bind_read(lb_bindings *bindings, int dtype, const void *device_ptr, size_t numel,
                       lb_handle *out);
lb_status lb_bind_read_write(lb_bindings *bindings, int dtype, void *device_ptr, size_t numel,
                             lb_handle *out);
/* take_read_write, binding.rs:93-107; the slot becomes vacant. */
lb_status lb_take_read_write(lb_bindings *bindings, lb_handle handle, void **device_ptr,
                             size_t *numel);

/* CommandScope::finish, submission.rs:131-151; `scope` is moved. */
lb_status lb_scope_finish(lb_scope *scope, lb_completion **out);
/* Drop of an unfinished CommandScope, submission.rs:296-329. */
void lb_scope_abandon(lb_scope *scope);
size_t lb_scope_submitted(const lb_scope *scope);

/* CommandCompletion::{is_complete, submitted, wait}, completion.rs:38-88 */
lb_status lb_completion_is_complete(lb_completion *completion, int *complete);
size_t lb_completion_submitted(const lb_completion *completion);
/* `completion` is moved; on success *out receives the reusable bindings. */
lb_status lb_completion_wait(lb_completion *completion, lb_bindings **out);
/* Drop for CommandCompletion, completion.rs:126-141 (settles, bindings are released). */
void lb_completion_abandon(lb_completion *completion);

/* ---- decode provider ----------------------------------------------------------------------- */

typedef struct lb_decode_provider lb_decode_provider; /* DecodeProvider, decode.rs:1001-1104 */
typedef struct lb_paged_decode_plan lb_paged_decode_plan; /* Bf16PagedBatchDecodePlan :1181-1297 */

/* Bf16PagedBatchDecodeAlgorithm, decode.rs:1157-1161, for this provider */
enum {
    LB_DECODE_DIRECT = 0,   /* one CTA per (request, head block); one command, no workspace */
    LB_DECODE_SPLIT_K = 1,  /* `partitions` page-balanced chunks per request + LSE merge */
    LB_DECODE_BALANCED = 2, /* the batch's pages cut evenly over the SMs + LSE merge; the choice
                               for ragged batches and for batches smaller than the device */
    LB_DECODE_CLUSTER_SPLIT = 3 /* `partitions` (2..8) chunks per request whose CTAs form one
                               thread-block cluster and merge their states through distributed
                               shared memory: split-K as ONE command, without a workspace; the
                               choice for a single short request (latency-bound) */
};

typedef struct lb_paged_decode_options {
    uint32_t partitions;    /* 0 = plan-time heuristic, 1 = direct, N>1 = split-K with N chunks */
    uint32_t heads_per_cta; /* 0 = heuristic; KV heads one CTA streams (1, 2, 4 or 8) */
    uint32_t balanced;      /* with partitions == 0: 0 = heuristic, 1 = force the balanced
                               algorithm, 2 = never use it */
    uint32_t balanced_ctas; /* CTAs of the balanced algorithm; 0 = heuristic (<= one per SM) */
    uint32_t indices_capacity; /* 0: the bound page_indices are exactly the table (the reference's
                                  rule, page_indptr[batch] == page_indices.len());
                                  1: page_indices may be bound LONGER than the table in use
                                  (page_indptr[batch] <= len, the tail is never read), so that a
                                  fixed-address Graph survives a change of the total page count.
                                  No reference counterpart (the reference lists the mutable-
                                  metadata Graph contract as open, docs/operator-catalog.md). */
    uint32_t wait_limit_us; /* limit of every bounded wait of the plan's kernels (a copy that never
                               arrives, a rank that never publishes), in microseconds; 0 = about
                               two seconds.  When it runs out the kernel writes nothing more,
                               records a status word (lb_decode_provider_device_status) and returns */
    uint32_t test_skip_page; /* tests of that give-up path only: 1 + the index, within every CTA's
                                page chunk, of a page whose barrier expects 16 bytes more than its
                                copies deliver (the page never becomes ready); 0 = none.  Direct
                                and split-K plans, a page of the ring's first round */
    uint32_t cluster;        /* with partitions 2..8: 1 = LB_DECODE_CLUSTER_SPLIT instead of the
                                two-command split-K */
    uint32_t merge_in_kernel; /* 1 = the kernel that computes the partial states also merges them
                                 (whoever counts the last state of an item; one command; needs a
                                 counting word of the queue per item), 2 = a second command merges
                                 (the reference's two-command form), 0 = the plan decides, which
                                 is the second command: merging in the kernel measured no faster
                                 on any shape of the benchmark and slower on some */
    uint32_t max_stages;     /* 0 = the plan decides; >= 2 caps the stages of the page ring (the
                                bytes a CTA keeps in flight) */
    uint32_t producer_warps; /* balanced plans: 0 = the plan decides, 1 = one warp issues the page
                                copies of all page slots, pages_per_stage = one warp per slot */
    uint32_t reserved;       /* zero */
} lb_paged_decode_options;

typedef struct lb_paged_decode_plan_info {
    int32_t algorithm;       /* LB_DECODE_DIRECT / _SPLIT_K / _BALANCED / _CLUSTER_SPLIT */
    uint32_t partitions;
    uint32_t heads_per_cta;
    uint32_t q_tiles;        /* 16-row MMA tiles per KV head group handled by one CTA */
    uint32_t q_blocks;       /* CTAs per KV head needed to cover the GQA group */
    uint32_t pages_per_stage;
    uint32_t stages;
    uint32_t grid, block, shared_bytes;
    uint32_t merge_grid, merge_block;
    uint32_t commands;       /* 1 direct or cluster split, 2 split or balanced (partials + merge) */
    size_t workspace_numel;  /* F32 elements the caller must bind (0 for direct) */
    size_t workspace_bytes;
    uint32_t merged_in_kernel; /* 1: a split-K or balanced plan that merges its partial states in
                                  the decode kernel (commands == 1, the workspace is still bound) */
    uint32_t reserved;
} lb_paged_decode_plan_info;

/* Bf16PagedBatchDecodeArgs, decode.rs:1451-1487, plus the split-K workspace
 * (Bf16SingleDecodeSplitKArgs.workspace, :1420-1449).  workspace is ignored by direct plans. */
typedef struct lb_paged_decode_args {
    lb_handle query, key_pages, value_pages, page_indptr, page_indices, last_page_len; /* Read */
    lb_handle output, lse;                                                              /* Write */
    lb_handle workspace;                                                                /* ReadWrite<f32> */
} lb_paged_decode_args;

/* DecodeProvider::load, decode.rs:1009-1014 */
lb_status lb_decode_provider_load(int device, lb_decode_provider **out);
void lb_decode_provider_destroy(lb_decode_provider *provider);
/* Reads (and clears) the provider's device status word: 0 = no kernel of this provider gave up
 * on a bounded wait since the last read (1 = a wait inside a CTA, 2 = the wait of a gathering
 * command for the other ranks; 0x1000 | site = the checked build of the library found a computed
 * index outside its operand and skipped the access).  Synchronises the device.  No reference
 * counterpart: the reference's kernels have no waits. */
lb_status lb_decode_provider_device_status(const lb_decode_provider *provider, int32_t *status);
/* DecodeProvider::plan_bf16_paged_batch, decode.rs:1067-1103; options may be NULL. */
lb_status lb_paged_decode_plan_create(const lb_decode_provider *provider,
                                      const lb_paged_spec *spec,
                                      const lb_paged_decode_options *options,
                                      lb_paged_decode_plan **out);
void lb_paged_decode_plan_destroy(lb_paged_decode_plan *plan);
/* Bf16PagedBatchDecodePlan::{spec, algorithm}, :1189-1196, and
 * workspace_required_{numel,bytes}, :1313-1319 */
lb_status lb_paged_decode_plan_info_get(const lb_paged_decode_plan *plan, lb_paged_spec *spec,
                                        lb_paged_decode_plan_info *info);
/* Bf16PagedBatchDecodePlan::enqueue_into, decode.rs:1199-1296 (direct) and the two-command
 * shape of Bf16SingleDecodeSplitKPlan::enqueue_into, :1322-1389 (split-K). */
lb_status lb_paged_decode_enqueue(const lb_paged_decode_plan *plan, lb_scope *scope,
                                  const lb_paged_decode_args *args);
/* The plan-time split heuristic as a pure function (testable without a device). */
lb_status lb_paged_decode_choose(const lb_paged_spec *spec, uint32_t sm_count,
                                 const lb_paged_decode_options *options,
                                 lb_paged_decode_plan_info *info);

/* No counterpart in the reference.  Split-K paged decode for a caller that has no way to
 * allocate device memory and so cannot bind the workspace a split plan requires: for example a
 * plug-in whose engine owns every device byte and forbids cudaMalloc, or a loop that must stay out
 * of the allocator.  The partial states go to a fixed array inside the library (on every GPU that
 * loads it, for the life of the process) instead; inputs and outputs are still the caller's raw
 * device pointers.  Same kernels, same results as a split plan with `partitions` chunks (>= 2).
 *   - what is checked: the spec, `partitions`, page_indices_len >= batch, that every pointer is
 *     device memory of the stream's GPU (BufferContextMismatch otherwise) and that query, pools
 *     and output are 16-byte aligned.  Raw pointers carry no length: the caller guarantees the
 *     lengths lb_paged_decode_enqueue would check (Q and O batch*qh*128, the pools
 *     max_pages*16*kvh*128, page_indptr batch+1, last_page_len batch, LSE batch*qh);
 *   - limit: batch * query_heads * partitions <= lb_paged_decode_split_noalloc_max_states()
 *     (16384 states = 8.1 MiB); beyond it the call fails with LB_STATIC_SCRATCH_EXCEEDED and
 *     launches nothing;
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine;
 *   - the first call on each GPU looks up the array's device address and sets kernel attributes
 *     (under a lock, so two threads may race to it); make that first call before any stream
 *     capture;
 *   - every call shares the one array and finds the previous call's states in it; nothing has to
 *     start at zero (each state a call merges is written by that call first), but two calls that
 *     overlap on the GPU -- different streams, or replays in flight together -- race on it;
 *   - a CTA that gives up on a bounded wait leaves its rows unwritten and sets a status word
 *     inside the library; lb_paged_decode_split_noalloc_status reads and clears it (it
 *     synchronises the device and allocates nothing).  0 = every call since the last read ran to
 *     completion. */
size_t lb_paged_decode_split_noalloc_max_states(void);
lb_status lb_paged_decode_split_noalloc(const lb_paged_spec *spec, uint32_t partitions,
                                        void *stream, const void *query, const void *key_pages,
                                        const void *value_pages, const int32_t *page_indptr,
                                        const int32_t *page_indices, size_t page_indices_len,
                                        const int32_t *last_page_len, void *output, float *lse);
lb_status lb_paged_decode_split_noalloc_status(int device, int32_t *status);

/* ---- output rows across GPUs (no reference counterpart) ------------------------------------------- */

/* The reference is a single-GPU operator layer.  Paged decode shards over the GPUs of a node by
 * request (or by KV head) with no exchange step; only the finished output rows cross GPUs, when the
 * caller wants one contiguous result.  One process per GPU; a peer group is the set of those
 * processes.  Creating a group, a peer buffer, and enqueueing a gathering command are collective:
 * every rank makes the same calls in the same order. */
typedef struct lb_peer_group lb_peer_group;
typedef struct lb_peer_buffer lb_peer_buffer;
#define LB_PEER_ID_BYTES 128u
#define LB_PEER_MAX_RANKS 32

/* One rank makes the id (ncclGetUniqueId) and hands it to the others by any host channel. */
lb_status lb_peer_group_unique_id(uint8_t *id /* [LB_PEER_ID_BYTES] */);
/* Joins the group (ncclCommInitRank; the library is resolved with dlopen here, so a single-GPU
 * host never loads it) and maps the group's signal block on every rank. */
lb_status lb_peer_group_create(int device, int world, int rank, const uint8_t *id,
                               lb_peer_group **out);
/* Not collective.  Call it after every rank has finished using the group (a host barrier). */
void lb_peer_group_destroy(lb_peer_group *group);
int lb_peer_group_rank(const lb_peer_group *group);
int lb_peer_group_world(const lb_peer_group *group);

/* `bytes` of device memory on every rank (cudaMalloc, zeroed), each rank's copy mapped into every
 * other rank's address space through CUDA IPC.  The local copy is bound like any caller buffer. */
lb_status lb_peer_buffer_create(lb_peer_group *group, size_t bytes, lb_peer_buffer **out);
void lb_peer_buffer_destroy(lb_peer_buffer *buffer); /* after a host barrier, as the group */
void *lb_peer_buffer_local(const lb_peer_buffer *buffer);
size_t lb_peer_buffer_bytes(const lb_peer_buffer *buffer);

/* The all-gather of per-rank rows as ONE command of the scope: ncclAllGather (grouped
 * ncclBroadcast when the ranks' row counts differ) on the queue's own stream, recorded like the
 * reference's vendor-library commands (record_external_submission, crates/loom-infer-cuda/src/
 * command/submission.rs:240-252; failure path :254-272): it counts in submitted(), completes under
 * the scope's fence, can be captured, and a failure poisons scope and queue with
 * LB_EXTERNAL_COMMAND (operand "nccl", a = the library's result code). */
typedef struct lb_output_gather_plan lb_output_gather_plan;
typedef struct lb_output_gather_args {
    lb_handle local;    /* Read:  this rank's rows, rows_per_rank[rank] * row_numel elements */
    lb_handle gathered; /* Write: every rank's rows in rank order, sum(rows) * row_numel elements */
} lb_output_gather_args;
lb_status lb_output_gather_plan_create(const lb_peer_group *group, int dtype,
                                       const size_t *rows_per_rank /* [world] */, size_t row_numel,
                                       lb_output_gather_plan **out);
void lb_output_gather_plan_destroy(lb_output_gather_plan *plan);
lb_status lb_output_gather_enqueue(const lb_output_gather_plan *plan, lb_scope *scope,
                                   const lb_output_gather_args *args);

/* Paged decode that leaves its result gathered on every rank, with no collective kernel and no
 * extra launch: the plan's own kernels store every finished row straight into every rank's copy
 * of `output` / `lse` (plain stores to peer-mapped memory over NVLink; never a TMA or multicast
 * load from a peer), the last CTA of the command's last kernel publishes an epoch to every rank
 * and waits, bounded by the plan's wait_limit_us, until every rank has published its own (when
 * the wait runs out the provider's device status word reads 2 and the gathered result is
 * incomplete on this GPU).  The command therefore completes under the scope's fence only when the
 * gathered result is whole on this GPU.  Same plan, same command count, same checks as lb_paged_decode_enqueue; `output` and
 * `lse` of the args are this rank's copies of the two peer buffers.
 *   Row r of the local batch, local query head h is row
 *       dest_rows[r] * gathered_query_heads + head_offset + h
 *   of the gathered BF16 [total_requests * gathered_query_heads, 128] output and F32 LSE, so a
 *   batch split by request (any assignment, no un-permute afterwards) and a batch split by KV
 *   head are both one call.
 *   Every rank must enqueue the same sequence of gathering commands on the group.  A rank must
 *   not overwrite a gathered buffer its peers may still be reading: alternate two buffers step by
 *   step (a rank that has completed step n+1 knows every rank has completed step n). */
typedef struct lb_gather_layout {
    size_t total_requests;       /* requests of the gathered result, over all ranks */
    size_t gathered_query_heads; /* query heads per request of the gathered result */
    size_t head_offset;          /* first gathered query head this rank's heads map to */
    uint32_t defer_wait;         /* 1: more gathering commands of the same step follow on this
                                    queue; this one stores its rows but leaves the
                                    epoch and the wait to the step's last gathering command, whose
                                    completion then covers the rows of all of them.  Every rank
                                    must make the same choice */
    uint32_t reserved;
} lb_gather_layout;
typedef struct lb_paged_decode_gather_args {
    lb_paged_decode_args decode; /* output / lse: bound local copies of the peer buffers below */
    lb_handle dest_rows;         /* Read<i32> [batch]: gathered request index of each local request */
} lb_paged_decode_gather_args;
lb_status lb_paged_decode_enqueue_gathered(const lb_paged_decode_plan *plan, lb_scope *scope,
                                           const lb_paged_decode_gather_args *args,
                                           const lb_gather_layout *layout, lb_peer_group *group,
                                           const lb_peer_buffer *output, const lb_peer_buffer *lse);

/* ---- RoPE + paged KV append provider --------------------------------------------------------- */

typedef struct lb_rope_provider lb_rope_provider;         /* RopeProvider, rope/mod.rs:579-683 */
typedef struct lb_rope_append_plan lb_rope_append_plan;   /* Bf16RopePagedKvAppend{,Tokens}Plan */

/* Bf16RopePagedKvAppendArgs / ...TokensArgs, rope/mod.rs:963-1077.  batch_indices and
 * positions are ignored by the one-token-per-request plan. */
typedef struct lb_rope_append_args {
    lb_handle query, key, value, batch_indices, positions, page_indptr, page_indices,
        last_page_len;                           /* Read */
    lb_handle query_output, key_pages, value_pages; /* Write */
    lb_handle workspace; /* ReadWrite<i32>, extended plans only (workspace_numel elements) */
} lb_rope_append_args;

typedef struct lb_rope_append_plan_info {
    int32_t explicit_tokens; /* 0: one token per request; 1: explicit token list */
    uint32_t tokens;
    uint32_t grid, block, shared_bytes;
    uint32_t commands;      /* 1; 2 for an extended plan (validate, then rotate and scatter) */
    size_t workspace_numel; /* I32 elements the caller must bind; 0 unless the plan is extended */
} lb_rope_append_plan_info;

/* RopeProvider::load, rope/mod.rs:586-590 */
lb_status lb_rope_provider_load(int device, lb_rope_provider **out);
void lb_rope_provider_destroy(lb_rope_provider *provider);
/* Reads (and clears) the provider's device status word.  The append kernels have no waits; only the
 * checked build of the library (LB_DEBUG_BOUNDS: every computed index compared with its operand's
 * length, a violation recorded as 0x1000 | site and the access skipped) ever writes it. */
lb_status lb_rope_provider_device_status(const lb_rope_provider *provider, int32_t *status);
/* Plan options of the append (NULL = all zero). */
typedef struct lb_rope_append_options {
    uint32_t indices_capacity; /* as lb_paged_decode_options.indices_capacity */
    uint32_t one_command;      /* extended (any-total) plans: 1 = validation and scatter in ONE
                                  kernel whose token CTAs wait for the validators on words of
                                  the queue (calls whose whole grid is resident at once: up to
                                  2048 tokens); 0 = two commands, which measured faster */
    uint32_t reserved[2];
} lb_rope_append_options;
/* RopeProvider::plan_bf16_paged_append, rope/mod.rs:628-654 */
lb_status lb_rope_append_plan_create(const lb_rope_provider *provider, const lb_paged_spec *spec,
                                     lb_rope_append_plan **out);
lb_status lb_rope_append_plan_create_with(const lb_rope_provider *provider,
                                          const lb_paged_spec *spec,
                                          const lb_rope_append_options *options,
                                          lb_rope_append_plan **out);
/* RopeProvider::plan_bf16_paged_append_tokens, rope/mod.rs:656-682 */
lb_status lb_rope_append_tokens_plan_create(const lb_rope_provider *provider,
                                            const lb_append_tokens_spec *spec,
                                            lb_rope_append_plan **out);
lb_status lb_rope_append_tokens_plan_create_with(const lb_rope_provider *provider,
                                                 const lb_append_tokens_spec *spec,
                                                 const lb_rope_append_options *options,
                                                 lb_rope_append_plan **out);
void lb_rope_append_plan_destroy(lb_rope_append_plan *plan);
lb_status lb_rope_append_plan_info_get(const lb_rope_append_plan *plan,
                                       lb_rope_append_plan_info *info);
/* Bf16RopePagedKvAppend{,Tokens}Plan::enqueue_into, rope/mod.rs:758-830,846-933 */
lb_status lb_rope_append_enqueue(const lb_rope_append_plan *plan, lb_scope *scope,
                                 const lb_rope_append_args *args);

/* ---- stand-alone NeoX RoPE over contiguous NHD Q and K ----------------------------------------- */

/* Bf16RopePosIdsSpec, crates/loom-infer/src/rope/mod.rs:9-108 */
typedef struct lb_rope_pos_ids_spec {
    size_t tokens, query_heads, key_heads, head_dim, rotary_dim;
    float rope_scale, rope_theta;
} lb_rope_pos_ids_spec;
/* Bf16RopePosIdsSpec::new, rope/mod.rs:21-62: ZeroDimension, InvalidRotaryDimension (zero, odd
 * or > head_dim), InvalidRopeScale (not finite or <= 0), InvalidRopeTheta (not finite or <= 1),
 * ElementCountOverflow. */
lb_status lb_rope_pos_ids_spec_new(size_t tokens, size_t query_heads, size_t key_heads,
                                   size_t head_dim, size_t rotary_dim, float rope_scale,
                                   float rope_theta, lb_rope_pos_ids_spec *out);
size_t lb_rope_pos_ids_spec_query_numel(const lb_rope_pos_ids_spec *spec);
size_t lb_rope_pos_ids_spec_key_numel(const lb_rope_pos_ids_spec *spec);

typedef struct lb_rope_pos_ids_plan lb_rope_pos_ids_plan; /* Bf16RopePosIdsPlan */
/* Bf16RopePosIdsArgs, crates/loom-infer-cuda/src/rope/mod.rs (resolve_rrrww at :705-711) */
typedef struct lb_rope_pos_ids_args {
    lb_handle query, key, position_ids; /* Read: BF16, BF16, I32 */
    lb_handle query_output, key_output; /* Write: BF16 */
} lb_rope_pos_ids_args;
/* RopeProvider::plan_bf16_pos_ids, rope/mod.rs:592-626: UnsupportedHeadDimension and
 * UnsupportedRotaryDimension unless both are 128; StateCountOverflow / StateCountOutOfRange. */
lb_status lb_rope_pos_ids_plan_create(const lb_rope_provider *provider,
                                      const lb_rope_pos_ids_spec *spec,
                                      lb_rope_pos_ids_plan **out);
void lb_rope_pos_ids_plan_destroy(lb_rope_pos_ids_plan *plan);
/* Bf16RopePosIdsPlan::enqueue_into, rope/mod.rs:698-742.  One command.  A token whose position
 * id is negative is left unwritten by the device guard (rope/mod.rs:64-67); the other tokens of
 * the call are rotated. */
lb_status lb_rope_pos_ids_enqueue(const lb_rope_pos_ids_plan *plan, lb_scope *scope,
                                  const lb_rope_pos_ids_args *args);

/* ---- state merge ------------------------------------------------------------------------------- */

/* Merges caller-provided attention states: the split-K merge kernel as an operator of its own.
 * No reference counterpart yet: the reference lists merge_state(s) as planned
 * (docs/flashinfer-parity.md:38); the arithmetic is its contiguous split-K merge
 * (single_decode_bf16_split_k_merge_reference, crates/loom-infer/src/attention/single_decode/
 * mod.rs:343-379).  states is F32 [rows, partitions, 130] with [max_log2, normaliser, wv[128]]
 * per state (single_decode/mod.rs:10-13); output BF16 [rows, 128]; lse F32 [rows], base 2.  A state
 * with a zero normaliser is skipped; a row whose states are all empty is left unwritten.  An
 * engine that splits one request's KV over several GPUs gathers the per-GPU states and merges
 * them with this. */
typedef struct lb_state_merge_plan lb_state_merge_plan;
typedef struct lb_state_merge_args {
    lb_handle states; /* Read<f32> */
    lb_handle output; /* Write<bf16> */
    lb_handle lse;    /* Write<f32> */
} lb_state_merge_args;
/* ZeroDimension (rows or partitions zero), InvalidPartitionCount (> 65535),
 * StateCountOutOfRange, ElementCountOverflow. */
lb_status lb_state_merge_plan_create(const lb_decode_provider *provider, size_t rows,
                                     size_t partitions, lb_state_merge_plan **out);
void lb_state_merge_plan_destroy(lb_state_merge_plan *plan);
lb_status lb_state_merge_enqueue(const lb_state_merge_plan *plan, lb_scope *scope,
                                 const lb_state_merge_args *args);

/* ---- paged causal prefill ------------------------------------------------------------------------ */

/* Bf16PagedPrefillSpec, crates/loom-infer/src/attention/paged_prefill/mod.rs:19-159.  Query and
 * output are BF16 [nnz_qo, query_heads, 128], partitioned into requests by qo_indptr; the pools are
 * the decode pools [max_num_pages, 16, kv_heads, 128]; LSE is F32 [nnz_qo, query_heads], base 2.
 * Causal mask, bottom-right aligned: query i of a request sees kv_index <= kv_len - qo_len + i. */
typedef struct lb_prefill_spec {
    size_t batch_size, nnz_qo, max_num_pages, num_query_heads, num_kv_heads;
    float softmax_scale; /* 1/sqrt(128) */
} lb_prefill_spec;

/* Bf16PagedPrefillSpec::new, paged_prefill/mod.rs:29-91 */
lb_status lb_prefill_spec_new(size_t batch_size, size_t nnz_qo, size_t max_num_pages,
                              size_t num_query_heads, size_t num_kv_heads, size_t head_dim,
                              size_t page_size, lb_prefill_spec *out);
/* numel accessors, paged_prefill/mod.rs:129-150 */
size_t lb_prefill_spec_query_numel(const lb_prefill_spec *spec);
size_t lb_prefill_spec_kv_pages_numel(const lb_prefill_spec *spec);
size_t lb_prefill_spec_lse_numel(const lb_prefill_spec *spec);
/* validate_metadata, paged_prefill/mod.rs:161-235 (host copies of the metadata) */
lb_status lb_prefill_spec_validate_metadata(const lb_prefill_spec *spec, const int32_t *qo_indptr,
                                            size_t qo_indptr_len, const int32_t *page_indptr,
                                            size_t page_indptr_len, const int32_t *page_indices,
                                            size_t page_indices_len,
                                            const int32_t *last_page_len,
                                            size_t last_page_len_len);
/* Bf16PagedPrefillMetadata::causal_kv_end, :321-329.  The metadata must have passed
 * validate_metadata.  Returns 0 (None) or 1 (Some). */
int lb_prefill_metadata_causal_kv_end(const lb_prefill_spec *spec, const int32_t *qo_indptr,
                                      const int32_t *page_indptr, const int32_t *last_page_len,
                                      size_t request, size_t query_index, size_t *kv_end);

typedef struct lb_prefill_provider lb_prefill_provider;     /* PrefillProvider, prefill.rs:2278-2330 */
typedef struct lb_paged_prefill_plan lb_paged_prefill_plan; /* Bf16PagedPrefillPlan, :2440-2584 */

/* Bf16PagedPrefillAlgorithm, prefill.rs:2411-2426, for this provider */
enum {
    LB_PREFILL_TOKEN_PARALLEL = 0, /* one CTA per (request, KV head, tile of packed query rows):
                                      warps share the row tiles and the pages (mma.sync); the
                                      choice for short, latency-bound calls; one command */
    LB_PREFILL_TILED = 1           /* one CTA per (request, KV head, 128 packed query rows) on the
                                      tcgen05 tensor cores with the accumulators in TMEM; the
                                      choice for long prompts; one command, or -- when the plan
                                      cuts the KV range of every tile into `partitions` chunks so
                                      that a short chunk over a long cache fills the device --
                                      two: chunk states into a workspace, then the LSE merge of
                                      the split-K contract (single_decode/mod.rs:343-379) */
};

typedef struct lb_paged_prefill_options {
    uint32_t q_tiles;          /* token-parallel only.  0 = plan-time heuristic; 16-row MMA tiles
                                  one CTA owns (1, 2, 4, 8): 8 / q_tiles warps then take different
                                  pages of the same rows */
    uint32_t indices_capacity; /* as lb_paged_decode_options.indices_capacity */
    uint32_t algorithm;        /* 0 = plan-time heuristic, 1 = token-parallel, 2 = tiled */
    uint32_t partitions;       /* tiled only.  0 = plan-time heuristic, 1 = one CTA per tile, N > 1
                                  (at most 64) = the 64-token KV blocks of every tile are shared
                                  out to up to N CTAs by the balanced rule of the split-K contract
                                  (single_decode/mod.rs:171-185); see min_chunk_blocks */
    uint32_t wait_limit_us;    /* tiled only: limit of every bounded wait, in microseconds; 0 = about
                                  two seconds.  When it runs out the CTA writes nothing, waits (bounded
                                  again) for its copies and MMAs in flight, frees its TMEM, and the
                                  provider's status word reads 1 */
    uint32_t test_lost_copy;   /* tiled only, tests of that give-up path: 1 = the barrier of a CTA's
                                  first K block expects 16 bytes more than its copies deliver */
    uint32_t reserved[2];
} lb_paged_prefill_options;

typedef struct lb_paged_prefill_plan_info {
    int32_t algorithm;
    uint32_t q_tiles, pages_per_stage, stages;
    uint32_t rows_per_cta;  /* packed (token, head-in-group) rows per CTA = 16 * q_tiles */
    uint32_t tiles;         /* upper bound of row tiles per KV head the grid covers */
    uint32_t grid, block, shared_bytes;
    uint32_t commands;      /* 1, or 2 when partitions > 1 */
    uint32_t partitions;    /* KV chunks per tile (1 unless tiled) */
    uint32_t merge_grid, merge_block; /* second command of a split plan */
    uint32_t min_chunk_blocks; /* on the device a tile of B 64-token blocks uses
                                  min(partitions, max(1, B / min_chunk_blocks)) chunks, and a tile
                                  of one chunk is finished by the first command: 16 when the plan
                                  chose the count (the KV length is not known at plan time; fewer
                                  than three chunks then count as one), 1 when the caller did */
    size_t workspace_numel; /* F32 elements the caller must bind: nnz_qo * qh * partitions * 130,
                               0 when partitions == 1 */
} lb_paged_prefill_plan_info;

/* Bf16PagedPrefillArgs, prefill.rs:2853-2891, plus the workspace of a split plan (as
 * Bf16SingleDecodeSplitKArgs.workspace, decode.rs:1420-1449); workspace is ignored when the plan's
 * partitions == 1. */
typedef struct lb_paged_prefill_args {
    lb_handle query, key_pages, value_pages, qo_indptr, page_indptr, page_indices,
        last_page_len;     /* Read */
    lb_handle output, lse; /* Write */
    lb_handle workspace;   /* ReadWrite<f32> */
} lb_paged_prefill_args;

/* PrefillProvider::load, prefill.rs:2283-2287 */
lb_status lb_prefill_provider_load(int device, lb_prefill_provider **out);
void lb_prefill_provider_destroy(lb_prefill_provider *provider);
/* As lb_decode_provider_device_status. */
lb_status lb_prefill_provider_device_status(const lb_prefill_provider *provider, int32_t *status);
/* PrefillProvider::plan_bf16_paged, prefill.rs:2289-2329; options may be NULL.
 * StateCountOutOfRange as PagedPrefillPlanError (:2934-2940). */
lb_status lb_paged_prefill_plan_create(const lb_prefill_provider *provider,
                                       const lb_prefill_spec *spec,
                                       const lb_paged_prefill_options *options,
                                       lb_paged_prefill_plan **out);
void lb_paged_prefill_plan_destroy(lb_paged_prefill_plan *plan);
lb_status lb_paged_prefill_plan_info_get(const lb_paged_prefill_plan *plan, lb_prefill_spec *spec,
                                         lb_paged_prefill_plan_info *info);
/* Bf16PagedPrefillPlan::enqueue_into, prefill.rs:2456-2583: one command (two for a split plan;
 * both must fit the scope before anything is launched).  Errors as
 * PagedPrefillEnqueueError (:2942-2963): LengthMismatch (operands "Q", "K_pages", "V_pages",
 * "qo_indptr", "page_indptr", "last_page_len", "O", "LSE", "workspace"), PageIndicesTooShort,
 * MisalignedBuffer
 * (16 bytes here, 4 in the reference), Command errors.  Device-resident metadata is never an
 * error: a query row whose request fails the kernel's guard keeps its previous output
 * (prefill.rs:289-347). */
lb_status lb_paged_prefill_enqueue(const lb_paged_prefill_plan *plan, lb_scope *scope,
                                   const lb_paged_prefill_args *args);
/* The plan-time choice as a pure function of the spec and the device. */
lb_status lb_paged_prefill_choose(const lb_prefill_spec *spec, uint32_t sm_count,
                                  const lb_paged_prefill_options *options,
                                  lb_paged_prefill_plan_info *info);

/* ---- fixed-address CUDA Graph ------------------------------------------------------------------ */

typedef struct lb_graph_queue lb_graph_queue;           /* GraphQueue, graph/mod.rs:27-71 */
typedef struct lb_captured_graph lb_captured_graph;     /* CapturedGraph, :165-215 */
typedef struct lb_graph_exec lb_graph_exec;             /* GraphExec, :217-382 */
typedef struct lb_graph_completion lb_graph_completion; /* GraphLaunchCompletion, :384-463 */

/* The closure given to GraphQueue::capture: enqueue plans into `scope`; return LB_OK or an
 * error status (reported as LB_GRAPH_CAPTURE_RECORD). */
typedef lb_status (*lb_record_fn)(lb_scope *scope, void *user);

/* GraphQueue::new, graph/mod.rs:34-40 (private non-default stream on `device`) */
lb_status lb_graph_queue_create(int device, size_t max_commands, lb_graph_queue **out);
void lb_graph_queue_destroy(lb_graph_queue *queue);
/* GraphQueue::bindings, :43-45 */
lb_status lb_graph_queue_bindings(lb_graph_queue *queue, size_t capacity, lb_bindings **out);
/* GraphQueue::capture, :54-70; `queue` and `bindings` are moved. */
lb_status lb_graph_capture(lb_graph_queue *queue, lb_bindings *bindings, lb_record_fn record,
                           void *user, lb_captured_graph **out);
size_t lb_captured_graph_commands(const lb_captured_graph *graph);
/* CapturedGraph::instantiate, :183-206; `graph` is moved. */
lb_status lb_captured_graph_instantiate(lb_captured_graph *graph, lb_graph_exec **out);
void lb_captured_graph_destroy(lb_captured_graph *graph);
size_t lb_graph_exec_commands(const lb_graph_exec *exec);
uint64_t lb_graph_exec_launches(const lb_graph_exec *exec);
/* GraphExec::launch, :249-293 */
lb_status lb_graph_exec_launch(lb_graph_exec *exec, lb_graph_completion **out);
/* GraphExec::measure_launch_ms, :301-323: one replay plus its completion event between two
 * timing events created and destroyed by the library on the capture stream. */
lb_status lb_graph_exec_measure_launch_ms(lb_graph_exec *exec, float *milliseconds);
/* GraphExec::into_bindings, :326-339; `exec` is moved. */
lb_status lb_graph_exec_into_bindings(lb_graph_exec *exec, lb_bindings **out);
void lb_graph_exec_destroy(lb_graph_exec *exec);
uint64_t lb_graph_completion_launch_index(const lb_graph_completion *completion);
lb_status lb_graph_completion_is_complete(lb_graph_completion *completion, int *complete);
/* GraphLaunchCompletion::wait, :420-437; `completion` is moved. */
lb_status lb_graph_completion_wait(lb_graph_completion *completion);
void lb_graph_completion_abandon(lb_graph_completion *completion);

/* ---- host-side fault injection (tests) ------------------------------------------------------------ */

/* Replaces the CUDA driver layer under the runtime with an in-process fake: no device is
 * touched, launches and event operations succeed unless a failure is armed.  The fake lets
 * the ownership / poisoning state machine be exercised on a machine without a GPU.  Kernels
 * never run under the fake; it cannot produce results. */
void lb_test_use_fake_driver(int enable, int fake_sm_count);
/* Arms the fake: the n-th next call of `what` ("launch", "event_record", "event_sync",
 * "event_query", "stream_sync", "device_sync", "graph_launch", "capture_begin",
 * "capture_end", "instantiate") returns `cuda_error`.  n = 1 fails the very next call. */
void lb_test_fake_fail(const char *what, int n, int cuda_error);
/* Number of kernel launches the fake (or the real driver layer) has accepted so far. */
uint64_t lb_test_launch_count(void);
/* 1 once lb_paged_decode_split_noalloc has resolved its static array on `device` (never under the
 * fake driver, which has no device to resolve it on). */
int lb_test_noalloc_is_set_up(int device);

#ifdef __cplusplus
}
#endif
#endif /* LOOM_B200_H */
