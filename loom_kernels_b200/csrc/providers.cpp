// Decode and RoPE-append providers: immutable plans and checked enqueue.
//
// Mirrors DecodeProvider / Bf16PagedBatchDecodePlan
// (crates/loom-infer-cuda/src/attention/decode.rs:1001-1104,1181-1297), the two-command
// split-K enqueue shape (:1322-1389) and RopeProvider / Bf16RopePagedKvAppend{,Tokens}Plan
// (crates/loom-infer-cuda/src/rope/mod.rs:579-683,745-934) of the reference.  A plan fixes the
// algorithm, split count, launch shape and workspace size before any enqueue; enqueue performs
// no re-dispatch and has no fallback.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>

#include "kernels.hpp"
#include "peer_group.hpp"
#include "runtime.hpp"

using namespace lb;

struct lb_decode_provider {
    int device = 0, sm_count = 0;
    size_t smem_optin = 0;
    int clock_khz = 0;
    int32_t *status = nullptr; // device word written by a kernel that gave up on a wait
};

struct lb_paged_decode_plan {
    lb_paged_spec spec;
    DecodeChoice choice;
    int device = 0;
    int32_t *status = nullptr;
    bool indices_capacity = false; // page_indices may be bound longer than the table in use
    long long wait_cycles = 0;     // 0 = the kernels' default (about two seconds)
    int32_t test_skip_page = 0;
};

// The one-command extended append keeps its slot hash set within this many bytes per CTA.
constexpr size_t kFusedHashBytes = 16384;

struct lb_rope_provider {
    int device = 0, sm_count = 0;
    size_t smem_optin = 0;
    int32_t *status = nullptr; // device word: the checked (bounds) build, a wait that ran out
    int fused_ctas_per_sm = 8; // CTAs of the one-command extended append that fit one SM
};

struct lb_rope_append_plan {
    lb_paged_spec spec;
    bool explicit_tokens = false;
    size_t tokens = 0;
    int device = 0;
    uint32_t grid = 0, block = 256, shared_bytes = 0, hash_slots = 0;
    // extended plans: validate + scatter as two commands over a caller-bound I32 workspace
    bool extended = false;
    uint32_t validate_grid = 0;
    size_t workspace_numel = 0;
    // ... or as ONE command whose token CTAs wait for the validators on words of the queue
    bool fused = false, fused_possible = false;
    uint32_t fused_grid = 0, fused_validators = 0;
    bool indices_capacity = false; // page_indices may be bound longer than the table in use
    int32_t *status = nullptr;
};

struct lb_state_merge_plan {
    size_t rows = 0, partitions = 0;
    int device = 0;
};

struct lb_rope_pos_ids_plan {
    lb_rope_pos_ids_spec spec;
    int device = 0;
    uint32_t grid = 0;
    float inverse_frequency[64];
};

namespace {

const float kLog2E = 1.44269504088896340736f;

lb_status require_exact_len(const char *operand, size_t actual, size_t expected) {
    if (actual == expected) return LB_OK;
    return fail(LB_ENQUEUE_LENGTH_MISMATCH, operand, (int64_t)expected, (int64_t)actual);
}

// The reference requires 4-byte bases (decode.rs:1585-1599); the 16-byte vector and TMA
// accesses of these kernels need 16.
lb_status require_alignment(const char *operand, const void *ptr, uint64_t alignment) {
    const uint64_t address = (uint64_t)(uintptr_t)ptr;
    if (address % alignment == 0) return LB_OK;
    return fail(LB_MISALIGNED_BUFFER, operand, (int64_t)address, (int64_t)alignment);
}

lb_status load_device(int device, int *sm_count, size_t *smem_optin) {
    int count = 0;
    int rc = driver().device_count(&count);
    if (rc) return fail(LB_DRIVER, "device_count", rc);
    if (device < 0 || device >= count) return fail(LB_INVALID_ARGUMENT, "device", device);
    int major = 0, minor = 0;
    size_t l2 = 0;
    if ((rc = driver().device_props(device, sm_count, &major, &minor, smem_optin, &l2)))
        return fail(LB_DRIVER, "device_props", rc);
    if (major != 10) return fail(LB_UNSUPPORTED_DEVICE, nullptr, major * 10 + minor);
    return LB_OK;
}

void fill_info(const DecodeChoice &c, lb_paged_decode_plan_info *info) {
    info->algorithm = (int32_t)c.algorithm;
    info->partitions = c.partitions;
    info->heads_per_cta = c.heads_per_cta;
    info->q_tiles = c.q_tiles;
    info->q_blocks = c.q_blocks;
    info->pages_per_stage = c.pages_per_stage;
    info->stages = c.stages;
    info->grid = c.grid;
    info->block = c.block;
    info->shared_bytes = c.shared_bytes;
    info->merge_grid = c.merge_grid;
    info->merge_block = c.merge_block;
    info->commands = c.algorithm == LB_DECODE_DIRECT || c.algorithm == LB_DECODE_CLUSTER_SPLIT ||
                             c.merged_in_kernel
                         ? 1
                         : 2;
    info->workspace_numel = c.workspace_numel;
    info->workspace_bytes = c.workspace_numel * sizeof(float);
    info->merged_in_kernel = c.merged_in_kernel;
    info->reserved = 0;
}

} // namespace

extern "C" {

// ---- decode ----------------------------------------------------------------------------------

lb_status lb_decode_provider_load(int device, lb_decode_provider **out) {
    if (!out) return fail(LB_INVALID_ARGUMENT, "out");
    *out = nullptr;
    int sm_count = 0;
    size_t smem = 0;
    lb_status rc = load_device(device, &sm_count, &smem);
    if (rc) return rc;
    int32_t *status = nullptr;
    const int error = driver().configure(device, [&]() -> int {
        int e = configure_decode_kernels(smem);
        if (e) return e;
        if ((e = cudaMalloc((void **)&status, 64))) return e;
        return cudaMemset(status, 0, 64);
    });
    if (error) return fail(LB_DRIVER, "provider_load", error);
    lb_decode_provider *provider = new lb_decode_provider();
    provider->device = device;
    provider->sm_count = sm_count;
    provider->smem_optin = smem;
    provider->status = status;
    driver().device_clock_khz(device, &provider->clock_khz);
    *out = provider;
    return LB_OK;
}

void lb_decode_provider_destroy(lb_decode_provider *provider) {
    if (!provider) return;
    if (provider->status) {
        int32_t *status = provider->status;
        driver().configure(provider->device, [&]() -> int { return cudaFree(status); });
    }
    delete provider;
}

lb_status lb_decode_provider_device_status(const lb_decode_provider *provider, int32_t *status) {
    if (!provider || !status) return fail(LB_INVALID_ARGUMENT, "provider");
    *status = 0;
    if (!provider->status) return LB_OK;
    const int error = driver().configure(provider->device, [&]() -> int {
        int e = cudaMemcpy(status, provider->status, sizeof(int32_t), cudaMemcpyDeviceToHost);
        if (e) return e;
        return cudaMemset(provider->status, 0, sizeof(int32_t));
    });
    if (error) return fail(LB_DRIVER, "device_status", error);
    return LB_OK;
}

lb_status lb_paged_decode_plan_create(const lb_decode_provider *provider, const lb_paged_spec *spec,
                                      const lb_paged_decode_options *options,
                                      lb_paged_decode_plan **out) {
    if (!provider || !spec || !out) return fail(LB_INVALID_ARGUMENT, "provider");
    *out = nullptr;
    // a spec not made by lb_paged_spec_new is re-validated
    lb_paged_spec checked;
    lb_status rc = lb_paged_spec_new(spec->batch_size, spec->max_num_pages, spec->num_query_heads,
                                     spec->num_kv_heads, LB_HEAD_DIM, LB_PAGE_SIZE, &checked);
    if (rc) return rc;
    if (spec->max_num_pages > (size_t)0x7fffffff / LB_PAGE_SIZE ||
        spec->num_kv_heads > 0x7fffffffu / LB_HEAD_DIM)
        return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)spec->max_num_pages);
    DecodeChoice choice;
    if ((rc = choose_decode(checked, (uint32_t)provider->sm_count, provider->smem_optin, options,
                            &choice)))
        return rc;
    if (options && options->indices_capacity > 1)
        return fail(LB_LAUNCH_CONTRACT, "indices_capacity", options->indices_capacity);
    if (options && options->test_skip_page && choice.algorithm == LB_DECODE_BALANCED)
        return fail(LB_LAUNCH_CONTRACT, "test_skip_page", options->test_skip_page);
    lb_paged_decode_plan *plan = new lb_paged_decode_plan();
    plan->indices_capacity = options && options->indices_capacity == 1;
    if (options && options->wait_limit_us) {
        const long long khz = provider->clock_khz > 0 ? provider->clock_khz : 1965000;
        plan->wait_cycles = (long long)options->wait_limit_us * khz / 1000;
    }
    plan->test_skip_page = options ? (int32_t)options->test_skip_page : 0;
    plan->spec = checked;
    plan->choice = choice;
    plan->device = provider->device;
    plan->status = provider->status;
    *out = plan;
    return LB_OK;
}

void lb_paged_decode_plan_destroy(lb_paged_decode_plan *plan) { delete plan; }

lb_status lb_paged_decode_plan_info_get(const lb_paged_decode_plan *plan, lb_paged_spec *spec,
                                        lb_paged_decode_plan_info *info) {
    if (!plan) return fail(LB_INVALID_ARGUMENT, "plan");
    if (spec) *spec = plan->spec;
    if (info) fill_info(plan->choice, info);
    return LB_OK;
}

namespace {

// Where a gathering enqueue sends its rows (lb_paged_decode_enqueue_gathered).
struct GatherTarget {
    const lb_gather_layout *layout;
    lb_peer_group *group;
    const lb_peer_buffer *output, *lse;
    lb_handle dest_rows;
};

lb_status enqueue_decode(const lb_paged_decode_plan *plan, lb_scope *scope,
                         const lb_paged_decode_args *args, const GatherTarget *gather);

} // namespace

lb_status lb_paged_decode_enqueue(const lb_paged_decode_plan *plan, lb_scope *scope,
                                  const lb_paged_decode_args *args) {
    if (!plan || !scope || !args) return fail(LB_INVALID_ARGUMENT, "plan");
    return enqueue_decode(plan, scope, args, nullptr);
}

lb_status lb_paged_decode_enqueue_gathered(const lb_paged_decode_plan *plan, lb_scope *scope,
                                           const lb_paged_decode_gather_args *args,
                                           const lb_gather_layout *layout, lb_peer_group *group,
                                           const lb_peer_buffer *output, const lb_peer_buffer *lse) {
    if (!plan || !scope || !args || !layout || !group || !output || !lse)
        return fail(LB_INVALID_ARGUMENT, "plan");
    if (peer_group_device(group) != plan->device)
        return fail(LB_BUFFER_CONTEXT_MISMATCH, nullptr, peer_group_device(group), plan->device);
    size_t heads_end, rows;
    if (layout->total_requests == 0 || layout->gathered_query_heads == 0)
        return fail(LB_ZERO_DIMENSION);
    if (layout->defer_wait > 1) return fail(LB_LAUNCH_CONTRACT, "defer_wait", layout->defer_wait);
    if (__builtin_add_overflow(layout->head_offset, plan->spec.num_query_heads, &heads_end) ||
        heads_end > layout->gathered_query_heads)
        return fail(LB_INVALID_HEAD_MAPPING, nullptr, (int64_t)layout->gathered_query_heads,
                    (int64_t)layout->head_offset);
    if (__builtin_mul_overflow(layout->total_requests, layout->gathered_query_heads, &rows) ||
        rows > (size_t)0x7fffffff)
        return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)rows);
    const GatherTarget target = {layout, group, output, lse, args->dest_rows};
    return enqueue_decode(plan, scope, &args->decode, &target);
}

namespace {

lb_status enqueue_decode(const lb_paged_decode_plan *plan, lb_scope *scope,
                         const lb_paged_decode_args *args, const GatherTarget *gather) {
    const lb_paged_spec &spec = plan->spec;
    const DecodeChoice &c = plan->choice;
    const bool balanced = c.algorithm == LB_DECODE_BALANCED;
    const bool split = c.algorithm == LB_DECODE_SPLIT_K || balanced; // states in a workspace
    const bool merge_command = split && !c.merged_in_kernel;          // ... merged by a second command
    if (scope->queue->device != plan->device)
        return fail(LB_BUFFER_CONTEXT_MISMATCH, nullptr, plan->device, scope->queue->device);
    // both commands of a split plan must fit before anything is launched (decode.rs:1327)
    lb_status rc = require_command_capacity(*scope, merge_command ? 2 : 1);
    if (rc) return rc;

    // operand 8 is the workspace of a split plan, else the row map of a gathering enqueue
    OperandRequest requests[10] = {
        {args->query, LB_BF16, false},       {args->key_pages, LB_BF16, false},
        {args->value_pages, LB_BF16, false}, {args->page_indptr, LB_I32, false},
        {args->page_indices, LB_I32, false}, {args->last_page_len, LB_I32, false},
        {args->output, LB_BF16, true},       {args->lse, LB_F32, true},
        {args->workspace, LB_F32, true},
    };
    size_t count = split ? 9 : 8;
    size_t rows_operand = 0;
    if (gather) {
        rows_operand = count;
        requests[count++] = {gather->dest_rows, LB_I32, false};
    }
    Operand op[10];
    if ((rc = resolve(*scope, requests, count, op))) return rc;
    const size_t pool = lb_paged_spec_kv_pages_numel(&spec);
    if ((rc = require_exact_len("Q", op[0].numel, lb_paged_spec_query_numel(&spec)))) return rc;
    if ((rc = require_exact_len("K_pages", op[1].numel, pool))) return rc;
    if ((rc = require_exact_len("V_pages", op[2].numel, pool))) return rc;
    if ((rc = require_exact_len("page_indptr", op[3].numel, spec.batch_size + 1))) return rc;
    if (op[4].numel < spec.batch_size)
        return fail(LB_PAGE_INDICES_TOO_SHORT, nullptr, (int64_t)spec.batch_size,
                    (int64_t)op[4].numel);
    if (op[4].numel > 0x7fffffffu)
        return fail(LB_ENQUEUE_LENGTH_MISMATCH, "page_indices", 0x7fffffff, (int64_t)op[4].numel);
    if ((rc = require_exact_len("last_page_len", op[5].numel, spec.batch_size))) return rc;
    if (split && (rc = require_exact_len("workspace", op[8].numel, c.workspace_numel))) return rc;
    size_t out_numel = lb_paged_spec_query_numel(&spec), lse_numel = lb_paged_spec_lse_numel(&spec);
    if (gather) {
        lse_numel = gather->layout->total_requests * gather->layout->gathered_query_heads;
        out_numel = lse_numel * LB_HEAD_DIM;
    }
    if ((rc = require_exact_len("O", op[6].numel, out_numel))) return rc;
    if ((rc = require_exact_len("LSE", op[7].numel, lse_numel))) return rc;
    if (gather) {
        if ((rc = require_exact_len("dest_rows", op[rows_operand].numel, spec.batch_size)))
            return rc;
        // the bound output and LSE must be this rank's copies of the peer buffers
        if (op[6].ptr != lb_peer_buffer_local(gather->output) ||
            lb_peer_buffer_bytes(gather->output) < out_numel * 2)
            return fail(LB_INVALID_ARGUMENT, "O is not the peer buffer");
        if (op[7].ptr != lb_peer_buffer_local(gather->lse) ||
            lb_peer_buffer_bytes(gather->lse) < lse_numel * 4)
            return fail(LB_INVALID_ARGUMENT, "LSE is not the peer buffer");
    }
    if ((rc = require_alignment("Q", op[0].ptr, 16))) return rc;
    if ((rc = require_alignment("K_pages", op[1].ptr, 16))) return rc;
    if ((rc = require_alignment("V_pages", op[2].ptr, 16))) return rc;
    if ((rc = require_alignment("O", op[6].ptr, 16))) return rc;
    if (split && (rc = require_alignment("workspace", op[8].ptr, 8))) return rc;

    DecodeLaunch launch;
    memset(&launch, 0, sizeof(launch));
    // K/V pools viewed as a rank-3 tensor [64 dims][token row][head half]: dimension 1 walks
    // the max_pages*16 token rows (stride kv_heads*256 B), dimension 2 the 2*kv_heads 128-byte
    // halves of a row (stride 128 B).  One box = 16 token rows of one page x the 2*HC halves of
    // the CTA's heads; in shared memory a head half is 16 consecutive 128-byte rows, which is
    // what makes the swizzled ldmatrix reads conflict-free.
    const uint64_t dims[3] = {64, (uint64_t)spec.max_num_pages * LB_PAGE_SIZE,
                              (uint64_t)spec.num_kv_heads * 2};
    const uint64_t strides[2] = {(uint64_t)spec.num_kv_heads * LB_HEAD_DIM * 2, 128};
    const uint32_t box[3] = {64, 16, c.heads_per_cta * 2};
    int error = driver().encode_tensor_map_3d(plan->device, launch.k_map, op[1].ptr, dims, strides,
                                              box);
    if (!error)
        error = driver().encode_tensor_map_3d(plan->device, launch.v_map, op[2].ptr, dims, strides,
                                              box);
    if (error) return fail(LB_LAUNCH_CONTRACT, "tensor_map", error);
    launch.query = op[0].ptr;
    launch.indptr = (const int32_t *)op[3].ptr;
    launch.indices = (const int32_t *)op[4].ptr;
    launch.last = (const int32_t *)op[5].ptr;
    launch.output = op[6].ptr;
    launch.lse = (float *)op[7].ptr;
    launch.workspace = split ? (float *)op[8].ptr : nullptr;
    launch.status = plan->status;
    launch.batch = (int32_t)spec.batch_size;
    launch.max_pages = (int32_t)spec.max_num_pages;
    launch.qh = (int32_t)spec.num_query_heads;
    launch.kvh = (int32_t)spec.num_kv_heads;
    launch.indices_len = (int32_t)op[4].numel;
    launch.indices_min = plan->indices_capacity ? 0 : launch.indices_len;
    launch.heads_per_cta = (int32_t)c.heads_per_cta;
    launch.pages_per_stage = (int32_t)c.pages_per_stage;
    launch.q_tiles = (int32_t)c.q_tiles;
    launch.q_blocks = (int32_t)c.q_blocks;
    launch.partitions = (int32_t)c.partitions;
    launch.stages = (int32_t)c.stages;
    launch.cluster = c.algorithm == LB_DECODE_CLUSTER_SPLIT ? 1 : 0;
    launch.producer_warps = (int32_t)c.producer_warps;
    launch.merge_four_warps = (int32_t)c.merge_four_warps;
    launch.scale_log2 = spec.softmax_scale * kLog2E;
    launch.grid = c.grid;
    launch.block = c.block;
    launch.shared_bytes = c.shared_bytes;
    launch.wait_cycles = plan->wait_cycles;
    launch.workspace_numel = split ? (long long)op[8].numel : 0;
    launch.test_skip_page = plan->test_skip_page;
    PeerOut peer;
    PeerSignal signal;
    memset(&peer, 0, sizeof(peer));
    memset(&signal, 0, sizeof(signal));
    if (gather) {
        peer.out = peer_buffer_table(gather->output);
        peer.lse = reinterpret_cast<float *const *>(peer_buffer_table(gather->lse));
        peer.dest_rows = (const int32_t *)op[rows_operand].ptr;
        peer.world = lb_peer_group_world(gather->group);
        peer.gathered_qh = (int32_t)gather->layout->gathered_query_heads;
        peer.head_offset = (int32_t)gather->layout->head_offset;
        signal = peer_signal_of(gather->group,
                                plan->wait_cycles ? plan->wait_cycles : default_wait_cycles());
        signal.status = plan->status; // reported by lb_decode_provider_device_status as 2
        signal.defer = gather->layout->defer_wait ? 1 : 0;
    }
    // rows leave from the kernel that finishes them; the command's last kernel signals
    if (c.algorithm != LB_DECODE_SPLIT_K || c.merged_in_kernel) launch.peer = peer;
    if (!merge_command) launch.signal = signal;
    if (c.merged_in_kernel) launch.counters = scope->queue->sync_words;
    void *stream = scope->queue->stream;
    if ((rc = submit_launch(*scope, [&]() {
             return balanced ? launch_balanced_decode(launch, stream)
                             : launch_paged_decode(launch, stream);
         })))
        return rc;
    if (!merge_command) return LB_OK;

    // second command: workspace is now a read operand (decode.rs:1374-1388)
    OperandRequest merge_requests[3] = {
        {lb_handle_read(args->workspace), LB_F32, false},
        {args->output, LB_BF16, true},
        {args->lse, LB_F32, true},
    };
    Operand merge_op[3];
    if ((rc = require_command_capacity(*scope, 1))) return rc;
    if ((rc = resolve(*scope, merge_requests, 3, merge_op))) return rc;
    if (balanced) {
        launch.signal = signal;
        return submit_launch(*scope, [&]() {
            return launch_balanced_merge(launch, c.merge_grid, c.merge_block, stream);
        });
    }
    MergeLaunch merge;
    memset(&merge, 0, sizeof(merge));
    merge.peer = peer;
    merge.signal = signal;
    merge.workspace_numel = launch.workspace_numel;
    merge.status = plan->status;
    merge.workspace = (const float *)merge_op[0].ptr;
    merge.output = merge_op[1].ptr;
    merge.lse = (float *)merge_op[2].ptr;
    merge.indptr = launch.indptr;
    merge.last = launch.last;
    merge.batch = launch.batch;
    merge.qh = launch.qh;
    merge.partitions = launch.partitions;
    merge.indices_len = launch.indices_len;
    merge.indices_min = launch.indices_min;
    merge.grid = c.merge_grid;
    merge.block = c.merge_block;
    return submit_launch(*scope, [&]() { return launch_split_merge(merge, stream); });
}

} // namespace

// ---- state merge -----------------------------------------------------------------------------------

lb_status lb_state_merge_plan_create(const lb_decode_provider *provider, size_t rows,
                                     size_t partitions, lb_state_merge_plan **out) {
    if (!provider || !out) return fail(LB_INVALID_ARGUMENT, "provider");
    *out = nullptr;
    if (rows == 0 || partitions == 0) return fail(LB_ZERO_DIMENSION);
    if (partitions > 65535)
        return fail(LB_INVALID_PARTITION_COUNT, nullptr, (int64_t)partitions, 65535);
    if (rows > 0x7fffffffu) return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)rows);
    size_t numel;
    if (__builtin_mul_overflow(rows, partitions, &numel) ||
        __builtin_mul_overflow(numel, (size_t)LB_PARTIAL_STATE_WIDTH, &numel) ||
        numel > SIZE_MAX / sizeof(float))
        return fail(LB_ELEMENT_COUNT_OVERFLOW);
    lb_state_merge_plan *plan = new lb_state_merge_plan();
    plan->rows = rows;
    plan->partitions = partitions;
    plan->device = provider->device;
    *out = plan;
    return LB_OK;
}

void lb_state_merge_plan_destroy(lb_state_merge_plan *plan) { delete plan; }

lb_status lb_state_merge_enqueue(const lb_state_merge_plan *plan, lb_scope *scope,
                                 const lb_state_merge_args *args) {
    if (!plan || !scope || !args) return fail(LB_INVALID_ARGUMENT, "plan");
    if (scope->queue->device != plan->device)
        return fail(LB_BUFFER_CONTEXT_MISMATCH, nullptr, plan->device, scope->queue->device);
    lb_status rc = require_command_capacity(*scope, 1);
    if (rc) return rc;
    OperandRequest requests[3] = {
        {args->states, LB_F32, false}, {args->output, LB_BF16, true}, {args->lse, LB_F32, true}};
    Operand op[3];
    if ((rc = resolve(*scope, requests, 3, op))) return rc;
    if ((rc = require_exact_len("states", op[0].numel,
                                plan->rows * plan->partitions * LB_PARTIAL_STATE_WIDTH)))
        return rc;
    if ((rc = require_exact_len("O", op[1].numel, plan->rows * LB_HEAD_DIM))) return rc;
    if ((rc = require_exact_len("LSE", op[2].numel, plan->rows))) return rc;
    if ((rc = require_alignment("states", op[0].ptr, 8))) return rc;
    if ((rc = require_alignment("O", op[1].ptr, 8))) return rc;
    MergeLaunch merge;
    memset(&merge, 0, sizeof(merge));
    merge.workspace_numel = (long long)op[0].numel;
    merge.workspace = (const float *)op[0].ptr;
    merge.output = op[1].ptr;
    merge.lse = (float *)op[2].ptr;
    merge.indptr = nullptr; // no request metadata: every row is merged
    merge.last = nullptr;
    merge.batch = (int32_t)plan->rows;
    merge.qh = 1;
    merge.partitions = (int32_t)plan->partitions;
    merge.indices_len = 0;
    merge.indices_min = 0;
    merge.grid = (uint32_t)((plan->rows + 3) / 4);
    merge.block = 128;
    void *stream = scope->queue->stream;
    return submit_launch(*scope, [&]() { return launch_split_merge(merge, stream); });
}

// ---- RoPE + append ---------------------------------------------------------------------------------

lb_status lb_rope_provider_load(int device, lb_rope_provider **out) {
    if (!out) return fail(LB_INVALID_ARGUMENT, "out");
    *out = nullptr;
    int sm_count = 0;
    size_t smem = 0;
    lb_status rc = load_device(device, &sm_count, &smem);
    if (rc) return rc;
    // inverse frequencies exactly as the CPU reference computes them
    // (crates/loom-infer/src/rope/mod.rs:148-149): powf(theta, -(2*pair/rotary_dim)) / scale
    float inverse_frequency[64];
    for (int pair = 0; pair < 64; ++pair) {
        const float exponent = 2.0f * (float)pair / 128.0f;
        inverse_frequency[pair] = powf(10000.0f, -exponent) / 1.0f;
    }
    const size_t hash_bytes = 2 * lb_append_extended_max_tokens() * sizeof(int);
    int32_t *status = nullptr;
    int fused_ctas = 8; // (what the fake driver's provider assumes)
    const int error = driver().configure(device, [&]() -> int {
        int e = configure_append_kernels(hash_bytes, inverse_frequency);
        if (e) return e;
        if ((e = cudaMalloc((void **)&status, 64))) return e;
        if ((e = cudaMemset(status, 0, 64))) return e;
        return append_fused_ctas_per_sm(&fused_ctas, kFusedHashBytes);
    });
    if (error) return fail(LB_DRIVER, "provider_load", error);
    lb_rope_provider *provider = new lb_rope_provider();
    provider->fused_ctas_per_sm = fused_ctas > 0 ? fused_ctas : 1;
    provider->status = status;
    provider->device = device;
    provider->sm_count = sm_count;
    provider->smem_optin = smem;
    *out = provider;
    return LB_OK;
}

void lb_rope_provider_destroy(lb_rope_provider *provider) {
    if (!provider) return;
    if (provider->status) {
        int32_t *status = provider->status;
        driver().configure(provider->device, [&]() -> int { return cudaFree(status); });
    }
    delete provider;
}

lb_status lb_rope_provider_device_status(const lb_rope_provider *provider, int32_t *status) {
    if (!provider || !status) return fail(LB_INVALID_ARGUMENT, "provider");
    *status = 0;
    if (!provider->status) return LB_OK;
    const int error = driver().configure(provider->device, [&]() -> int {
        int e = cudaMemcpy(status, provider->status, sizeof(int32_t), cudaMemcpyDeviceToHost);
        if (e) return e;
        return cudaMemset(provider->status, 0, sizeof(int32_t));
    });
    if (error) return fail(LB_DRIVER, "device_status", error);
    return LB_OK;
}

static lb_status make_append_plan(const lb_rope_provider *provider, const lb_paged_spec &spec,
                                  bool explicit_tokens, size_t tokens, bool extended,
                                  lb_rope_append_plan **out) {
    // state count checks of plan_bf16_paged_append{,_tokens}, rope/mod.rs:628-682
    size_t heads, states;
    if (__builtin_add_overflow(spec.num_query_heads, spec.num_kv_heads, &heads) ||
        __builtin_mul_overflow(tokens, heads, &states))
        return fail(LB_STATE_COUNT_OVERFLOW);
    if (states > 0xffffffffu) return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)states);
    if (tokens > lb_append_extended_max_tokens())
        return fail(LB_UNSUPPORTED_APPEND_TOKEN_COUNT, nullptr,
                    (int64_t)lb_append_extended_max_tokens(), (int64_t)tokens);
    if (spec.max_num_pages > (size_t)0x7fffffff / LB_PAGE_SIZE)
        return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)spec.max_num_pages);
    lb_rope_append_plan *plan = new lb_rope_append_plan();
    plan->spec = spec;
    plan->explicit_tokens = explicit_tokens;
    plan->tokens = tokens;
    plan->device = provider->device;
    plan->status = provider->status;
    uint32_t hash_slots = 128;
    while (hash_slots < 2 * tokens) hash_slots *= 2;
    plan->hash_slots = hash_slots;
    plan->shared_bytes = hash_slots * (uint32_t)sizeof(int);
    // one CTA per token up to two CTAs per SM: every CTA validates the whole call, so more CTAs
    // buy parallel rotation at the price of repeated validation; a CTA never owns more tokens
    // than the kernel's per-CTA token list holds
    plan->block = (uint32_t)append_block_threads();
    const uint32_t cap = 2u * (uint32_t)(provider->sm_count ? provider->sm_count : 148);
    const uint32_t per_cta = (uint32_t)append_max_tokens_per_cta();
    const uint32_t floor = (uint32_t)((tokens + per_cta - 1) / per_cta);
    plan->grid = tokens < cap ? (uint32_t)tokens : (cap > floor ? cap : floor);
    if (extended) {
        // one validation CTA for the tokens plus one scanner per 8192 pages of the pool
        plan->extended = true;
        const size_t scanners = (spec.max_num_pages + 8191) / 8192;
        plan->validate_grid = (uint32_t)(1 + (scanners > 31 ? 31 : scanners));
        plan->workspace_numel = (size_t)append_workspace_numel(tokens);
        // One command is possible when the call is small enough for every CTA of the grid to be
        // resident at once (the token CTAs wait for the validators inside the kernel): a hash set of at most
        // kFusedHashBytes, validators of a quarter of the threads (so four times as many
        // scanners), one token CTA per token up to what the device holds.
        const size_t validators = 1 + (4 * scanners > 31 ? 31 : 4 * scanners);
        const size_t resident =
            (size_t)provider->fused_ctas_per_sm * (size_t)(provider->sm_count ? provider->sm_count : 148);
        if (plan->shared_bytes <= kFusedHashBytes && resident > validators + 1) {
            // (a token CTA holds two tokens ahead of the verdict: half as many CTAs as tokens
            // when the call is larger than the device holds)
            const size_t room = resident - validators;
            const size_t token_ctas = tokens <= room ? tokens : ((tokens + 1) / 2 <= room ? (tokens + 1) / 2 : room);
            plan->fused_possible = true; // (chosen by the one_command option only)
            plan->fused_validators = (uint32_t)validators;
            plan->fused_grid = (uint32_t)(validators + token_ctas);
        }
    }
    *out = plan;
    return LB_OK;
}

static lb_status apply_append_options(const lb_rope_append_options *options,
                                      lb_rope_append_plan **plan) {
    if (!options) return LB_OK;
    if (options->indices_capacity > 1) {
        delete *plan;
        *plan = nullptr;
        return fail(LB_LAUNCH_CONTRACT, "indices_capacity", options->indices_capacity);
    }
    if (options->one_command > 1 || (options->one_command == 1 && !(*plan)->fused_possible)) {
        delete *plan;
        *plan = nullptr;
        return fail(LB_LAUNCH_CONTRACT, "one_command", options->one_command);
    }
    (*plan)->indices_capacity = options->indices_capacity == 1;
    (*plan)->fused = options->one_command == 1;
    return LB_OK;
}

lb_status lb_rope_append_plan_create(const lb_rope_provider *provider, const lb_paged_spec *spec,
                                     lb_rope_append_plan **out) {
    return lb_rope_append_plan_create_with(provider, spec, nullptr, out);
}

lb_status lb_rope_append_plan_create_with(const lb_rope_provider *provider,
                                          const lb_paged_spec *spec,
                                          const lb_rope_append_options *options,
                                          lb_rope_append_plan **out) {
    if (!provider || !spec || !out) return fail(LB_INVALID_ARGUMENT, "provider");
    *out = nullptr;
    lb_paged_spec checked;
    lb_status rc = lb_paged_spec_new(spec->batch_size, spec->max_num_pages, spec->num_query_heads,
                                     spec->num_kv_heads, LB_HEAD_DIM, LB_PAGE_SIZE, &checked);
    if (rc) return rc;
    if ((rc = make_append_plan(provider, checked, false, checked.batch_size, false, out)))
        return rc;
    return apply_append_options(options, out);
}

lb_status lb_rope_append_tokens_plan_create(const lb_rope_provider *provider,
                                            const lb_append_tokens_spec *spec,
                                            lb_rope_append_plan **out) {
    return lb_rope_append_tokens_plan_create_with(provider, spec, nullptr, out);
}

lb_status lb_rope_append_tokens_plan_create_with(const lb_rope_provider *provider,
                                                 const lb_append_tokens_spec *spec,
                                                 const lb_rope_append_options *options,
                                                 lb_rope_append_plan **out) {
    if (!provider || !spec || !out) return fail(LB_INVALID_ARGUMENT, "provider");
    *out = nullptr;
    lb_append_tokens_spec checked;
    lb_status rc =
        spec->max_tokens == 0
            ? lb_append_tokens_spec_new_extended(spec->tokens, spec->paged.batch_size,
                                                 spec->paged.max_num_pages,
                                                 spec->paged.num_query_heads,
                                                 spec->paged.num_kv_heads, LB_HEAD_DIM,
                                                 LB_PAGE_SIZE, &checked)
            : lb_append_tokens_spec_new(spec->tokens, spec->paged.batch_size,
                                        spec->paged.max_num_pages, spec->paged.num_query_heads,
                                        spec->paged.num_kv_heads, LB_HEAD_DIM, LB_PAGE_SIZE,
                                        &checked);
    if (rc) return rc;
    if ((rc = make_append_plan(provider, checked.paged, true, checked.tokens,
                               checked.max_tokens == 0, out)))
        return rc;
    return apply_append_options(options, out);
}

void lb_rope_append_plan_destroy(lb_rope_append_plan *plan) { delete plan; }

lb_status lb_rope_append_plan_info_get(const lb_rope_append_plan *plan,
                                       lb_rope_append_plan_info *info) {
    if (!plan || !info) return fail(LB_INVALID_ARGUMENT, "plan");
    info->explicit_tokens = plan->explicit_tokens ? 1 : 0;
    info->tokens = (uint32_t)plan->tokens;
    info->grid = plan->grid;
    info->block = plan->block;
    info->shared_bytes = plan->shared_bytes;
    info->commands = plan->extended && !plan->fused ? 2 : 1;
    info->workspace_numel = plan->workspace_numel;
    return LB_OK;
}

lb_status lb_rope_append_enqueue(const lb_rope_append_plan *plan, lb_scope *scope,
                                 const lb_rope_append_args *args) {
    if (!plan || !scope || !args) return fail(LB_INVALID_ARGUMENT, "plan");
    const lb_paged_spec &spec = plan->spec;
    if (scope->queue->device != plan->device)
        return fail(LB_BUFFER_CONTEXT_MISMATCH, nullptr, plan->device, scope->queue->device);
    // both commands of an extended plan must fit before anything is launched
    lb_status rc = require_command_capacity(*scope, plan->extended && !plan->fused ? 2 : 1);
    if (rc) return rc;

    Operand op[11];
    const size_t tokens = plan->tokens;
    const size_t q_numel = tokens * spec.num_query_heads * LB_HEAD_DIM;
    const size_t kv_numel = tokens * spec.num_kv_heads * LB_HEAD_DIM;
    const size_t pool = lb_paged_spec_kv_pages_numel(&spec);
    int indptr_i, indices_i, last_i, qout_i;
    if (plan->explicit_tokens) {
        OperandRequest requests[11] = {
            {args->query, LB_BF16, false},        {args->key, LB_BF16, false},
            {args->value, LB_BF16, false},        {args->batch_indices, LB_I32, false},
            {args->positions, LB_I32, false},     {args->page_indptr, LB_I32, false},
            {args->page_indices, LB_I32, false},  {args->last_page_len, LB_I32, false},
            {args->query_output, LB_BF16, true},  {args->key_pages, LB_BF16, true},
            {args->value_pages, LB_BF16, true},
        };
        if ((rc = resolve(*scope, requests, 11, op))) return rc;
        indptr_i = 5; indices_i = 6; last_i = 7; qout_i = 8;
    } else {
        OperandRequest requests[9] = {
            {args->query, LB_BF16, false},        {args->key, LB_BF16, false},
            {args->value, LB_BF16, false},        {args->page_indptr, LB_I32, false},
            {args->page_indices, LB_I32, false},  {args->last_page_len, LB_I32, false},
            {args->query_output, LB_BF16, true},  {args->key_pages, LB_BF16, true},
            {args->value_pages, LB_BF16, true},
        };
        if ((rc = resolve(*scope, requests, 9, op))) return rc;
        indptr_i = 3; indices_i = 4; last_i = 5; qout_i = 6;
    }
    if ((rc = require_exact_len("query", op[0].numel, q_numel))) return rc;
    if ((rc = require_exact_len("key", op[1].numel, kv_numel))) return rc;
    if ((rc = require_exact_len("value", op[2].numel, kv_numel))) return rc;
    if (plan->explicit_tokens) {
        if ((rc = require_exact_len("batch_indices", op[3].numel, tokens))) return rc;
        if ((rc = require_exact_len("positions", op[4].numel, tokens))) return rc;
    }
    if ((rc = require_exact_len("page_indptr", op[indptr_i].numel, spec.batch_size + 1))) return rc;
    if (op[indices_i].numel < spec.batch_size)
        return fail(LB_PAGE_INDICES_TOO_SHORT, nullptr, (int64_t)spec.batch_size,
                    (int64_t)op[indices_i].numel);
    if (op[indices_i].numel > 0x7fffffffu)
        return fail(LB_ENQUEUE_LENGTH_MISMATCH, "page_indices", 0x7fffffff,
                    (int64_t)op[indices_i].numel);
    if ((rc = require_exact_len("last_page_len", op[last_i].numel, spec.batch_size))) return rc;
    if ((rc = require_exact_len("query_output", op[qout_i].numel, q_numel))) return rc;
    if ((rc = require_exact_len("key_pages", op[qout_i + 1].numel, pool))) return rc;
    if ((rc = require_exact_len("value_pages", op[qout_i + 2].numel, pool))) return rc;
    if ((rc = require_alignment("query", op[0].ptr, 16))) return rc;
    if ((rc = require_alignment("key", op[1].ptr, 16))) return rc;
    if ((rc = require_alignment("value", op[2].ptr, 16))) return rc;
    if ((rc = require_alignment("query_output", op[qout_i].ptr, 16))) return rc;
    if ((rc = require_alignment("key_pages", op[qout_i + 1].ptr, 16))) return rc;
    if ((rc = require_alignment("value_pages", op[qout_i + 2].ptr, 16))) return rc;

    AppendLaunch launch;
    memset(&launch, 0, sizeof(launch));
    launch.query = op[0].ptr;
    launch.key = op[1].ptr;
    launch.value = op[2].ptr;
    launch.batch_indices = plan->explicit_tokens ? (const int32_t *)op[3].ptr : nullptr;
    launch.positions = plan->explicit_tokens ? (const int32_t *)op[4].ptr : nullptr;
    launch.indptr = (const int32_t *)op[indptr_i].ptr;
    launch.indices = (const int32_t *)op[indices_i].ptr;
    launch.last = (const int32_t *)op[last_i].ptr;
    launch.query_output = op[qout_i].ptr;
    launch.key_pages = op[qout_i + 1].ptr;
    launch.value_pages = op[qout_i + 2].ptr;
    launch.tokens = (int32_t)tokens;
    launch.batch = (int32_t)spec.batch_size;
    launch.max_pages = (int32_t)spec.max_num_pages;
    launch.qh = (int32_t)spec.num_query_heads;
    launch.kvh = (int32_t)spec.num_kv_heads;
    launch.indices_len = (int32_t)op[indices_i].numel;
    launch.indices_min = plan->indices_capacity ? 0 : launch.indices_len;
    launch.hash_slots = (int32_t)plan->hash_slots;
    launch.grid = plan->grid;
    launch.block = plan->block;
    launch.shared_bytes = plan->shared_bytes;
    launch.status = plan->status;
    void *stream = scope->queue->stream;
    if (!plan->extended)
        return submit_launch(*scope, [&]() { return launch_rope_append(launch, stream); });

    // extended: command 1 validates into the workspace, command 2 reads it (write, then read,
    // like the split-K workspace)
    OperandRequest ws_request[1] = {{args->workspace, LB_I32, true}};
    Operand ws[1];
    if ((rc = resolve(*scope, ws_request, 1, ws))) return rc;
    if ((rc = require_exact_len("workspace", ws[0].numel, plan->workspace_numel))) return rc;
    launch.workspace = (int32_t *)ws[0].ptr;
    launch.workspace_numel = (int32_t)ws[0].numel;
    launch.validate_grid = plan->validate_grid;
    if (plan->fused) {
        launch.grid = plan->fused_grid;
        launch.validate_grid = plan->fused_validators;
        launch.words = scope->queue->sync_words;
        return submit_launch(*scope, [&]() { return launch_append_fused(launch, stream); });
    }
    if ((rc = submit_launch(*scope, [&]() { return launch_append_validate(launch, stream); })))
        return rc;
    if ((rc = require_command_capacity(*scope, 1))) return rc;
    return submit_launch(*scope, [&]() { return launch_append_scatter(launch, stream); });
}

// ---- stand-alone RoPE ------------------------------------------------------------------------------

lb_status lb_rope_pos_ids_plan_create(const lb_rope_provider *provider,
                                      const lb_rope_pos_ids_spec *spec,
                                      lb_rope_pos_ids_plan **out) {
    if (!provider || !spec || !out) return fail(LB_INVALID_ARGUMENT, "provider");
    *out = nullptr;
    lb_rope_pos_ids_spec checked;
    lb_status rc = lb_rope_pos_ids_spec_new(spec->tokens, spec->query_heads, spec->key_heads,
                                            spec->head_dim, spec->rotary_dim, spec->rope_scale,
                                            spec->rope_theta, &checked);
    if (rc) return rc;
    // plan_bf16_pos_ids, crates/loom-infer-cuda/src/rope/mod.rs:592-626
    if (checked.head_dim != LB_HEAD_DIM)
        return fail(LB_UNSUPPORTED_HEAD_DIMENSION, nullptr, LB_HEAD_DIM, (int64_t)checked.head_dim);
    if (checked.rotary_dim != LB_HEAD_DIM)
        return fail(LB_UNSUPPORTED_ROTARY_DIMENSION, nullptr, LB_HEAD_DIM,
                    (int64_t)checked.rotary_dim);
    size_t heads, states;
    if (__builtin_add_overflow(checked.query_heads, checked.key_heads, &heads) ||
        __builtin_mul_overflow(checked.tokens, heads, &states))
        return fail(LB_STATE_COUNT_OVERFLOW);
    if (states > 0xffffffffu) return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)states);
    lb_rope_pos_ids_plan *plan = new lb_rope_pos_ids_plan();
    plan->spec = checked;
    plan->device = provider->device;
    const size_t cap = 8u * (size_t)(provider->sm_count ? provider->sm_count : 148);
    plan->grid = (uint32_t)(checked.tokens < cap ? checked.tokens : cap);
    // the CPU reference's expression (crates/loom-infer/src/rope/mod.rs:148-149), evaluated in
    // F32 on the host so that the device angle is bit-identical to the reference's
    for (int pair = 0; pair < 64; ++pair) {
        const float exponent = 2.0f * (float)pair / (float)checked.rotary_dim;
        plan->inverse_frequency[pair] = powf(checked.rope_theta, -exponent) / checked.rope_scale;
    }
    *out = plan;
    return LB_OK;
}

void lb_rope_pos_ids_plan_destroy(lb_rope_pos_ids_plan *plan) { delete plan; }

lb_status lb_rope_pos_ids_enqueue(const lb_rope_pos_ids_plan *plan, lb_scope *scope,
                                  const lb_rope_pos_ids_args *args) {
    if (!plan || !scope || !args) return fail(LB_INVALID_ARGUMENT, "plan");
    const lb_rope_pos_ids_spec &spec = plan->spec;
    if (scope->queue->device != plan->device)
        return fail(LB_BUFFER_CONTEXT_MISMATCH, nullptr, plan->device, scope->queue->device);
    lb_status rc = require_command_capacity(*scope, 1);
    if (rc) return rc;
    OperandRequest requests[5] = {
        {args->query, LB_BF16, false},       {args->key, LB_BF16, false},
        {args->position_ids, LB_I32, false}, {args->query_output, LB_BF16, true},
        {args->key_output, LB_BF16, true},
    };
    Operand op[5];
    if ((rc = resolve(*scope, requests, 5, op))) return rc;
    const size_t q_numel = lb_rope_pos_ids_spec_query_numel(&spec);
    const size_t k_numel = lb_rope_pos_ids_spec_key_numel(&spec);
    if ((rc = require_exact_len("query", op[0].numel, q_numel))) return rc;
    if ((rc = require_exact_len("key", op[1].numel, k_numel))) return rc;
    if ((rc = require_exact_len("position_ids", op[2].numel, spec.tokens))) return rc;
    if ((rc = require_exact_len("query_output", op[3].numel, q_numel))) return rc;
    if ((rc = require_exact_len("key_output", op[4].numel, k_numel))) return rc;
    if ((rc = require_alignment("query", op[0].ptr, 16))) return rc;
    if ((rc = require_alignment("key", op[1].ptr, 16))) return rc;
    if ((rc = require_alignment("query_output", op[3].ptr, 16))) return rc;
    if ((rc = require_alignment("key_output", op[4].ptr, 16))) return rc;
    RopeLaunch launch;
    launch.query = op[0].ptr;
    launch.key = op[1].ptr;
    launch.position_ids = (const int32_t *)op[2].ptr;
    launch.query_output = op[3].ptr;
    launch.key_output = op[4].ptr;
    launch.tokens = (int32_t)spec.tokens;
    launch.qh = (int32_t)spec.query_heads;
    launch.kh = (int32_t)spec.key_heads;
    memcpy(launch.inverse_frequency, plan->inverse_frequency, sizeof(launch.inverse_frequency));
    launch.grid = plan->grid;
    void *stream = scope->queue->stream;
    return submit_launch(*scope, [&]() { return launch_rope_pos_ids(launch, stream); });
}

}
