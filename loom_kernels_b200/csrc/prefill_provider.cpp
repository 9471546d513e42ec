// Paged causal prefill: the validated spec, host-side metadata validation, and the provider with
// its immutable plan and checked enqueue.
//
// Mirrors Bf16PagedPrefillSpec / Bf16PagedPrefillMetadata
// (crates/loom-infer/src/attention/paged_prefill/mod.rs:19-359) and PrefillProvider /
// Bf16PagedPrefillPlan (crates/loom-infer-cuda/src/attention/prefill.rs:2278-2330,2411-2584)
// of the reference.  A plan fixes the launch shape from the spec and the device alone; enqueue
// performs no re-dispatch and has no fallback.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>

#include "kernels.hpp"
#include "runtime.hpp"

using namespace lb;

struct lb_prefill_provider {
    int device = 0, sm_count = 0;
    size_t smem_optin = 0;
    int32_t *status = nullptr; // device word written by a kernel that gave up on a wait
};

struct lb_paged_prefill_plan {
    lb_prefill_spec spec;
    lb_paged_prefill_plan_info info;
    int device = 0;
    int32_t *status = nullptr;
    bool indices_capacity = false;
    long long wait_cycles = 0; // tiled kernel: 0 = the default limit
    int32_t test_lost_copy = 0;
};

namespace {

const float kLog2E = 1.44269504088896340736f;

bool mul_overflow(size_t a, size_t b, size_t *out) { return __builtin_mul_overflow(a, b, out); }

lb_status require_len(const char *buffer, size_t actual, size_t expected) {
    if (actual == expected) return LB_OK;
    return fail(LB_LENGTH_MISMATCH, buffer, (int64_t)expected, (int64_t)actual);
}

lb_status require_exact_len(const char *operand, size_t actual, size_t expected) {
    if (actual == expected) return LB_OK;
    return fail(LB_ENQUEUE_LENGTH_MISMATCH, operand, (int64_t)expected, (int64_t)actual);
}

// The reference requires 4-byte bases (prefill.rs:3015-3029); the vector and TMA accesses of this
// kernel need 16.
lb_status require_alignment(const char *operand, const void *ptr, uint64_t alignment) {
    const uint64_t address = (uint64_t)(uintptr_t)ptr;
    if (address % alignment == 0) return LB_OK;
    return fail(LB_MISALIGNED_BUFFER, operand, (int64_t)address, (int64_t)alignment);
}

// paged_prefill/mod.rs:238-266
lb_status validate_query_indptr(const int32_t *indptr, size_t len, size_t expected_total) {
    if (indptr[0] != 0) return fail(LB_INVALID_INDPTR_START, "qo_indptr", indptr[0]);
    for (size_t request = 0; request + 1 < len; ++request) {
        const int32_t start = indptr[request], end = indptr[request + 1];
        if (end < start)
            return fail(LB_NON_MONOTONIC_INDPTR, "qo_indptr", (int64_t)request, start, end);
        if (end == start) return fail(LB_EMPTY_RAGGED_REQUEST, "qo_indptr", (int64_t)request);
    }
    if (indptr[len - 1] < 0) return fail(LB_ELEMENT_COUNT_OVERFLOW);
    return require_len("qo_indptr", (size_t)indptr[len - 1], expected_total);
}

// Plan-time launch shape.  Inputs are the spec and the device only: neither the query ranges nor
// the page table are known when a plan is made.
//
//   q_tiles (MT)     16-row MMA tiles of packed (token, head-in-group) rows one CTA owns; the
//                    other 8 / MT warp groups take different pages of the same rows.  Few rows
//                    (a short chunk, a decode-like append) want MT = 1: eight pages in flight
//                    per CTA and many CTAs; many rows want MT = 8: every page a CTA loads is
//                    used by 128 rows.
//   tiles            floor(nnz_qo * group / (16 * MT)) + batch: every request adds at most one
//                    partly filled tile.
lb_status choose_prefill(const lb_prefill_spec &spec, uint32_t sm_count, size_t smem_optin,
                         const lb_paged_prefill_options *options,
                         lb_paged_prefill_plan_info *out) {
    const uint32_t sms = sm_count ? sm_count : 148;
    const size_t smem = smem_optin ? smem_optin : 232448;
    const size_t group = spec.num_query_heads / spec.num_kv_heads;
    size_t states;
    // PagedPrefillPlanError::StateCountOutOfRange, prefill.rs:2293-2299
    if (mul_overflow(spec.nnz_qo, spec.num_query_heads, &states))
        return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, INT64_MAX);
    if (states > 0xffffffffu) return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)states);
    const size_t packed_rows = spec.nnz_qo * group; // per KV head, over all requests

    uint32_t q_tiles = options ? options->q_tiles : 0;
    if (q_tiles != 0 && q_tiles != 1 && q_tiles != 2 && q_tiles != 4 && q_tiles != 8)
        return fail(LB_LAUNCH_CONTRACT, "q_tiles", q_tiles);
    if (options && options->indices_capacity > 1)
        return fail(LB_LAUNCH_CONTRACT, "indices_capacity", options->indices_capacity);
    const uint32_t algorithm_option = options ? options->algorithm : 0;
    if (algorithm_option > 2) return fail(LB_LAUNCH_CONTRACT, "algorithm", algorithm_option);
    uint32_t partitions = options ? options->partitions : 0;
    if (partitions > 64) return fail(LB_INVALID_PARTITION_COUNT, nullptr, partitions, 64);
    if (partitions > 1 && algorithm_option == 1)
        return fail(LB_LAUNCH_CONTRACT, "partitions", partitions);
    // Tiled (tcgen05, 128-row tiles) when the call has a whole tile per KV head and either 512
    // packed rows (128 tokens of a 4-head group) with room for a few blocks of KV per request in
    // the pool, or room for 4096 tokens per request (a short chunk over a long cache: the KV
    // range is shared out below).  Shorter calls are latency-bound and take the token-parallel
    // kernel.  (Measured back to back on B200, 32 query / 8 KV heads: 128 queries over 512
    // tokens 13.9 us tiled against 20.3; 64 over 512 13.8 against 11.0; 32 over 8192 31.7
    // against 65.7.)
    const size_t full_tiles = (packed_rows / 128) * spec.num_kv_heads;
    const size_t average_kv = spec.max_num_pages * LB_PAGE_SIZE / spec.batch_size;
    const bool tiled =
        algorithm_option == 2 ||
        (algorithm_option == 0 && q_tiles == 0 &&
         (partitions > 1 ||
          (full_tiles >= 1 && ((packed_rows >= 512 && average_kv >= 256) || average_kv >= 4096))));
    // chunks exist only in the tiled kernel: a count next to a token-parallel tile shape is a
    // contradiction, not something to drop silently
    if (!tiled && partitions > 1) return fail(LB_LAUNCH_CONTRACT, "partitions", partitions);
    if (tiled) {
        const uint32_t shared = (uint32_t)prefill_tiled_shared_bytes();
        if (shared > smem) return fail(LB_LAUNCH_CONTRACT, "shared_memory", shared);
        const size_t tiles = packed_rows / 128 + spec.batch_size;
        uint32_t min_chunk_blocks = 1; // the caller's count is taken literally
        if (partitions == 0) {
            min_chunk_blocks = 16;
            // Two CTAs run per SM.  When the tiles are fewer than half of those slots, the
            // 64-token KV blocks of every tile are shared out to several CTAs -- as many as fit
            // the slots in one wave, never fewer than sixteen blocks (1024 tokens of the average
            // request's room in the pool) per CTA, at most sixteen CTAs -- and a second command
            // merges their states.  Every request has at least one tile per KV head.  The pool's
            // room is an upper bound of the KV lengths a call will bring (an engine's pool is
            // usually its whole cache), so the kernels apply the sixteen-block rule again to the
            // length they meet: a tile too short for two chunks is finished by the first command
            // alone (min_chunk_blocks).
            const size_t slots = 2 * (size_t)sms;
            const size_t request_tiles = spec.batch_size * spec.num_kv_heads;
            const size_t work = full_tiles > request_tiles ? full_tiles : request_tiles;
            size_t wanted = slots / work;
            const size_t room = average_kv / 1024;
            if (wanted > room) wanted = room;
            if (wanted > 16) wanted = 16;
            // a range of fewer than three times sixteen blocks does not pay for the merge
            partitions = wanted > 1 && room >= 3 ? (uint32_t)wanted : 1;
        }
        size_t grid, workspace = 0;
        if (mul_overflow(tiles, spec.num_kv_heads, &grid) || mul_overflow(grid, partitions, &grid) ||
            grid > 0x7fffffffu)
            return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)states);
        if (partitions > 1 && (mul_overflow(states, (size_t)partitions * 130, &workspace) ||
                               workspace > ((size_t)1 << 40)))
            return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)states);
        memset(out, 0, sizeof(*out));
        out->algorithm = LB_PREFILL_TILED;
        out->q_tiles = 8;
        out->pages_per_stage = 4; // blocks of 64 KV tokens
        out->stages = 2;
        out->rows_per_cta = 128;
        out->tiles = (uint32_t)tiles;
        out->grid = (uint32_t)grid;
        out->block = 192;
        out->shared_bytes = shared;
        out->commands = partitions > 1 ? 2 : 1;
        out->partitions = partitions;
        out->merge_grid = partitions > 1 ? (uint32_t)((states + 3) / 4) : 0;
        out->merge_block = partitions > 1 ? 128 : 0;
        out->min_chunk_blocks = min_chunk_blocks;
        out->workspace_numel = workspace;
        return LB_OK;
    }
    if (q_tiles == 0) {
        // the largest tile that still gives every SM two CTAs; short calls take the smallest
        q_tiles = 1;
        for (uint32_t mt = 8; mt > 1; mt /= 2) {
            const size_t ctas = (packed_rows / (16 * mt)) * spec.num_kv_heads;
            if (ctas >= 2 * (size_t)sms) {
                q_tiles = mt;
                break;
            }
        }
    }
    const uint32_t pps = 8 / q_tiles;
    const uint32_t stage_bytes = pps * 8192u;
    // a ring of about 192 KB, at most 8 stages; with several page slots the ring also has to
    // hold the 68 KB of states the slots merge through
    uint32_t stages = (uint32_t)((192u * 1024u) / stage_bytes);
    if (stages > 8) stages = 8;
    if (stages < 2) stages = 2;
    const uint32_t shared = 1024 + stages * stage_bytes + 2 * stages * pps * 8 + 16;
    if (shared > smem) return fail(LB_LAUNCH_CONTRACT, "shared_memory", shared);
    const size_t tiles = packed_rows / (16 * q_tiles) + spec.batch_size;
    size_t grid;
    if (mul_overflow(tiles, spec.num_kv_heads, &grid) || grid > 0x7fffffffu)
        return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)states);
    memset(out, 0, sizeof(*out));
    out->algorithm = LB_PREFILL_TOKEN_PARALLEL;
    out->q_tiles = q_tiles;
    out->pages_per_stage = pps;
    out->stages = stages;
    out->rows_per_cta = 16 * q_tiles;
    out->tiles = (uint32_t)tiles;
    out->grid = (uint32_t)grid;
    out->block = 288;
    out->shared_bytes = shared;
    out->commands = 1;
    out->partitions = 1;
    return LB_OK;
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

} // namespace

extern "C" {

// ---- contract ------------------------------------------------------------------------------------

lb_status lb_prefill_spec_new(size_t batch, size_t nnz_qo, size_t max_pages, size_t qh, size_t kvh,
                              size_t head_dim, size_t page_size, lb_prefill_spec *out) {
    if (!out) return fail(LB_INVALID_ARGUMENT, "out");
    if (batch == 0 || nnz_qo == 0 || max_pages == 0 || qh == 0 || kvh == 0 || head_dim == 0 ||
        page_size == 0)
        return fail(LB_ZERO_DIMENSION);
    if (head_dim != LB_HEAD_DIM)
        return fail(LB_UNSUPPORTED_HEAD_DIMENSION, nullptr, LB_HEAD_DIM, (int64_t)head_dim);
    if (page_size != LB_PAGE_SIZE)
        return fail(LB_UNSUPPORTED_PAGE_SIZE, nullptr, LB_PAGE_SIZE, (int64_t)page_size);
    if (qh % kvh != 0) return fail(LB_INVALID_HEAD_MAPPING, nullptr, (int64_t)qh, (int64_t)kvh);
    if (nnz_qo > (size_t)INT32_MAX) return fail(LB_ELEMENT_COUNT_OVERFLOW);
    size_t t;
    if (batch + 1 < batch || mul_overflow(nnz_qo, qh, &t) || mul_overflow(t, head_dim, &t))
        return fail(LB_ELEMENT_COUNT_OVERFLOW);
    if (mul_overflow(max_pages, page_size, &t) || mul_overflow(t, kvh, &t) ||
        mul_overflow(t, head_dim, &t))
        return fail(LB_ELEMENT_COUNT_OVERFLOW);
    out->batch_size = batch;
    out->nnz_qo = nnz_qo;
    out->max_num_pages = max_pages;
    out->num_query_heads = qh;
    out->num_kv_heads = kvh;
    out->softmax_scale = 1.0f / sqrtf((float)head_dim);
    return LB_OK;
}

size_t lb_prefill_spec_query_numel(const lb_prefill_spec *spec) {
    return spec->nnz_qo * spec->num_query_heads * LB_HEAD_DIM;
}
size_t lb_prefill_spec_kv_pages_numel(const lb_prefill_spec *spec) {
    return spec->max_num_pages * LB_PAGE_SIZE * spec->num_kv_heads * LB_HEAD_DIM;
}
size_t lb_prefill_spec_lse_numel(const lb_prefill_spec *spec) {
    return spec->nnz_qo * spec->num_query_heads;
}

lb_status lb_prefill_spec_validate_metadata(const lb_prefill_spec *spec, const int32_t *qo_indptr,
                                            size_t qo_indptr_len, const int32_t *page_indptr,
                                            size_t page_indptr_len, const int32_t *indices,
                                            size_t indices_len, const int32_t *last,
                                            size_t last_len) {
    if (!spec) return fail(LB_INVALID_ARGUMENT, "spec");
    const size_t batch = spec->batch_size;
    lb_status rc;
    if ((rc = require_len("qo_indptr", qo_indptr_len, batch + 1))) return rc;
    if ((rc = require_len("page_indptr", page_indptr_len, batch + 1))) return rc;
    if ((rc = require_len("last_page_len", last_len, batch))) return rc;
    if ((rc = validate_query_indptr(qo_indptr, qo_indptr_len, spec->nnz_qo))) return rc;
    if (page_indptr[0] != 0) return fail(LB_INVALID_PAGE_INDPTR_START, nullptr, page_indptr[0]);
    for (size_t request = 0; request < batch; ++request) {
        const int32_t start = page_indptr[request], end = page_indptr[request + 1];
        if (end < start)
            return fail(LB_NON_MONOTONIC_PAGE_INDPTR, nullptr, (int64_t)request, start, end);
        if (end == start) return fail(LB_EMPTY_PAGED_REQUEST, nullptr, (int64_t)request);
        const int32_t tail = last[request];
        if (tail < 1 || tail > (int32_t)LB_PAGE_SIZE)
            return fail(LB_INVALID_LAST_PAGE_LENGTH, nullptr, (int64_t)request, tail, LB_PAGE_SIZE);
        const size_t qo_len = (size_t)(qo_indptr[request + 1] - qo_indptr[request]);
        const size_t kv_len = (size_t)(end - start - 1) * LB_PAGE_SIZE + (size_t)tail;
        if (qo_len > kv_len)
            return fail(LB_RAGGED_QUERY_LONGER_THAN_KV, nullptr, (int64_t)request, (int64_t)qo_len,
                        (int64_t)kv_len);
    }
    if (page_indptr[batch] < 0) return fail(LB_ELEMENT_COUNT_OVERFLOW);
    if ((rc = require_len("page_indices", indices_len, (size_t)page_indptr[batch]))) return rc;
    for (size_t position = 0; position < indices_len; ++position) {
        const int32_t index = indices[position];
        if (index < 0 || (size_t)index >= spec->max_num_pages)
            return fail(LB_PAGE_INDEX_OUT_OF_RANGE, nullptr, (int64_t)position, index,
                        (int64_t)spec->max_num_pages);
    }
    return LB_OK;
}

int lb_prefill_metadata_causal_kv_end(const lb_prefill_spec *spec, const int32_t *qo_indptr,
                                      const int32_t *page_indptr, const int32_t *last,
                                      size_t request, size_t query_index, size_t *kv_end) {
    if (!spec || request >= spec->batch_size) return 0;
    const size_t qo_len = (size_t)(qo_indptr[request + 1] - qo_indptr[request]);
    if (query_index >= qo_len) return 0;
    const size_t pages = (size_t)(page_indptr[request + 1] - page_indptr[request]);
    const size_t kv_len = (pages - 1) * LB_PAGE_SIZE + (size_t)last[request];
    if (kv_end) *kv_end = kv_len - qo_len + query_index + 1;
    return 1;
}

// ---- provider ------------------------------------------------------------------------------------

lb_status lb_prefill_provider_load(int device, lb_prefill_provider **out) {
    if (!out) return fail(LB_INVALID_ARGUMENT, "out");
    *out = nullptr;
    int sm_count = 0;
    size_t smem = 0;
    lb_status rc = load_device(device, &sm_count, &smem);
    if (rc) return rc;
    int32_t *status = nullptr;
    const int error = driver().configure(device, [&]() -> int {
        int e = configure_prefill_kernels(smem);
        if (e) return e;
        if ((e = configure_prefill_tiled_kernel(smem))) return e;
        if ((e = cudaMalloc((void **)&status, 64))) return e;
        return cudaMemset(status, 0, 64);
    });
    if (error) return fail(LB_DRIVER, "provider_load", error);
    lb_prefill_provider *provider = new lb_prefill_provider();
    provider->device = device;
    provider->sm_count = sm_count;
    provider->smem_optin = smem;
    provider->status = status;
    *out = provider;
    return LB_OK;
}

void lb_prefill_provider_destroy(lb_prefill_provider *provider) {
    if (!provider) return;
    if (provider->status) {
        int32_t *status = provider->status;
        driver().configure(provider->device, [&]() -> int { return cudaFree(status); });
    }
    delete provider;
}

lb_status lb_prefill_provider_device_status(const lb_prefill_provider *provider, int32_t *status) {
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

lb_status lb_paged_prefill_choose(const lb_prefill_spec *spec, uint32_t sm_count,
                                  const lb_paged_prefill_options *options,
                                  lb_paged_prefill_plan_info *info) {
    if (!spec || !info) return fail(LB_INVALID_ARGUMENT, "spec");
    lb_prefill_spec checked;
    lb_status rc = lb_prefill_spec_new(spec->batch_size, spec->nnz_qo, spec->max_num_pages,
                                       spec->num_query_heads, spec->num_kv_heads, LB_HEAD_DIM,
                                       LB_PAGE_SIZE, &checked);
    if (rc) return rc;
    return choose_prefill(checked, sm_count, 0, options, info);
}

lb_status lb_paged_prefill_plan_create(const lb_prefill_provider *provider,
                                       const lb_prefill_spec *spec,
                                       const lb_paged_prefill_options *options,
                                       lb_paged_prefill_plan **out) {
    if (!provider || !spec || !out) return fail(LB_INVALID_ARGUMENT, "provider");
    *out = nullptr;
    lb_prefill_spec checked;
    lb_status rc = lb_prefill_spec_new(spec->batch_size, spec->nnz_qo, spec->max_num_pages,
                                       spec->num_query_heads, spec->num_kv_heads, LB_HEAD_DIM,
                                       LB_PAGE_SIZE, &checked);
    if (rc) return rc;
    if (spec->max_num_pages > (size_t)0x7fffffff / LB_PAGE_SIZE ||
        spec->num_kv_heads > 0x7fffffffu / LB_HEAD_DIM || spec->batch_size > 0x7ffffffeu)
        return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)spec->max_num_pages);
    lb_paged_prefill_plan_info info;
    if ((rc = choose_prefill(checked, (uint32_t)provider->sm_count, provider->smem_optin, options,
                             &info)))
        return rc;
    lb_paged_prefill_plan *plan = new lb_paged_prefill_plan();
    plan->spec = checked;
    plan->info = info;
    plan->device = provider->device;
    plan->status = provider->status;
    plan->indices_capacity = options && options->indices_capacity == 1;
    if (options && options->wait_limit_us) {
        int khz = 0;
        driver().device_clock_khz(provider->device, &khz);
        plan->wait_cycles = (long long)options->wait_limit_us * (khz > 0 ? khz : 1965000) / 1000;
    }
    plan->test_lost_copy = options && options->test_lost_copy ? 1 : 0;
    *out = plan;
    return LB_OK;
}

void lb_paged_prefill_plan_destroy(lb_paged_prefill_plan *plan) { delete plan; }

lb_status lb_paged_prefill_plan_info_get(const lb_paged_prefill_plan *plan, lb_prefill_spec *spec,
                                         lb_paged_prefill_plan_info *info) {
    if (!plan) return fail(LB_INVALID_ARGUMENT, "plan");
    if (spec) *spec = plan->spec;
    if (info) *info = plan->info;
    return LB_OK;
}

lb_status lb_paged_prefill_enqueue(const lb_paged_prefill_plan *plan, lb_scope *scope,
                                   const lb_paged_prefill_args *args) {
    if (!plan || !scope || !args) return fail(LB_INVALID_ARGUMENT, "plan");
    const lb_prefill_spec &spec = plan->spec;
    const lb_paged_prefill_plan_info &c = plan->info;
    if (scope->queue->device != plan->device)
        return fail(LB_BUFFER_CONTEXT_MISMATCH, nullptr, plan->device, scope->queue->device);
    const bool split = c.partitions > 1; // two commands and a workspace
    lb_status rc = require_command_capacity(*scope, split ? 2 : 1);
    if (rc) return rc;
    OperandRequest requests[10] = {
        {args->query, LB_BF16, false},         {args->key_pages, LB_BF16, false},
        {args->value_pages, LB_BF16, false},   {args->qo_indptr, LB_I32, false},
        {args->page_indptr, LB_I32, false},    {args->page_indices, LB_I32, false},
        {args->last_page_len, LB_I32, false},  {args->output, LB_BF16, true},
        {args->lse, LB_F32, true},             {args->workspace, LB_F32, true},
    };
    Operand op[10];
    if ((rc = resolve(*scope, requests, split ? 10 : 9, op))) return rc;
    // the order of the reference's checks, prefill.rs:2475-2510
    const size_t pool = lb_prefill_spec_kv_pages_numel(&spec);
    if ((rc = require_exact_len("Q", op[0].numel, lb_prefill_spec_query_numel(&spec)))) return rc;
    if ((rc = require_exact_len("K_pages", op[1].numel, pool))) return rc;
    if ((rc = require_exact_len("V_pages", op[2].numel, pool))) return rc;
    if ((rc = require_exact_len("qo_indptr", op[3].numel, spec.batch_size + 1))) return rc;
    if ((rc = require_exact_len("page_indptr", op[4].numel, spec.batch_size + 1))) return rc;
    if (op[5].numel < spec.batch_size)
        return fail(LB_PAGE_INDICES_TOO_SHORT, nullptr, (int64_t)spec.batch_size,
                    (int64_t)op[5].numel);
    if (op[5].numel > 0x7fffffffu)
        return fail(LB_ENQUEUE_LENGTH_MISMATCH, "page_indices", 0x7fffffff, (int64_t)op[5].numel);
    if ((rc = require_exact_len("last_page_len", op[6].numel, spec.batch_size))) return rc;
    if ((rc = require_exact_len("O", op[7].numel, lb_prefill_spec_query_numel(&spec)))) return rc;
    if ((rc = require_exact_len("LSE", op[8].numel, lb_prefill_spec_lse_numel(&spec)))) return rc;
    if (split && (rc = require_exact_len("workspace", op[9].numel, c.workspace_numel))) return rc;
    if ((rc = require_alignment("Q", op[0].ptr, 16))) return rc;
    if ((rc = require_alignment("K_pages", op[1].ptr, 16))) return rc;
    if ((rc = require_alignment("V_pages", op[2].ptr, 16))) return rc;
    if ((rc = require_alignment("O", op[7].ptr, 16))) return rc;
    if (split && (rc = require_alignment("workspace", op[9].ptr, 8))) return rc;

    PrefillLaunch launch;
    memset(&launch, 0, sizeof(launch));
    // the pools as the decode kernels see them: [64 dims][token row][head half], one box = the
    // 16 token rows of a page x the two 128-byte halves of one KV head
    const uint64_t dims[3] = {64, (uint64_t)spec.max_num_pages * LB_PAGE_SIZE,
                              (uint64_t)spec.num_kv_heads * 2};
    const uint64_t strides[2] = {(uint64_t)spec.num_kv_heads * LB_HEAD_DIM * 2, 128};
    const uint32_t box[3] = {64, 16, 2};
    // the tiled kernel loads K by 64-dim halves, so that the 128 token rows of a block lie 128
    // bytes apart in shared memory and form one MMA operand
    const bool tiled = c.algorithm == LB_PREFILL_TILED;
    const uint32_t k_box[3] = {64, 16, tiled ? 1u : 2u};
    int error = driver().encode_tensor_map_3d(plan->device, launch.k_map, op[1].ptr, dims, strides,
                                              k_box);
    if (!error)
        error = driver().encode_tensor_map_3d(plan->device, launch.v_map, op[2].ptr, dims, strides,
                                              box);
    if (error) return fail(LB_LAUNCH_CONTRACT, "tensor_map", error);
    launch.query = op[0].ptr;
    launch.qo_indptr = (const int32_t *)op[3].ptr;
    launch.indptr = (const int32_t *)op[4].ptr;
    launch.indices = (const int32_t *)op[5].ptr;
    launch.last = (const int32_t *)op[6].ptr;
    launch.output = op[7].ptr;
    launch.lse = (float *)op[8].ptr;
    launch.status = plan->status;
    launch.batch = (int32_t)spec.batch_size;
    launch.nnz_qo = (int32_t)spec.nnz_qo;
    launch.max_pages = (int32_t)spec.max_num_pages;
    launch.qh = (int32_t)spec.num_query_heads;
    launch.kvh = (int32_t)spec.num_kv_heads;
    launch.indices_len = (int32_t)op[5].numel;
    launch.indices_min = plan->indices_capacity ? 0 : launch.indices_len;
    launch.q_tiles = (int32_t)c.q_tiles;
    launch.pages_per_stage = (int32_t)c.pages_per_stage;
    launch.stages = (int32_t)c.stages;
    launch.tiles = (int32_t)c.tiles;
    launch.scale_log2 = spec.softmax_scale * kLog2E;
    launch.grid = c.grid;
    launch.block = c.block;
    launch.shared_bytes = c.shared_bytes;
    launch.workspace = split ? (float *)op[9].ptr : nullptr;
    launch.partitions = (int32_t)c.partitions;
    launch.min_chunk_blocks = (int32_t)c.min_chunk_blocks;
    launch.wait_cycles = plan->wait_cycles;
    launch.test_lost_copy = plan->test_lost_copy;
    void *stream = scope->queue->stream;
    if ((rc = submit_launch(*scope, [&]() {
             return tiled ? launch_paged_prefill_tiled(launch, stream)
                          : launch_paged_prefill(launch, stream);
         })))
        return rc;
    if (!split) return LB_OK;

    // second command: the workspace is now a read operand, as in the split-K decode
    // (decode.rs:1374-1388)
    OperandRequest merge_requests[3] = {
        {lb_handle_read(args->workspace), LB_F32, false},
        {args->output, LB_BF16, true},
        {args->lse, LB_F32, true},
    };
    Operand merge_op[3];
    if ((rc = require_command_capacity(*scope, 1))) return rc;
    if ((rc = resolve(*scope, merge_requests, 3, merge_op))) return rc;
    return submit_launch(*scope, [&]() { return launch_prefill_merge(launch, stream); });
}

}
