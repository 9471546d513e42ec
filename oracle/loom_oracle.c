/*
 * CPU oracle for the Loom Infer paged-decode hot path.  TEST INFRASTRUCTURE ONLY:
 * the checker for tests, the smoke entry and the benchmark's CPU-baseline leg.
 * Nothing in the product library includes, links or calls this file.
 *
 * Parity status: PINNED by the reference's published CPU-reference digests
 * (tests/golden/reference_digests.json; checked by tests/test_oracle_golden.py).
 *
 * Build: gcc -O2 -ffp-contract=off -pthread.  Contraction must stay
 * off: the reference fuses only the Q.K dot product (explicit mul_add).
 */
#include "loom_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#define HEAD_DIM 128u  /* crates/loom-infer/src/attention/single_decode/mod.rs:8 */
#define PAGE_SIZE 16u  /* crates/loom-infer/src/attention/paged_decode/mod.rs:9 */
#define STATE_WIDTH 130u /* single_decode/mod.rs:13 */
static const float LOG2_E_F32 = 1.44269504088896340736f;

/* ---- error helpers --------------------------------------------------------------------- */

static int fail(lo_error *err, int code, const char *buffer, int64_t a, int64_t b, int64_t c,
                int64_t d) {
    if (err) {
        memset(err, 0, sizeof(*err));
        err->code = code;
        if (buffer) strncpy(err->buffer, buffer, sizeof(err->buffer) - 1);
        err->a = a; err->b = b; err->c = c; err->d = d;
    }
    return code;
}

/* crates/loom-infer/src/error.rs:276-290 */
static int require_len(lo_error *err, const char *buffer, size_t actual, size_t expected) {
    if (actual == expected) return LO_OK;
    return fail(err, LO_LENGTH_MISMATCH, buffer, (int64_t)expected, (int64_t)actual, 0, 0);
}

static int mul_overflow(size_t a, size_t b, size_t *out) { return __builtin_mul_overflow(a, b, out); }

/* ---- bf16, fixture, digests ------------------------------------------------------------ */

/* Round-to-nearest-even with NaN quieting, as half 2.7.1 bf16::from_f32 (Cargo.lock:232). */
uint16_t lo_bf16_from_f32(float value) {
    uint32_t x;
    memcpy(&x, &value, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x0040u);
    const uint32_t round_bit = 0x8000u;
    if ((x & round_bit) != 0 && (x & (3 * round_bit - 1)) != 0) return (uint16_t)((x >> 16) + 1);
    return (uint16_t)(x >> 16);
}

float lo_bf16_to_f32(uint16_t bits) {
    uint32_t x = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &x, 4);
    return value;
}

/* crates/loom-infer-validation/src/support/fixture.rs:5-16 */
void lo_fixture_bf16(uint16_t *out, size_t len, uint64_t salt) {
    uint64_t state = 0x9e3779b97f4a7c15ull ^ salt;
    for (size_t i = 0; i < len; ++i) {
        state ^= state << 13;
        state ^= state >> 7;
        state ^= state << 17;
        int32_t sign = (int32_t)(state % 2001) - 1000;
        out[i] = lo_bf16_from_f32((float)sign / 2048.0f);
    }
}

/* crates/loom-infer-validation/src/support/comparison.rs:6-21 */
uint64_t lo_digest_u16(const uint16_t *values, size_t len) {
    uint64_t digest = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < len; ++i) digest = (digest ^ (uint64_t)values[i]) * 0x00000100000001b3ull;
    return digest;
}

/* comparison.rs:33-45 (f32 bits) and benchmarks/matched.rs:175-179 (i32 as u32) */
uint64_t lo_digest_u32(const uint32_t *values, size_t len) {
    uint64_t digest = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < len; ++i) digest = (digest ^ (uint64_t)values[i]) * 0x00000100000001b3ull;
    return digest;
}

/* ---- paged spec + page table ----------------------------------------------------------- */

/* crates/loom-infer/src/attention/paged_decode/mod.rs:28-82 */
int lo_paged_spec_new(size_t batch, size_t max_pages, size_t qh, size_t kvh, size_t head_dim,
                      size_t page_size, lo_paged_spec *spec, lo_error *err) {
    if (batch == 0 || max_pages == 0 || qh == 0 || kvh == 0 || head_dim == 0 || page_size == 0)
        return fail(err, LO_ZERO_DIMENSION, NULL, 0, 0, 0, 0);
    if (head_dim != HEAD_DIM)
        return fail(err, LO_UNSUPPORTED_HEAD_DIMENSION, NULL, HEAD_DIM, (int64_t)head_dim, 0, 0);
    if (page_size != PAGE_SIZE)
        return fail(err, LO_UNSUPPORTED_PAGE_SIZE, NULL, PAGE_SIZE, (int64_t)page_size, 0, 0);
    if (qh % kvh != 0)
        return fail(err, LO_INVALID_HEAD_MAPPING, NULL, (int64_t)qh, (int64_t)kvh, 0, 0);
    size_t t;
    if (batch + 1 < batch || mul_overflow(batch, qh, &t) || mul_overflow(t, head_dim, &t))
        return fail(err, LO_ELEMENT_COUNT_OVERFLOW, NULL, 0, 0, 0, 0);
    if (mul_overflow(max_pages, page_size, &t) || mul_overflow(t, kvh, &t) ||
        mul_overflow(t, head_dim, &t))
        return fail(err, LO_ELEMENT_COUNT_OVERFLOW, NULL, 0, 0, 0, 0);
    spec->batch_size = batch;
    spec->max_num_pages = max_pages;
    spec->num_query_heads = qh;
    spec->num_kv_heads = kvh;
    return LO_OK;
}

static size_t kv_pages_numel(const lo_paged_spec *s) {
    return s->max_num_pages * PAGE_SIZE * s->num_kv_heads * HEAD_DIM;
}
static size_t query_numel(const lo_paged_spec *s) {
    return s->batch_size * s->num_query_heads * HEAD_DIM;
}

/* paged_decode/mod.rs:152-213 */
int lo_validate_page_table(const lo_paged_spec *spec, const int32_t *indptr, size_t indptr_len,
                           const int32_t *indices, size_t indices_len, const int32_t *last,
                           size_t last_len, lo_error *err) {
    int rc;
    if ((rc = require_len(err, "page_indptr", indptr_len, spec->batch_size + 1))) return rc;
    if ((rc = require_len(err, "last_page_len", last_len, spec->batch_size))) return rc;
    if (indptr[0] != 0) return fail(err, LO_INVALID_PAGE_INDPTR_START, NULL, indptr[0], 0, 0, 0);
    for (size_t request = 0; request < spec->batch_size; ++request) {
        int32_t start = indptr[request], end = indptr[request + 1];
        if (end < start)
            return fail(err, LO_NON_MONOTONIC_PAGE_INDPTR, NULL, (int64_t)request, start, end, 0);
        if (end == start) return fail(err, LO_EMPTY_PAGED_REQUEST, NULL, (int64_t)request, 0, 0, 0);
        int32_t length = last[request];
        if (length < 1 || length > (int32_t)PAGE_SIZE)
            return fail(err, LO_INVALID_LAST_PAGE_LENGTH, NULL, (int64_t)request, length,
                        PAGE_SIZE, 0);
    }
    if (indptr[spec->batch_size] < 0) return fail(err, LO_ELEMENT_COUNT_OVERFLOW, NULL, 0, 0, 0, 0);
    if ((rc = require_len(err, "page_indices", indices_len, (size_t)indptr[spec->batch_size])))
        return rc;
    for (size_t position = 0; position < indices_len; ++position) {
        int32_t index = indices[position];
        if (index < 0 || (size_t)index >= spec->max_num_pages)
            return fail(err, LO_PAGE_INDEX_OUT_OF_RANGE, NULL, (int64_t)position, index,
                        (int64_t)spec->max_num_pages, 0);
    }
    return LO_OK;
}

/* paged_decode/mod.rs:252-257 */
static size_t request_kv_len(const int32_t *indptr, const int32_t *last, size_t request) {
    size_t pages = (size_t)(indptr[request + 1] - indptr[request]);
    return (pages - 1) * PAGE_SIZE + (size_t)last[request];
}

/* paged_decode/mod.rs:260-278 */
static void physical_slot(const int32_t *indptr, const int32_t *indices, size_t request,
                          size_t token, size_t *page, size_t *offset) {
    *page = (size_t)indices[(size_t)indptr[request] + token / PAGE_SIZE];
    *offset = token % PAGE_SIZE;
}

/* ---- paged decode reference ------------------------------------------------------------ */

/* paged_decode/mod.rs:309-361: one (request, query head) */
static void paged_decode_one(const lo_paged_spec *spec, const uint16_t *q, const uint16_t *k_pages,
                             const uint16_t *v_pages, const int32_t *indptr,
                             const int32_t *indices, const int32_t *last, size_t request,
                             size_t query_head, uint16_t *out, float *lse) {
    const size_t qh = spec->num_query_heads, kvh = spec->num_kv_heads;
    const float scale = 1.0f / sqrtf((float)HEAD_DIM);
    const size_t kv_len = request_kv_len(indptr, last, request);
    const size_t query_offset = (request * qh + query_head) * HEAD_DIM;
    const size_t kv_head = query_head / (qh / kvh);
    float query[HEAD_DIM];
    for (size_t c = 0; c < HEAD_DIM; ++c) query[c] = lo_bf16_to_f32(q[query_offset + c]);
    float state[HEAD_DIM];
    float max_score = 0.0f, normalizer = 0.0f;
    memset(state, 0, sizeof(state));
    for (size_t token = 0; token < kv_len; ++token) {
        size_t page, offset;
        physical_slot(indptr, indices, request, token, &page, &offset);
        const size_t kv_offset = ((page * PAGE_SIZE + offset) * kvh + kv_head) * HEAD_DIM;
        float dot = 0.0f;
        for (size_t c = 0; c < HEAD_DIM; ++c)
            dot = fmaf(query[c], lo_bf16_to_f32(k_pages[kv_offset + c]), dot);
        const float score = dot * scale;
        if (token == 0) {
            max_score = score;
            normalizer = 1.0f;
            for (size_t c = 0; c < HEAD_DIM; ++c) state[c] = lo_bf16_to_f32(v_pages[kv_offset + c]);
            continue;
        }
        const float next_max = fmaxf(max_score, score);
        const float previous_weight = expf(max_score - next_max);
        const float current_weight = expf(score - next_max);
        normalizer = normalizer * previous_weight + current_weight;
        for (size_t c = 0; c < HEAD_DIM; ++c)
            state[c] = state[c] * previous_weight +
                       lo_bf16_to_f32(v_pages[kv_offset + c]) * current_weight;
        max_score = next_max;
    }
    for (size_t c = 0; c < HEAD_DIM; ++c)
        out[query_offset + c] = lo_bf16_from_f32(state[c] / normalizer);
    lse[request * qh + query_head] = (max_score + logf(normalizer)) * LOG2_E_F32;
}

struct decode_job {
    const lo_paged_spec *spec;
    const uint16_t *q, *k_pages, *v_pages;
    const int32_t *indptr, *indices, *last;
    uint16_t *out;
    float *lse;
    size_t pairs;
    size_t next; /* claimed with an atomic fetch-add */
};

static void *decode_worker(void *arg) {
    struct decode_job *job = (struct decode_job *)arg;
    for (;;) {
        const size_t pair = __atomic_fetch_add(&job->next, 1, __ATOMIC_RELAXED);
        if (pair >= job->pairs) break;
        paged_decode_one(job->spec, job->q, job->k_pages, job->v_pages, job->indptr, job->indices,
                         job->last, pair / job->spec->num_query_heads,
                         pair % job->spec->num_query_heads, job->out, job->lse);
    }
    return NULL;
}

/* paged_decode/mod.rs:287-366.  threads > 1 distributes (request, head) pairs over POSIX
 * threads; every pair keeps the reference's arithmetic order, so results are identical. */
int lo_paged_decode_ref(const lo_paged_spec *spec, const uint16_t *q, size_t q_len,
                        const uint16_t *k_pages, size_t k_len, const uint16_t *v_pages,
                        size_t v_len, const int32_t *indptr, size_t indptr_len,
                        const int32_t *indices, size_t indices_len, const int32_t *last,
                        size_t last_len, uint16_t *out, size_t out_len, float *lse,
                        size_t lse_len, int threads, lo_error *err) {
    int rc;
    if ((rc = require_len(err, "Q", q_len, query_numel(spec)))) return rc;
    if ((rc = require_len(err, "K_pages", k_len, kv_pages_numel(spec)))) return rc;
    if ((rc = require_len(err, "V_pages", v_len, kv_pages_numel(spec)))) return rc;
    if ((rc = require_len(err, "O", out_len, query_numel(spec)))) return rc;
    if ((rc = require_len(err, "LSE", lse_len, spec->batch_size * spec->num_query_heads)))
        return rc;
    if ((rc = lo_validate_page_table(spec, indptr, indptr_len, indices, indices_len, last,
                                     last_len, err)))
        return rc;
    struct decode_job job = {spec, q, k_pages, v_pages, indptr, indices, last, out, lse,
                             spec->batch_size * spec->num_query_heads, 0};
    if (threads <= 1) {
        decode_worker(&job);
        return LO_OK;
    }
    if (threads > 256) threads = 256;
    pthread_t workers[256];
    int started = 0;
    for (int t = 0; t < threads - 1; ++t)
        if (pthread_create(&workers[started], NULL, decode_worker, &job) == 0) ++started;
    decode_worker(&job);
    for (int t = 0; t < started; ++t) pthread_join(workers[t], NULL);
    return LO_OK;
}

/* ---- contiguous single decode + split-K ------------------------------------------------ */

/* single_decode/mod.rs:200-261 */
int lo_single_decode_ref(size_t kv_len, size_t qh, size_t kvh, const uint16_t *q,
                         const uint16_t *k, const uint16_t *v, uint16_t *out, float *lse,
                         lo_error *err) {
    if (kv_len == 0 || qh == 0 || kvh == 0) return fail(err, LO_ZERO_DIMENSION, NULL, 0, 0, 0, 0);
    if (qh % kvh != 0)
        return fail(err, LO_INVALID_HEAD_MAPPING, NULL, (int64_t)qh, (int64_t)kvh, 0, 0);
    const float scale = 1.0f / sqrtf((float)HEAD_DIM);
    for (size_t query_head = 0; query_head < qh; ++query_head) {
        const size_t query_offset = query_head * HEAD_DIM;
        const size_t kv_head = query_head / (qh / kvh);
        float state[HEAD_DIM];
        memset(state, 0, sizeof(state));
        float max_score = 0.0f, normalizer = 0.0f;
        for (size_t token = 0; token < kv_len; ++token) {
            const size_t kv_offset = (token * kvh + kv_head) * HEAD_DIM;
            float dot = 0.0f;
            for (size_t c = 0; c < HEAD_DIM; ++c)
                dot = fmaf(lo_bf16_to_f32(q[query_offset + c]), lo_bf16_to_f32(k[kv_offset + c]),
                           dot);
            const float score = dot * scale;
            if (token == 0) {
                max_score = score;
                normalizer = 1.0f;
                for (size_t c = 0; c < HEAD_DIM; ++c) state[c] = lo_bf16_to_f32(v[kv_offset + c]);
                continue;
            }
            const float next_max = fmaxf(max_score, score);
            const float previous_weight = expf(max_score - next_max);
            const float current_weight = expf(score - next_max);
            normalizer = normalizer * previous_weight + current_weight;
            for (size_t c = 0; c < HEAD_DIM; ++c)
                state[c] = state[c] * previous_weight +
                           lo_bf16_to_f32(v[kv_offset + c]) * current_weight;
            max_score = next_max;
        }
        for (size_t c = 0; c < HEAD_DIM; ++c)
            out[query_offset + c] = lo_bf16_from_f32(state[c] / normalizer);
        lse[query_head] = (max_score + logf(normalizer)) * LOG2_E_F32;
    }
    return LO_OK;
}

/* single_decode/mod.rs:171-185 */
int lo_split_k_partition_range(size_t kv_len, size_t partitions, size_t partition, size_t *start,
                               size_t *end) {
    if (partition >= partitions) return 1;
    const size_t base = kv_len / partitions, remainder = kv_len % partitions;
    const size_t extra_before = partition < remainder ? partition : remainder;
    *start = partition * base + extra_before;
    *end = *start + base + (partition < remainder ? 1 : 0);
    return 0;
}

/* One unnormalised state over `count` tokens; token i's K/V row offsets come from
 * `row_offset(i)`.  Arithmetic: single_decode/mod.rs:294-325 (log2 domain, exp2). */
typedef size_t (*row_offset_fn)(const void *ctx, size_t token);

static void partial_state(const float *query, const uint16_t *k, const uint16_t *v,
                          row_offset_fn row_offset, const void *ctx, size_t token_start,
                          size_t token_end, float *state /* 130 */) {
    const float scale = 1.0f / sqrtf((float)HEAD_DIM);
    float *weighted = state + 2;
    for (size_t c = 0; c < HEAD_DIM; ++c) weighted[c] = 0.0f;
    float max_log2 = 0.0f, normalizer = 0.0f;
    for (size_t token = token_start; token < token_end; ++token) {
        const size_t kv_offset = row_offset(ctx, token);
        float dot = 0.0f;
        for (size_t c = 0; c < HEAD_DIM; ++c)
            dot = fmaf(query[c], lo_bf16_to_f32(k[kv_offset + c]), dot);
        const float score_log2 = dot * scale * LOG2_E_F32;
        if (token == token_start) {
            max_log2 = score_log2;
            normalizer = 1.0f;
            for (size_t c = 0; c < HEAD_DIM; ++c) weighted[c] = lo_bf16_to_f32(v[kv_offset + c]);
            continue;
        }
        const float next_max = fmaxf(max_log2, score_log2);
        const float previous_weight = exp2f(max_log2 - next_max);
        const float current_weight = exp2f(score_log2 - next_max);
        normalizer = normalizer * previous_weight + current_weight;
        for (size_t c = 0; c < HEAD_DIM; ++c)
            weighted[c] = weighted[c] * previous_weight +
                          lo_bf16_to_f32(v[kv_offset + c]) * current_weight;
        max_log2 = next_max;
    }
    state[0] = max_log2;
    state[1] = normalizer;
}

struct contiguous_ctx { size_t kvh, kv_head; };
static size_t contiguous_row(const void *ctx, size_t token) {
    const struct contiguous_ctx *c = (const struct contiguous_ctx *)ctx;
    return (token * c->kvh + c->kv_head) * HEAD_DIM;
}

/* single_decode/mod.rs:264-329 */
int lo_split_k_partials_ref(size_t kv_len, size_t qh, size_t kvh, size_t partitions,
                            const uint16_t *q, const uint16_t *k, const uint16_t *v,
                            float *workspace, size_t workspace_len, lo_error *err) {
    if (partitions == 0 || partitions > kv_len)
        return fail(err, LO_INVALID_PARTITION_COUNT, NULL, (int64_t)partitions, (int64_t)kv_len, 0,
                    0);
    int rc;
    if ((rc = require_len(err, "workspace", workspace_len, qh * partitions * STATE_WIDTH)))
        return rc;
    for (size_t query_head = 0; query_head < qh; ++query_head) {
        float query[HEAD_DIM];
        for (size_t c = 0; c < HEAD_DIM; ++c)
            query[c] = lo_bf16_to_f32(q[query_head * HEAD_DIM + c]);
        struct contiguous_ctx ctx = {kvh, query_head / (qh / kvh)};
        for (size_t partition = 0; partition < partitions; ++partition) {
            size_t start, end;
            lo_split_k_partition_range(kv_len, partitions, partition, &start, &end);
            partial_state(query, k, v, contiguous_row, &ctx, start, end,
                          workspace + (query_head * partitions + partition) * STATE_WIDTH);
        }
    }
    return LO_OK;
}

/* single_decode/mod.rs:343-379.  skip_empty additionally ignores states whose normaliser is
 * zero, as the device merge does (crates/loom-infer-cuda/src/attention/decode.rs:635); the
 * contiguous contract never produces one, the page-granular paged split can. */
static void merge_states(const float *states, size_t partitions, int skip_empty, uint16_t *out,
                         float *lse) {
    float merged[HEAD_DIM];
    float merged_max = 0.0f, merged_normalizer = 0.0f;
    for (size_t partition = 0; partition < partitions; ++partition) {
        const float *state = states + partition * STATE_WIDTH;
        if (partition == 0) {
            merged_max = state[0];
            merged_normalizer = state[1];
            memcpy(merged, state + 2, sizeof(merged));
            continue;
        }
        if (skip_empty && state[1] == 0.0f) continue;
        const float next_max = fmaxf(merged_max, state[0]);
        const float merged_weight = exp2f(merged_max - next_max);
        const float partition_weight = exp2f(state[0] - next_max);
        merged_normalizer = merged_normalizer * merged_weight + state[1] * partition_weight;
        for (size_t c = 0; c < HEAD_DIM; ++c)
            merged[c] = merged[c] * merged_weight + state[c + 2] * partition_weight;
        merged_max = next_max;
    }
    for (size_t c = 0; c < HEAD_DIM; ++c) out[c] = lo_bf16_from_f32(merged[c] / merged_normalizer);
    *lse = merged_max + log2f(merged_normalizer);
}

/* single_decode/mod.rs:332-381 */
int lo_split_k_merge_ref(size_t qh, size_t partitions, const float *workspace,
                         size_t workspace_len, uint16_t *out, float *lse, lo_error *err) {
    int rc;
    if ((rc = require_len(err, "workspace", workspace_len, qh * partitions * STATE_WIDTH)))
        return rc;
    for (size_t query_head = 0; query_head < qh; ++query_head)
        merge_states(workspace + query_head * partitions * STATE_WIDTH, partitions, 0,
                     out + query_head * HEAD_DIM, lse + query_head);
    return LO_OK;
}

/* ---- paged split-K (extension of the contiguous split-K contract to the page table) ----- */

struct paged_ctx {
    const int32_t *indptr, *indices;
    size_t request, kvh, kv_head;
};
static size_t paged_row(const void *ctx, size_t token) {
    const struct paged_ctx *c = (const struct paged_ctx *)ctx;
    size_t page, offset;
    physical_slot(c->indptr, c->indices, c->request, token, &page, &offset);
    return ((page * PAGE_SIZE + offset) * c->kvh + c->kv_head) * HEAD_DIM;
}

/* The reference has no paged split-K.  This applies its partial-state arithmetic
 * (single_decode/mod.rs:294-325) to each request's tokens, partitioned by the balanced rule
 * of :171-185 applied to the request's PAGE count (so chunks are whole pages).  Workspace
 * layout [batch, query_heads, partitions, 130] extends partial_state_offset (:187-193) with
 * a leading request dimension.  A chunk with no pages yields the state [0, 0, 0...]. */
int lo_paged_split_k_partials_ref(const lo_paged_spec *spec, size_t partitions,
                                  const uint16_t *q, const uint16_t *k_pages,
                                  const uint16_t *v_pages, const int32_t *indptr,
                                  const int32_t *indices, size_t indices_len,
                                  const int32_t *last, float *workspace, lo_error *err) {
    int rc;
    if (partitions == 0)
        return fail(err, LO_INVALID_PARTITION_COUNT, NULL, 0, 0, 0, 0);
    if ((rc = lo_validate_page_table(spec, indptr, spec->batch_size + 1, indices, indices_len,
                                     last, spec->batch_size, err)))
        return rc;
    const size_t qh = spec->num_query_heads, kvh = spec->num_kv_heads;
    for (size_t request = 0; request < spec->batch_size; ++request) {
        const size_t pages = (size_t)(indptr[request + 1] - indptr[request]);
        const size_t kv_len = request_kv_len(indptr, last, request);
        for (size_t query_head = 0; query_head < qh; ++query_head) {
            float query[HEAD_DIM];
            for (size_t c = 0; c < HEAD_DIM; ++c)
                query[c] = lo_bf16_to_f32(q[(request * qh + query_head) * HEAD_DIM + c]);
            struct paged_ctx ctx = {indptr, indices, request, kvh, query_head / (qh / kvh)};
            for (size_t partition = 0; partition < partitions; ++partition) {
                size_t page_start, page_end;
                lo_split_k_partition_range(pages, partitions, partition, &page_start, &page_end);
                size_t token_start = page_start * PAGE_SIZE, token_end = page_end * PAGE_SIZE;
                if (token_end > kv_len) token_end = kv_len;
                if (token_start > token_end) token_start = token_end;
                partial_state(query, k_pages, v_pages, paged_row, &ctx, token_start, token_end,
                              workspace +
                                  ((request * qh + query_head) * partitions + partition) *
                                      STATE_WIDTH);
            }
        }
    }
    return LO_OK;
}

int lo_paged_split_k_merge_ref(const lo_paged_spec *spec, size_t partitions,
                               const float *workspace, uint16_t *out, float *lse) {
    const size_t states = spec->batch_size * spec->num_query_heads;
    for (size_t s = 0; s < states; ++s)
        merge_states(workspace + s * partitions * STATE_WIDTH, partitions, 1, out + s * HEAD_DIM,
                     lse + s);
    return LO_OK;
}

/* ---- RoPE ------------------------------------------------------------------------------ */

/* crates/loom-infer/src/rope/mod.rs:136-161 */
static void rotate_tensor(const uint16_t *input, const int32_t *positions, size_t tokens,
                          uint16_t *output, size_t heads, size_t head_dim, size_t rotary_dim,
                          float rope_scale, float rope_theta) {
    const size_t half = rotary_dim / 2;
    for (size_t token = 0; token < tokens; ++token) {
        const int32_t position = positions[token];
        for (size_t head = 0; head < heads; ++head) {
            const size_t base = (token * heads + head) * head_dim;
            for (size_t pair = 0; pair < half; ++pair) {
                const float exponent = 2.0f * (float)pair / (float)rotary_dim;
                const float inverse_frequency = powf(rope_theta, -exponent) / rope_scale;
                const float angle = (float)position * inverse_frequency;
                const float s = sinf(angle), c = cosf(angle);
                const float first = lo_bf16_to_f32(input[base + pair]);
                const float second = lo_bf16_to_f32(input[base + half + pair]);
                output[base + pair] = lo_bf16_from_f32(first * c - second * s);
                output[base + half + pair] = lo_bf16_from_f32(second * c + first * s);
            }
            for (size_t c = rotary_dim; c < head_dim; ++c) output[base + c] = input[base + c];
        }
    }
}

/* rope/mod.rs:21-63 (spec checks) and :111-134 */
int lo_rope_ref(size_t tokens, size_t qh, size_t kh, size_t head_dim, size_t rotary_dim,
                float rope_scale, float rope_theta, const uint16_t *q, size_t q_len,
                const uint16_t *k, size_t k_len, const int32_t *positions, size_t pos_len,
                uint16_t *q_out, size_t q_out_len, uint16_t *k_out, size_t k_out_len,
                lo_error *err) {
    if (tokens == 0 || qh == 0 || kh == 0 || head_dim == 0)
        return fail(err, LO_ZERO_DIMENSION, NULL, 0, 0, 0, 0);
    if (rotary_dim == 0 || rotary_dim % 2 != 0 || rotary_dim > head_dim)
        return fail(err, LO_INVALID_ROTARY_DIMENSION, NULL, (int64_t)rotary_dim,
                    (int64_t)head_dim, 0, 0);
    if (!isfinite(rope_scale) || rope_scale <= 0.0f)
        return fail(err, LO_INVALID_ROPE_SCALE, NULL, 0, 0, 0, 0);
    if (!isfinite(rope_theta) || rope_theta <= 1.0f)
        return fail(err, LO_INVALID_ROPE_THETA, NULL, 0, 0, 0, 0);
    int rc;
    if ((rc = require_len(err, "query", q_len, tokens * qh * head_dim))) return rc;
    if ((rc = require_len(err, "key", k_len, tokens * kh * head_dim))) return rc;
    if ((rc = require_len(err, "position_ids", pos_len, tokens))) return rc;
    if ((rc = require_len(err, "query_output", q_out_len, tokens * qh * head_dim))) return rc;
    if ((rc = require_len(err, "key_output", k_out_len, tokens * kh * head_dim))) return rc;
    for (size_t token = 0; token < tokens; ++token)
        if (positions[token] < 0)
            return fail(err, LO_NEGATIVE_POSITION_ID, NULL, (int64_t)token, positions[token], 0, 0);
    rotate_tensor(q, positions, tokens, q_out, qh, head_dim, rotary_dim, rope_scale, rope_theta);
    rotate_tensor(k, positions, tokens, k_out, kh, head_dim, rotary_dim, rope_scale, rope_theta);
    return LO_OK;
}

/* ---- fused RoPE + paged append --------------------------------------------------------- */

/* crates/loom-infer/src/attention/paged_append/mod.rs:95-131 */
int lo_append_validate_page_table(const lo_paged_spec *spec, const int32_t *indptr,
                                  size_t indptr_len, const int32_t *indices, size_t indices_len,
                                  const int32_t *last, size_t last_len, lo_error *err) {
    int rc;
    if ((rc = lo_validate_page_table(spec, indptr, indptr_len, indices, indices_len, last,
                                     last_len, err)))
        return rc;
    for (size_t first = 0; first < spec->batch_size; ++first) {
        size_t first_page, first_offset;
        physical_slot(indptr, indices, first, request_kv_len(indptr, last, first) - 1,
                      &first_page, &first_offset);
        for (size_t second = first + 1; second < spec->batch_size; ++second) {
            size_t second_page, second_offset;
            physical_slot(indptr, indices, second, request_kv_len(indptr, last, second) - 1,
                          &second_page, &second_offset);
            if (first_page == second_page && first_offset == second_offset)
                return fail(err, LO_DUPLICATE_PAGE_APPEND_SLOT, NULL, (int64_t)first,
                            (int64_t)second, (int64_t)first_page, (int64_t)first_offset);
        }
    }
    return LO_OK;
}

/* paged_append/mod.rs:144-177 (token count) and :244-317 (metadata).  max_tokens is the
 * contract cap (64); pass 0 to lift the cap for the extended any-total command, which is
 * otherwise the same validation. */
int lo_append_tokens_validate(const lo_paged_spec *spec, size_t tokens, size_t max_tokens,
                              const int32_t *batch_indices, size_t batch_indices_len,
                              const int32_t *positions, size_t positions_len,
                              const int32_t *indptr, size_t indptr_len, const int32_t *indices,
                              size_t indices_len, const int32_t *last, size_t last_len,
                              int64_t *slots_out, lo_error *err) {
    if (tokens == 0) return fail(err, LO_ZERO_DIMENSION, NULL, 0, 0, 0, 0);
    if (max_tokens != 0 && tokens > max_tokens)
        return fail(err, LO_UNSUPPORTED_APPEND_TOKEN_COUNT, NULL, (int64_t)max_tokens,
                    (int64_t)tokens, 0, 0);
    int rc;
    if ((rc = require_len(err, "batch_indices", batch_indices_len, tokens))) return rc;
    if ((rc = require_len(err, "positions", positions_len, tokens))) return rc;
    if ((rc = lo_validate_page_table(spec, indptr, indptr_len, indices, indices_len, last,
                                     last_len, err)))
        return rc;
    int64_t *slots = slots_out ? slots_out : (int64_t *)malloc(tokens * 2 * sizeof(int64_t));
    rc = LO_OK;
    for (size_t token = 0; token < tokens && rc == LO_OK; ++token) {
        const int32_t index = batch_indices[token];
        if (index < 0 || (size_t)index >= spec->batch_size) {
            rc = fail(err, LO_APPEND_BATCH_INDEX_OUT_OF_RANGE, NULL, (int64_t)token, index,
                      (int64_t)spec->batch_size, 0);
            break;
        }
        const size_t request = (size_t)index;
        const size_t kv_len = request_kv_len(indptr, last, request);
        const int32_t position = positions[token];
        if (position < 0 || (size_t)position >= kv_len) {
            rc = fail(err, LO_APPEND_POSITION_OUT_OF_RANGE, NULL, (int64_t)token,
                      (int64_t)request, position, (int64_t)kv_len);
            break;
        }
        size_t page, offset;
        physical_slot(indptr, indices, request, (size_t)position, &page, &offset);
        for (size_t first = 0; first < token; ++first) {
            if (slots[first * 2] == (int64_t)page && slots[first * 2 + 1] == (int64_t)offset) {
                rc = fail(err, LO_DUPLICATE_PAGE_APPEND_TOKEN_SLOT, NULL, (int64_t)first,
                          (int64_t)token, (int64_t)page, (int64_t)offset);
                break;
            }
        }
        slots[token * 2] = (int64_t)page;
        slots[token * 2 + 1] = (int64_t)offset;
    }
    if (!slots_out) free(slots);
    return rc;
}

static void scatter_rows(const lo_paged_spec *spec, size_t page, size_t offset, size_t source_row,
                         const uint16_t *rotated_key, const uint16_t *value, uint16_t *k_pages,
                         uint16_t *v_pages) {
    const size_t kvh = spec->num_kv_heads;
    for (size_t kv_head = 0; kv_head < kvh; ++kv_head) {
        const size_t source = (source_row * kvh + kv_head) * HEAD_DIM;
        const size_t destination = ((page * PAGE_SIZE + offset) * kvh + kv_head) * HEAD_DIM;
        memcpy(k_pages + destination, rotated_key + source, HEAD_DIM * sizeof(uint16_t));
        memcpy(v_pages + destination, value + source, HEAD_DIM * sizeof(uint16_t));
    }
}

/* paged_append/mod.rs:360-425 */
int lo_rope_append_ref(const lo_paged_spec *spec, const uint16_t *q, size_t q_len,
                       const uint16_t *k, size_t k_len, const uint16_t *v, size_t v_len,
                       const int32_t *indptr, size_t indptr_len, const int32_t *indices,
                       size_t indices_len, const int32_t *last, size_t last_len, uint16_t *q_out,
                       size_t q_out_len, uint16_t *k_pages, size_t k_pages_len,
                       uint16_t *v_pages, size_t v_pages_len, lo_error *err) {
    const size_t batch = spec->batch_size, qh = spec->num_query_heads, kvh = spec->num_kv_heads;
    int rc;
    if ((rc = require_len(err, "query", q_len, batch * qh * HEAD_DIM))) return rc;
    if ((rc = require_len(err, "key", k_len, batch * kvh * HEAD_DIM))) return rc;
    if ((rc = require_len(err, "value", v_len, batch * kvh * HEAD_DIM))) return rc;
    if ((rc = require_len(err, "query_output", q_out_len, batch * qh * HEAD_DIM))) return rc;
    if ((rc = require_len(err, "key_pages", k_pages_len, kv_pages_numel(spec)))) return rc;
    if ((rc = require_len(err, "value_pages", v_pages_len, kv_pages_numel(spec)))) return rc;
    if ((rc = lo_append_validate_page_table(spec, indptr, indptr_len, indices, indices_len, last,
                                            last_len, err)))
        return rc;
    int32_t *positions = (int32_t *)malloc(batch * sizeof(int32_t));
    uint16_t *rotated = (uint16_t *)malloc(batch * kvh * HEAD_DIM * sizeof(uint16_t));
    for (size_t request = 0; request < batch; ++request)
        positions[request] = (int32_t)(request_kv_len(indptr, last, request) - 1);
    rc = lo_rope_ref(batch, qh, kvh, HEAD_DIM, HEAD_DIM, 1.0f, 10000.0f, q, q_len, k, k_len,
                     positions, batch, q_out, q_out_len, rotated, batch * kvh * HEAD_DIM, err);
    if (rc == LO_OK) {
        for (size_t request = 0; request < batch; ++request) {
            size_t page, offset;
            physical_slot(indptr, indices, request, (size_t)positions[request], &page, &offset);
            scatter_rows(spec, page, offset, request, rotated, v, k_pages, v_pages);
        }
    }
    free(positions);
    free(rotated);
    return rc;
}

/* paged_append/mod.rs:429-489 */
int lo_rope_append_tokens_ref(const lo_paged_spec *spec, size_t tokens, size_t max_tokens,
                              const uint16_t *q, size_t q_len, const uint16_t *k, size_t k_len,
                              const uint16_t *v, size_t v_len, const int32_t *batch_indices,
                              size_t batch_indices_len, const int32_t *positions,
                              size_t positions_len, const int32_t *indptr, size_t indptr_len,
                              const int32_t *indices, size_t indices_len, const int32_t *last,
                              size_t last_len, uint16_t *q_out, size_t q_out_len,
                              uint16_t *k_pages, size_t k_pages_len, uint16_t *v_pages,
                              size_t v_pages_len, lo_error *err) {
    const size_t qh = spec->num_query_heads, kvh = spec->num_kv_heads;
    int rc;
    if (tokens == 0) return fail(err, LO_ZERO_DIMENSION, NULL, 0, 0, 0, 0);
    if (max_tokens != 0 && tokens > max_tokens)
        return fail(err, LO_UNSUPPORTED_APPEND_TOKEN_COUNT, NULL, (int64_t)max_tokens,
                    (int64_t)tokens, 0, 0);
    if ((rc = require_len(err, "query", q_len, tokens * qh * HEAD_DIM))) return rc;
    if ((rc = require_len(err, "key", k_len, tokens * kvh * HEAD_DIM))) return rc;
    if ((rc = require_len(err, "value", v_len, tokens * kvh * HEAD_DIM))) return rc;
    if ((rc = require_len(err, "query_output", q_out_len, tokens * qh * HEAD_DIM))) return rc;
    if ((rc = require_len(err, "key_pages", k_pages_len, kv_pages_numel(spec)))) return rc;
    if ((rc = require_len(err, "value_pages", v_pages_len, kv_pages_numel(spec)))) return rc;
    int64_t *slots = (int64_t *)malloc(tokens * 2 * sizeof(int64_t));
    uint16_t *rotated = (uint16_t *)malloc(tokens * kvh * HEAD_DIM * sizeof(uint16_t));
    rc = lo_append_tokens_validate(spec, tokens, max_tokens, batch_indices, batch_indices_len,
                                   positions, positions_len, indptr, indptr_len, indices,
                                   indices_len, last, last_len, slots, err);
    if (rc == LO_OK)
        rc = lo_rope_ref(tokens, qh, kvh, HEAD_DIM, HEAD_DIM, 1.0f, 10000.0f, q, q_len, k, k_len,
                         positions, positions_len, q_out, q_out_len, rotated,
                         tokens * kvh * HEAD_DIM, err);
    if (rc == LO_OK)
        for (size_t token = 0; token < tokens; ++token)
            scatter_rows(spec, (size_t)slots[token * 2], (size_t)slots[token * 2 + 1], token,
                         rotated, v, k_pages, v_pages);
    free(slots);
    free(rotated);
    return rc;
}

/* ---- paged causal prefill --------------------------------------------------------------- */

/* crates/loom-infer/src/attention/paged_prefill/mod.rs:29-91 */
int lo_prefill_spec_new(size_t batch, size_t nnz_qo, size_t max_pages, size_t qh, size_t kvh,
                        size_t head_dim, size_t page_size, lo_prefill_spec *spec, lo_error *err) {
    if (batch == 0 || nnz_qo == 0 || max_pages == 0 || qh == 0 || kvh == 0 || head_dim == 0 ||
        page_size == 0)
        return fail(err, LO_ZERO_DIMENSION, NULL, 0, 0, 0, 0);
    if (head_dim != HEAD_DIM)
        return fail(err, LO_UNSUPPORTED_HEAD_DIMENSION, NULL, HEAD_DIM, (int64_t)head_dim, 0, 0);
    if (page_size != PAGE_SIZE)
        return fail(err, LO_UNSUPPORTED_PAGE_SIZE, NULL, PAGE_SIZE, (int64_t)page_size, 0, 0);
    if (qh % kvh != 0)
        return fail(err, LO_INVALID_HEAD_MAPPING, NULL, (int64_t)qh, (int64_t)kvh, 0, 0);
    if (nnz_qo > (size_t)INT32_MAX) return fail(err, LO_ELEMENT_COUNT_OVERFLOW, NULL, 0, 0, 0, 0);
    size_t t;
    if (batch + 1 < batch || mul_overflow(nnz_qo, qh, &t) || mul_overflow(t, head_dim, &t))
        return fail(err, LO_ELEMENT_COUNT_OVERFLOW, NULL, 0, 0, 0, 0);
    if (mul_overflow(max_pages, page_size, &t) || mul_overflow(t, kvh, &t) ||
        mul_overflow(t, head_dim, &t))
        return fail(err, LO_ELEMENT_COUNT_OVERFLOW, NULL, 0, 0, 0, 0);
    spec->batch_size = batch;
    spec->nnz_qo = nnz_qo;
    spec->max_num_pages = max_pages;
    spec->num_query_heads = qh;
    spec->num_kv_heads = kvh;
    return LO_OK;
}

/* paged_prefill/mod.rs:238-266 */
static int validate_query_indptr(const int32_t *indptr, size_t len, size_t expected_total,
                                 lo_error *err) {
    if (indptr[0] != 0) return fail(err, LO_INVALID_INDPTR_START, "qo_indptr", indptr[0], 0, 0, 0);
    for (size_t request = 0; request + 1 < len; ++request) {
        const int32_t start = indptr[request], end = indptr[request + 1];
        if (end < start)
            return fail(err, LO_NON_MONOTONIC_INDPTR, "qo_indptr", (int64_t)request, start, end, 0);
        if (end == start)
            return fail(err, LO_EMPTY_RAGGED_REQUEST, "qo_indptr", (int64_t)request, 0, 0, 0);
    }
    if (indptr[len - 1] < 0) return fail(err, LO_ELEMENT_COUNT_OVERFLOW, NULL, 0, 0, 0, 0);
    return require_len(err, "qo_indptr", (size_t)indptr[len - 1], expected_total);
}

/* paged_prefill/mod.rs:161-235 */
int lo_prefill_validate_metadata(const lo_prefill_spec *spec, const int32_t *qo_indptr,
                                 size_t qo_indptr_len, const int32_t *page_indptr,
                                 size_t page_indptr_len, const int32_t *indices,
                                 size_t indices_len, const int32_t *last, size_t last_len,
                                 lo_error *err) {
    int rc;
    const size_t batch = spec->batch_size;
    if ((rc = require_len(err, "qo_indptr", qo_indptr_len, batch + 1))) return rc;
    if ((rc = require_len(err, "page_indptr", page_indptr_len, batch + 1))) return rc;
    if ((rc = require_len(err, "last_page_len", last_len, batch))) return rc;
    if ((rc = validate_query_indptr(qo_indptr, qo_indptr_len, spec->nnz_qo, err))) return rc;
    if (page_indptr[0] != 0)
        return fail(err, LO_INVALID_PAGE_INDPTR_START, NULL, page_indptr[0], 0, 0, 0);
    for (size_t request = 0; request < batch; ++request) {
        const int32_t start = page_indptr[request], end = page_indptr[request + 1];
        if (end < start)
            return fail(err, LO_NON_MONOTONIC_PAGE_INDPTR, NULL, (int64_t)request, start, end, 0);
        if (end == start) return fail(err, LO_EMPTY_PAGED_REQUEST, NULL, (int64_t)request, 0, 0, 0);
        const int32_t tail = last[request];
        if (tail < 1 || tail > (int32_t)PAGE_SIZE)
            return fail(err, LO_INVALID_LAST_PAGE_LENGTH, NULL, (int64_t)request, tail, PAGE_SIZE,
                        0);
        const size_t qo_len = (size_t)(qo_indptr[request + 1] - qo_indptr[request]);
        const size_t kv_len = (size_t)(end - start - 1) * PAGE_SIZE + (size_t)tail;
        if (qo_len > kv_len)
            return fail(err, LO_RAGGED_QUERY_LONGER_THAN_KV, NULL, (int64_t)request,
                        (int64_t)qo_len, (int64_t)kv_len, 0);
    }
    if (page_indptr[batch] < 0) return fail(err, LO_ELEMENT_COUNT_OVERFLOW, NULL, 0, 0, 0, 0);
    if ((rc = require_len(err, "page_indices", indices_len, (size_t)page_indptr[batch]))) return rc;
    for (size_t position = 0; position < indices_len; ++position) {
        const int32_t index = indices[position];
        if (index < 0 || (size_t)index >= spec->max_num_pages)
            return fail(err, LO_PAGE_INDEX_OUT_OF_RANGE, NULL, (int64_t)position, index,
                        (int64_t)spec->max_num_pages, 0);
    }
    return LO_OK;
}

/* paged_prefill/mod.rs:383-443: one (query row, query head); the row sees the logical tokens
 * [0, kv_len - qo_len + query_index] of its request (bottom-right aligned causal mask). */
static void paged_prefill_one(const lo_prefill_spec *spec, const uint16_t *q,
                              const uint16_t *k_pages, const uint16_t *v_pages,
                              const int32_t *page_indptr, const int32_t *indices, size_t request,
                              size_t causal_kv_end, size_t query_row, size_t query_head,
                              uint16_t *out, float *lse) {
    const size_t qh = spec->num_query_heads, kvh = spec->num_kv_heads;
    const float scale = 1.0f / sqrtf((float)HEAD_DIM);
    const size_t query_offset = (query_row * qh + query_head) * HEAD_DIM;
    const size_t kv_head = query_head / (qh / kvh);
    float query[HEAD_DIM], state[HEAD_DIM];
    for (size_t c = 0; c < HEAD_DIM; ++c) query[c] = lo_bf16_to_f32(q[query_offset + c]);
    memset(state, 0, sizeof(state));
    float max_score = 0.0f, normalizer = 0.0f;
    for (size_t token = 0; token < causal_kv_end; ++token) {
        size_t page, offset;
        physical_slot(page_indptr, indices, request, token, &page, &offset);
        const size_t kv_offset = ((page * PAGE_SIZE + offset) * kvh + kv_head) * HEAD_DIM;
        float dot = 0.0f;
        for (size_t c = 0; c < HEAD_DIM; ++c)
            dot = fmaf(query[c], lo_bf16_to_f32(k_pages[kv_offset + c]), dot);
        const float score = dot * scale;
        if (token == 0) {
            max_score = score;
            normalizer = 1.0f;
            for (size_t c = 0; c < HEAD_DIM; ++c) state[c] = lo_bf16_to_f32(v_pages[kv_offset + c]);
            continue;
        }
        const float next_max = fmaxf(max_score, score);
        const float previous_weight = expf(max_score - next_max);
        const float current_weight = expf(score - next_max);
        normalizer = normalizer * previous_weight + current_weight;
        for (size_t c = 0; c < HEAD_DIM; ++c)
            state[c] = state[c] * previous_weight +
                       lo_bf16_to_f32(v_pages[kv_offset + c]) * current_weight;
        max_score = next_max;
    }
    for (size_t c = 0; c < HEAD_DIM; ++c)
        out[query_offset + c] = lo_bf16_from_f32(state[c] / normalizer);
    lse[query_row * qh + query_head] = (max_score + logf(normalizer)) * LOG2_E_F32;
}

struct prefill_job {
    const lo_prefill_spec *spec;
    const uint16_t *q, *k_pages, *v_pages;
    const int32_t *qo_indptr, *page_indptr, *indices, *last;
    uint16_t *out;
    float *lse;
    size_t rows;
    size_t next; /* query rows, claimed with an atomic fetch-add */
};

static void *prefill_worker(void *arg) {
    struct prefill_job *job = (struct prefill_job *)arg;
    const size_t batch = job->spec->batch_size;
    for (;;) {
        const size_t row = __atomic_fetch_add(&job->next, 1, __ATOMIC_RELAXED);
        if (row >= job->rows) break;
        size_t request = 0;
        while (request + 1 < batch && (size_t)job->qo_indptr[request + 1] <= row) ++request;
        const size_t qo_start = (size_t)job->qo_indptr[request];
        const size_t qo_len = (size_t)job->qo_indptr[request + 1] - qo_start;
        const size_t kv_len = request_kv_len(job->page_indptr, job->last, request);
        const size_t causal_kv_end = kv_len - qo_len + (row - qo_start) + 1; /* mod.rs:321-329 */
        for (size_t head = 0; head < job->spec->num_query_heads; ++head)
            paged_prefill_one(job->spec, job->q, job->k_pages, job->v_pages, job->page_indptr,
                              job->indices, request, causal_kv_end, row, head, job->out, job->lse);
    }
    return NULL;
}

/* paged_prefill/mod.rs:361-446.  threads > 1 distributes query rows over POSIX threads; every
 * (row, head) keeps the reference's arithmetic order, so results are identical. */
int lo_paged_prefill_ref(const lo_prefill_spec *spec, const uint16_t *q, size_t q_len,
                         const uint16_t *k_pages, size_t k_len, const uint16_t *v_pages,
                         size_t v_len, const int32_t *qo_indptr, size_t qo_indptr_len,
                         const int32_t *page_indptr, size_t page_indptr_len,
                         const int32_t *indices, size_t indices_len, const int32_t *last,
                         size_t last_len, uint16_t *out, size_t out_len, float *lse,
                         size_t lse_len, int threads, lo_error *err) {
    int rc;
    const size_t q_numel = spec->nnz_qo * spec->num_query_heads * HEAD_DIM;
    const size_t kv_numel = spec->max_num_pages * PAGE_SIZE * spec->num_kv_heads * HEAD_DIM;
    if ((rc = require_len(err, "Q", q_len, q_numel))) return rc;
    if ((rc = require_len(err, "K_pages", k_len, kv_numel))) return rc;
    if ((rc = require_len(err, "V_pages", v_len, kv_numel))) return rc;
    if ((rc = require_len(err, "O", out_len, q_numel))) return rc;
    if ((rc = require_len(err, "LSE", lse_len, spec->nnz_qo * spec->num_query_heads))) return rc;
    if ((rc = lo_prefill_validate_metadata(spec, qo_indptr, qo_indptr_len, page_indptr,
                                           page_indptr_len, indices, indices_len, last, last_len,
                                           err)))
        return rc;
    struct prefill_job job = {spec, q, k_pages, v_pages, qo_indptr, page_indptr, indices, last,
                              out, lse, spec->nnz_qo, 0};
    if (threads <= 1) {
        prefill_worker(&job);
        return LO_OK;
    }
    if (threads > 256) threads = 256;
    pthread_t workers[256];
    int started = 0;
    for (int t = 0; t < threads - 1; ++t)
        if (pthread_create(&workers[started], NULL, prefill_worker, &job) == 0) ++started;
    prefill_worker(&job);
    for (int t = 0; t < started; ++t) pthread_join(workers[t], NULL);
    return LO_OK;
}
