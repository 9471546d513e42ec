/*
 * CPU oracle for the Loom Infer paged-decode hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's CPU references, used as the
 * checker by the test-suite, the smoke entry and the CPU-baseline leg of the
 * benchmark.  It is never linked into, loaded by, or called from the product
 * library.  Each function cites the reference source it follows (paths are
 * relative to the reference project root).
 *
 * Parity status: PINNED.  The restatement reproduces the digests the reference
 * published for its own CPU references (see tests/golden/reference_digests.json).
 * Paged prefill has no published CPU-side digest; it is pinned by the known-answer
 * cases of the reference's unit tests, by the published fixture digests, by bit
 * equality with the digest-pinned paged decode where the operators coincide, and by
 * the published digests of the reference's DEVICE outputs, which the restatement
 * reproduces up to exactly the published number of differing elements
 * (tests/test_oracle_prefill.py).
 *
 * Build with -O2 -ffp-contract=off: the reference only fuses multiply-add where
 * it writes mul_add explicitly (the Q.K dot product).
 */
#ifndef LOOM_ORACLE_H
#define LOOM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Mirrors ContractError, crates/loom-infer/src/error.rs:6-109 (same order). */
enum lo_status {
    LO_OK = 0,
    LO_ZERO_DIMENSION,
    LO_ELEMENT_COUNT_OVERFLOW,
    LO_INVALID_EPSILON,
    LO_UNSUPPORTED_HEAD_DIMENSION,
    LO_UNSUPPORTED_PAGE_SIZE,
    LO_INVALID_HEAD_MAPPING,
    LO_INVALID_PARTITION_COUNT,
    LO_INVALID_INDPTR_START,
    LO_NON_MONOTONIC_INDPTR,
    LO_EMPTY_RAGGED_REQUEST,
    LO_RAGGED_QUERY_LONGER_THAN_KV,
    LO_INVALID_PAGE_INDPTR_START,
    LO_NON_MONOTONIC_PAGE_INDPTR,
    LO_EMPTY_PAGED_REQUEST,
    LO_PAGE_INDEX_OUT_OF_RANGE,
    LO_INVALID_LAST_PAGE_LENGTH,
    LO_INVALID_ROTARY_DIMENSION,
    LO_INVALID_ROPE_SCALE,
    LO_INVALID_ROPE_THETA,
    LO_NEGATIVE_POSITION_ID,
    LO_UNSUPPORTED_APPEND_TOKEN_COUNT,
    LO_APPEND_BATCH_INDEX_OUT_OF_RANGE,
    LO_APPEND_POSITION_OUT_OF_RANGE,
    LO_DUPLICATE_PAGE_APPEND_SLOT,
    LO_DUPLICATE_PAGE_APPEND_TOKEN_SLOT,
    LO_UNSUPPORTED_DTYPE,
    LO_LENGTH_MISMATCH
};

/* Payload of the error variant; field use follows the variant's field order. */
typedef struct lo_error {
    int32_t code;
    char buffer[24]; /* LengthMismatch.buffer */
    int64_t a, b, c, d;
} lo_error;

typedef struct lo_paged_spec {
    size_t batch_size, max_num_pages, num_query_heads, num_kv_heads;
} lo_paged_spec;

uint16_t lo_bf16_from_f32(float value);
float lo_bf16_to_f32(uint16_t bits);
void lo_fixture_bf16(uint16_t *out, size_t len, uint64_t salt);
uint64_t lo_digest_u16(const uint16_t *values, size_t len);
uint64_t lo_digest_u32(const uint32_t *values, size_t len);

int lo_paged_spec_new(size_t batch, size_t max_pages, size_t qh, size_t kvh, size_t head_dim,
                      size_t page_size, lo_paged_spec *spec, lo_error *err);
int lo_validate_page_table(const lo_paged_spec *spec, const int32_t *indptr, size_t indptr_len,
                           const int32_t *indices, size_t indices_len, const int32_t *last,
                           size_t last_len, lo_error *err);
int lo_append_validate_page_table(const lo_paged_spec *spec, const int32_t *indptr,
                                  size_t indptr_len, const int32_t *indices, size_t indices_len,
                                  const int32_t *last, size_t last_len, lo_error *err);
int lo_append_tokens_validate(const lo_paged_spec *spec, size_t tokens, size_t max_tokens,
                              const int32_t *batch_indices, size_t batch_indices_len,
                              const int32_t *positions, size_t positions_len,
                              const int32_t *indptr, size_t indptr_len, const int32_t *indices,
                              size_t indices_len, const int32_t *last, size_t last_len,
                              int64_t *slots_out /* tokens*2: page, offset */, lo_error *err);

int lo_paged_decode_ref(const lo_paged_spec *spec, const uint16_t *q, size_t q_len,
                        const uint16_t *k_pages, size_t k_len, const uint16_t *v_pages,
                        size_t v_len, const int32_t *indptr, size_t indptr_len,
                        const int32_t *indices, size_t indices_len, const int32_t *last,
                        size_t last_len, uint16_t *out, size_t out_len, float *lse,
                        size_t lse_len, int threads, lo_error *err);

int lo_single_decode_ref(size_t kv_len, size_t qh, size_t kvh, const uint16_t *q,
                         const uint16_t *k, const uint16_t *v, uint16_t *out, float *lse,
                         lo_error *err);
int lo_split_k_partition_range(size_t kv_len, size_t partitions, size_t partition, size_t *start,
                               size_t *end);
int lo_split_k_partials_ref(size_t kv_len, size_t qh, size_t kvh, size_t partitions,
                            const uint16_t *q, const uint16_t *k, const uint16_t *v,
                            float *workspace, size_t workspace_len, lo_error *err);
int lo_split_k_merge_ref(size_t qh, size_t partitions, const float *workspace,
                         size_t workspace_len, uint16_t *out, float *lse, lo_error *err);

int lo_paged_split_k_partials_ref(const lo_paged_spec *spec, size_t partitions,
                                  const uint16_t *q, const uint16_t *k_pages,
                                  const uint16_t *v_pages, const int32_t *indptr,
                                  const int32_t *indices, size_t indices_len,
                                  const int32_t *last, float *workspace, lo_error *err);
int lo_paged_split_k_merge_ref(const lo_paged_spec *spec, size_t partitions,
                               const float *workspace, uint16_t *out, float *lse);

int lo_rope_ref(size_t tokens, size_t qh, size_t kh, size_t head_dim, size_t rotary_dim,
                float rope_scale, float rope_theta, const uint16_t *q, size_t q_len,
                const uint16_t *k, size_t k_len, const int32_t *positions, size_t pos_len,
                uint16_t *q_out, size_t q_out_len, uint16_t *k_out, size_t k_out_len,
                lo_error *err);
int lo_rope_append_ref(const lo_paged_spec *spec, const uint16_t *q, size_t q_len,
                       const uint16_t *k, size_t k_len, const uint16_t *v, size_t v_len,
                       const int32_t *indptr, size_t indptr_len, const int32_t *indices,
                       size_t indices_len, const int32_t *last, size_t last_len, uint16_t *q_out,
                       size_t q_out_len, uint16_t *k_pages, size_t k_pages_len,
                       uint16_t *v_pages, size_t v_pages_len, lo_error *err);
int lo_rope_append_tokens_ref(const lo_paged_spec *spec, size_t tokens, size_t max_tokens,
                              const uint16_t *q, size_t q_len, const uint16_t *k, size_t k_len,
                              const uint16_t *v, size_t v_len, const int32_t *batch_indices,
                              size_t batch_indices_len, const int32_t *positions,
                              size_t positions_len, const int32_t *indptr, size_t indptr_len,
                              const int32_t *indices, size_t indices_len, const int32_t *last,
                              size_t last_len, uint16_t *q_out, size_t q_out_len,
                              uint16_t *k_pages, size_t k_pages_len, uint16_t *v_pages,
                              size_t v_pages_len, lo_error *err);

/* Paged causal prefill, crates/loom-infer/src/attention/paged_prefill/mod.rs:19-27. */
typedef struct lo_prefill_spec {
    size_t batch_size, nnz_qo, max_num_pages, num_query_heads, num_kv_heads;
} lo_prefill_spec;

int lo_prefill_spec_new(size_t batch, size_t nnz_qo, size_t max_pages, size_t qh, size_t kvh,
                        size_t head_dim, size_t page_size, lo_prefill_spec *spec, lo_error *err);
int lo_prefill_validate_metadata(const lo_prefill_spec *spec, const int32_t *qo_indptr,
                                 size_t qo_indptr_len, const int32_t *page_indptr,
                                 size_t page_indptr_len, const int32_t *indices,
                                 size_t indices_len, const int32_t *last, size_t last_len,
                                 lo_error *err);
int lo_paged_prefill_ref(const lo_prefill_spec *spec, const uint16_t *q, size_t q_len,
                         const uint16_t *k_pages, size_t k_len, const uint16_t *v_pages,
                         size_t v_len, const int32_t *qo_indptr, size_t qo_indptr_len,
                         const int32_t *page_indptr, size_t page_indptr_len,
                         const int32_t *indices, size_t indices_len, const int32_t *last,
                         size_t last_len, uint16_t *out, size_t out_len, float *lse,
                         size_t lse_len, int threads, lo_error *err);

#ifdef __cplusplus
}
#endif
#endif
