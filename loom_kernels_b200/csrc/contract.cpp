// Host-side contract: validated specs, page-table and append metadata validation, split-K
// partition rule, and the plan-time launch heuristic.  Pure functions; no CUDA.
//
// Follows crates/loom-infer/src/attention/paged_decode/mod.rs:26-279,
// crates/loom-infer/src/attention/paged_append/mod.rs:95-131,144-177,244-317 and
// crates/loom-infer/src/attention/single_decode/mod.rs:131-194 of the reference.
#include <cmath>
#include <vector>

#include "runtime.hpp"

namespace lb {
namespace {

bool mul_overflow(size_t a, size_t b, size_t *out) { return __builtin_mul_overflow(a, b, out); }

lb_status require_len(const char *buffer, size_t actual, size_t expected) {
    if (actual == expected) return LB_OK;
    return fail(LB_LENGTH_MISMATCH, buffer, (int64_t)expected, (int64_t)actual);
}

size_t kv_len_of(const int32_t *indptr, const int32_t *last, size_t request) {
    const size_t pages = (size_t)(indptr[request + 1] - indptr[request]);
    return (pages - 1) * LB_PAGE_SIZE + (size_t)last[request];
}

uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

} // namespace

// Plan-time choice of the decode algorithm and launch shape.  Inputs are the spec and the device
// only; the page table is not known when a plan is made.
//
//   q_tiles (MT)      16-row MMA tiles that cover the GQA group, a power of two <= warps
//   q_blocks          CTAs per KV head when the group exceeds 16*MT rows
//   units             warps / MT (page, KV head) tiles one pipeline stage holds
//   heads_per_cta     KV heads one CTA streams (divides kv_heads and units)
//   pages_per_stage   units / heads_per_cta
//   algorithm         direct (1 chunk, 1 command) | split-K (caller-pinned chunks per request)
//                     | balanced (the batch's pages cut evenly over one CTA per SM)
lb_status choose_decode(const lb_paged_spec &spec, uint32_t sm_count, size_t smem_optin,
                        const lb_paged_decode_options *options, DecodeChoice *out) {
    const uint32_t warps = 8;
    const uint32_t sms = sm_count ? sm_count : 148;
    const size_t smem = smem_optin ? smem_optin : 232448;
    const size_t group = spec.num_query_heads / spec.num_kv_heads;
    size_t states;
    if (mul_overflow(spec.batch_size, spec.num_query_heads, &states))
        return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, INT64_MAX);
    if (states > 0x7fffffffu) return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)states);

    uint32_t q_tiles = 1;
    while (q_tiles < warps && (size_t)q_tiles * 16 < group) q_tiles *= 2;
    const uint32_t q_blocks = (uint32_t)((group + (size_t)q_tiles * 16 - 1) / ((size_t)q_tiles * 16));
    const uint32_t units = warps / q_tiles;
    const uint32_t stage_bytes = units * 8192u;

    // heads per CTA: powers of two dividing both kv_heads and units
    auto valid_hc = [&](uint32_t hc) {
        return hc >= 1 && hc <= units && units % hc == 0 && spec.num_kv_heads % hc == 0;
    };
    uint32_t partitions = options ? options->partitions : 0;
    uint32_t hc = options ? options->heads_per_cta : 0;
    const uint32_t balanced_option = options ? options->balanced : 0;
    if (hc != 0 && !valid_hc(hc)) return fail(LB_LAUNCH_CONTRACT, "heads_per_cta", hc);
    if (balanced_option > 2) return fail(LB_LAUNCH_CONTRACT, "balanced", balanced_option);

    auto items_for = [&](uint32_t h, uint32_t p) -> size_t {
        return spec.batch_size * (spec.num_kv_heads / h) * q_blocks * (size_t)p;
    };
    // Relative cost of a direct / split candidate.  Measured on B200: the HBM ceiling for
    // scattered pages is ~6.5 TB/s; one SM pulls ~80 GB/s through 32 KB TMA boxes (8 heads per
    // CTA) but only ~45 GB/s through 4 KB boxes (1 head); the rates below are what the whole
    // kernel sustains per CTA.  A launch takes max(bytes / HBM, waves * bytes_per_cta / rate).
    auto cost_of = [&](uint32_t h, uint32_t p) -> double {
        const double n = (double)items_for(h, p);
        const double rate = h >= 8 ? 66.0 : h >= 4 ? 60.0 : h >= 2 ? 50.0 : 42.0; // GB/s per CTA
        const double waves = std::ceil(n / sms);
        const double hbm_time = 1.0 / 6500.0;
        const double cta_time = waves / (n * rate);
        double cost = hbm_time > cta_time ? hbm_time : cta_time;
        cost *= 1.0 + 0.01 * (waves - 1.0); // each extra wave adds a fill/drain bubble
        if (p > 1) cost *= 1.04;            // workspace round trip + merge launch
        return cost;
    };

    // The balanced algorithm keeps the page prefix of every request in shared memory and packs
    // (page id, head block) pairs, which bounds what it accepts.
    const uint32_t widest_hc = [&] {
        for (uint32_t h = units; h >= 1; h /= 2)
            if (valid_hc(h)) return h;
        return 1u;
    }();
    const uint32_t balanced_hc = hc ? hc : widest_hc;
    const size_t balanced_extra = (3 * spec.batch_size + 2) * sizeof(int32_t);
    const bool balanced_possible =
        spec.batch_size <= 1024 && spec.max_num_pages < (1u << 23) &&
        (spec.num_kv_heads / balanced_hc) * q_blocks <= 4096 &&
        2 * stage_bytes + 3072 + balanced_extra <= smem;

    const uint32_t merge_option = options ? options->merge_in_kernel : 0;
    if (merge_option > 2) return fail(LB_LAUNCH_CONTRACT, "merge_in_kernel", merge_option);
    const bool cluster_option = options && options->cluster == 1;
    if (options && options->cluster > 1) return fail(LB_LAUNCH_CONTRACT, "cluster", options->cluster);
    if (cluster_option && (partitions < 2 || partitions > 8))
        return fail(LB_INVALID_PARTITION_COUNT, nullptr, partitions, 8);
    bool cluster = cluster_option;
    uint32_t algorithm;
    if (partitions == 1) {
        algorithm = LB_DECODE_DIRECT;
    } else if (partitions > 1) {
        algorithm = LB_DECODE_SPLIT_K;
    } else if (balanced_option == 1) {
        if (!balanced_possible) return fail(LB_LAUNCH_CONTRACT, "balanced", 1);
        algorithm = LB_DECODE_BALANCED;
    } else {
        // Direct wins when whole (request, head block) items already tile the device: no merge
        // launch, no workspace.  That needs many more items than SMs, because requests of one
        // batch differ in length.  Otherwise cut by pages.
        // A pool of at most 64 pages (1024 tokens in all) has nothing to balance either: such
        // calls are launch-latency bound and a second launch would only add to it.
        const size_t direct_items = items_for(widest_hc, 1);
        const bool plenty = direct_items >= 8 * (size_t)sms || spec.max_num_pages <= 64;
        if (plenty) {
            algorithm = LB_DECODE_DIRECT;
        } else if (spec.batch_size == 1 &&
                   spec.max_num_pages * spec.num_kv_heads <= 64 * (size_t)sms) {
            // One short request (at most 64 page-heads per SM even if it fills the pool) has
            // nothing ragged to balance, and such calls are latency-bound: a
            // static split into about half a wave of CTAs (fewer, longer chunks beat more states
            // to merge; measured on MHA 32/32 at context 1024: 8 chunks x 8 head blocks 12.5 us,
            // 16 chunks 14.9 us, balanced 21.7 us), two page slots per CTA where the heads allow.
            uint32_t h = hc;
            if (h == 0) {
                h = units >= 2 ? units / 2 : 1;
                while (h > 1 && !valid_hc(h)) h /= 2;
            }
            size_t limit = spec.max_num_pages / 8; // >= 8 pages a chunk if the pool is one request
            if (limit > 64) limit = 64;
            size_t p = (sms / 2) / items_for(h, 1);
            if (p > limit) p = limit;
            if (p < 1) p = 1;
            // up to eight chunks fit one thread-block cluster, which merges them through
            // distributed shared memory: one command instead of two (C1: 8.2 -> see the
            // measurement notes), so the count is capped there
            if (p > 8) p = 8;
            hc = h;
            partitions = (uint32_t)p;
            algorithm = p > 1 ? LB_DECODE_SPLIT_K : LB_DECODE_DIRECT;
            cluster = p > 1;
        } else if (balanced_possible && balanced_option != 2) algorithm = LB_DECODE_BALANCED;
        else algorithm = LB_DECODE_SPLIT_K; // best static split below (may come out as 1 chunk)
    }

    if (algorithm == LB_DECODE_BALANCED) {
        hc = balanced_hc;
        partitions = 1;
    } else {
        size_t max_partitions = (spec.max_num_pages / spec.batch_size) / 8; // >= 8 pages a chunk
        if (max_partitions < 1) max_partitions = 1;
        if (max_partitions > 64) max_partitions = 64;
        const bool choose_p = partitions == 0;
        if (algorithm == LB_DECODE_DIRECT && choose_p) partitions = 1;
        const bool sweep_p = choose_p && algorithm == LB_DECODE_SPLIT_K;
        if (hc == 0 || sweep_p) {
            double best = 0.0;
            uint32_t best_hc = 0, best_p = 0;
            for (uint32_t h = units; h >= 1; h /= 2) {
                if (!valid_hc(h) || (hc != 0 && h != hc)) continue;
                const uint32_t p_lo = sweep_p ? 1 : partitions;
                const uint32_t p_hi = sweep_p ? (uint32_t)max_partitions : partitions;
                for (uint32_t p = p_lo; p <= p_hi; ++p) {
                    const double cost = cost_of(h, p);
                    if (best_hc == 0 || cost < best * 0.999) {
                        best = cost;
                        best_hc = h;
                        best_p = p;
                    }
                }
            }
            hc = best_hc;
            partitions = best_p;
        }
        algorithm = partitions > 1 ? LB_DECODE_SPLIT_K : LB_DECODE_DIRECT;
        if (partitions > spec.max_num_pages)
            return fail(LB_INVALID_PARTITION_COUNT, nullptr, partitions,
                        (int64_t)spec.max_num_pages);
    }

    const uint32_t pps = units / hc;
    size_t extra = 3072; // alignment slack, barriers, flags
    if (algorithm == LB_DECODE_BALANCED) extra += balanced_extra;
    uint32_t stages = (uint32_t)((smem - extra) / stage_bytes);
    if (stages > 6) stages = 6;
    // A balanced plan with one KV head per CTA (4 KB boxes, a producer warp per page slot) keeps
    // four stages = 128 KB in flight per SM: scattered 4 KB reads stream best with about 100 KB
    // in flight (a probe: 6.5 TB/s with 96 KB, 6.0 with 192 KB), and the kernel measured 108.3 us
    // on the ragged MQA batch with four stages against 109.8 with six (111.2 with three).
    if (algorithm == LB_DECODE_BALANCED && hc == 1 && pps > 1 && pps <= 4 && stages > 4 &&
        !(options && (options->producer_warps == 1 || options->max_stages != 0)))
        stages = 4;
    if (options && options->max_stages >= 2 && stages > options->max_stages)
        stages = options->max_stages;
    // direct/split CTAs merge their warps' states in the ring: 8 warps x 68 x 32 floats
    if (stages < 2 || (algorithm != LB_DECODE_BALANCED && pps > 1 &&
                       (size_t)stages * stage_bytes < 8u * 68u * 32u * 4u))
        return fail(LB_LAUNCH_CONTRACT, "shared_memory", (int64_t)smem);

    if (cluster && algorithm == LB_DECODE_SPLIT_K) {
        // the chunk states of a CTA sit in the ring beyond the scratch of its slot merge
        const size_t rows = group < 16u * q_tiles ? group : 16u * q_tiles;
        const size_t needed = 8u * 68u * 32u * 4u + (size_t)hc * 16u * q_tiles * 520u;
        (void)rows;
        if ((size_t)stages * stage_bytes >= needed) algorithm = LB_DECODE_CLUSTER_SPLIT;
        else if (cluster_option) return fail(LB_LAUNCH_CONTRACT, "cluster", (int64_t)needed);
    }
    size_t grid, workspace = 0;
    if (algorithm == LB_DECODE_BALANCED) {
        grid = options && options->balanced_ctas ? options->balanced_ctas : sms;
        if (grid > sms) grid = sms; // workers share nothing, but one CTA per SM is the design
        const size_t workers = grid * pps;
        const size_t rows = group < 16u * q_tiles ? group : 16u * q_tiles;
        // states, then the page prefix (batch + 1 ints) and the cut the merge kernel reuses
        workspace = workers * 2 * hc * rows * LB_PARTIAL_STATE_WIDTH + spec.batch_size + 8;
    } else {
        grid = items_for(hc, partitions);
        if (grid > 0x7fffffffu) return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)grid);
        if (partitions > 1 && algorithm != LB_DECODE_CLUSTER_SPLIT) {
            if (mul_overflow(states, partitions, &workspace) ||
                mul_overflow(workspace, LB_PARTIAL_STATE_WIDTH, &workspace) ||
                workspace > SIZE_MAX / sizeof(float))
                return fail(LB_ELEMENT_COUNT_OVERFLOW);
        }
    }

    // Balanced plans whose boxes are small (one KV head per CTA: 4 KB) give every page slot a
    // producer warp of its own; the others keep one.
    uint32_t producer_warps = 1;
    const uint32_t producer_option = options ? options->producer_warps : 0;
    if (producer_option > 1 && (algorithm != LB_DECODE_BALANCED || producer_option != pps))
        return fail(LB_LAUNCH_CONTRACT, "producer_warps", producer_option);
    if (algorithm == LB_DECODE_BALANCED && pps > 1 && pps <= 4 &&
        (producer_option == pps || (producer_option == 0 && hc == 1)))
        producer_warps = pps;
    // On request a static split is merged inside its own kernel: every chunk counts itself on a
    // word of the queue and the last one of an item merges it.  One command instead of two, at
    // no gain in time -- the tail of the last CTAs is as long as a merge kernel that starts under
    // programmatic dependent launch (C1 8.9 against 8.6 us per Graph node), and a large plan
    // loses the parallel merge (C4 split 16: 179.9 against 163.8 us) -- so the plan never
    // chooses it by itself.
    uint32_t merged_in_kernel = 0;
    if (algorithm == LB_DECODE_SPLIT_K) {
        const bool fits = grid / partitions <= kQueueSyncWords;
        if (merge_option == 1 && !fits)
            return fail(LB_LAUNCH_CONTRACT, "merge_in_kernel", (int64_t)(grid / partitions));
        merged_in_kernel = merge_option == 1 ? 1 : 0;
    } else if (algorithm == LB_DECODE_BALANCED) {
        // On request a balanced plan merges its cut items in the decode kernel: the warp that
        // counts the last state of an item merges the rows of its tile and publishes them.  The
        // plan does not choose it either: a warp that merges stalls its page slot, and on ragged
        // MQA (32 rows per item) the kernel went from 110 to 143 us; C3 and ragged GQA4 were
        // unchanged (172 / 527 us).  It needs a word of the queue per (item, KV head, row tile).
        const size_t words =
            spec.batch_size * (spec.num_kv_heads / hc) * q_blocks * (size_t)hc * q_tiles;
        if (merge_option == 1 && words > kQueueSyncWords)
            return fail(LB_LAUNCH_CONTRACT, "merge_in_kernel", (int64_t)words);
        merged_in_kernel = merge_option == 1 ? 1 : 0;
    } else if (merge_option == 1) {
        return fail(LB_LAUNCH_CONTRACT, "merge_in_kernel", 1);
    }
    out->merged_in_kernel = merged_in_kernel;
    out->algorithm = algorithm;
    out->partitions = partitions;
    out->heads_per_cta = hc;
    out->q_tiles = q_tiles;
    out->q_blocks = q_blocks;
    out->pages_per_stage = pps;
    out->stages = stages;
    out->warps = warps;
    out->grid = (uint32_t)grid;
    out->producer_warps = producer_warps;
    out->block = (warps + producer_warps) * 32;
    out->shared_bytes = (uint32_t)(stages * stage_bytes + extra);
    out->merge_block = 128;
    // One warp per (request, query head), four items per CTA.  Where the balanced cut leaves many
    // states per item -- few requests on many workers: eight or more workers per (request, head
    // block) -- every item gets a whole CTA whose four warps share its states.  (With two or
    // three states per item that form only multiplies CTAs: C3 merged in 19 us instead of 7.)
    const bool many_states_per_item =
        algorithm == LB_DECODE_BALANCED && states <= 2048 &&
        (size_t)grid * pps >= 8 * spec.batch_size * (spec.num_kv_heads / hc) * q_blocks;
    out->merge_four_warps = many_states_per_item ? 1 : 0;
    out->merge_grid = algorithm == LB_DECODE_DIRECT || algorithm == LB_DECODE_CLUSTER_SPLIT ||
                              merged_in_kernel
                          ? 0
                      : many_states_per_item ? (uint32_t)states
                                             : ceil_div((uint32_t)states, 4);
    out->workspace_numel = workspace;
    return LB_OK;
}

} // namespace lb

using namespace lb;

extern "C" {

lb_status lb_paged_spec_new(size_t batch, size_t max_pages, size_t qh, size_t kvh, size_t head_dim,
                            size_t page_size, lb_paged_spec *out) {
    if (!out) return fail(LB_INVALID_ARGUMENT, "out");
    if (batch == 0 || max_pages == 0 || qh == 0 || kvh == 0 || head_dim == 0 || page_size == 0)
        return fail(LB_ZERO_DIMENSION);
    if (head_dim != LB_HEAD_DIM)
        return fail(LB_UNSUPPORTED_HEAD_DIMENSION, nullptr, LB_HEAD_DIM, (int64_t)head_dim);
    if (page_size != LB_PAGE_SIZE)
        return fail(LB_UNSUPPORTED_PAGE_SIZE, nullptr, LB_PAGE_SIZE, (int64_t)page_size);
    if (qh % kvh != 0) return fail(LB_INVALID_HEAD_MAPPING, nullptr, (int64_t)qh, (int64_t)kvh);
    size_t t;
    if (batch + 1 < batch || mul_overflow(batch, qh, &t) || mul_overflow(t, head_dim, &t))
        return fail(LB_ELEMENT_COUNT_OVERFLOW);
    if (mul_overflow(max_pages, page_size, &t) || mul_overflow(t, kvh, &t) ||
        mul_overflow(t, head_dim, &t))
        return fail(LB_ELEMENT_COUNT_OVERFLOW);
    out->batch_size = batch;
    out->max_num_pages = max_pages;
    out->num_query_heads = qh;
    out->num_kv_heads = kvh;
    out->softmax_scale = 1.0f / std::sqrt((float)head_dim);
    return LB_OK;
}

size_t lb_paged_spec_query_numel(const lb_paged_spec *s) {
    return s->batch_size * s->num_query_heads * LB_HEAD_DIM;
}
size_t lb_paged_spec_kv_pages_numel(const lb_paged_spec *s) {
    return s->max_num_pages * LB_PAGE_SIZE * s->num_kv_heads * LB_HEAD_DIM;
}
size_t lb_paged_spec_lse_numel(const lb_paged_spec *s) {
    return s->batch_size * s->num_query_heads;
}
size_t lb_paged_spec_gqa_group_size(const lb_paged_spec *s) {
    return s->num_query_heads / s->num_kv_heads;
}
int64_t lb_paged_spec_kv_head_for_query_head(const lb_paged_spec *s, size_t query_head) {
    if (query_head >= s->num_query_heads) return -1;
    return (int64_t)(query_head / lb_paged_spec_gqa_group_size(s));
}

lb_status lb_paged_spec_validate_page_table(const lb_paged_spec *spec, const int32_t *indptr,
                                            size_t indptr_len, const int32_t *indices,
                                            size_t indices_len, const int32_t *last,
                                            size_t last_len) {
    if (!spec) return fail(LB_INVALID_ARGUMENT, "spec");
    lb_status rc;
    if ((rc = require_len("page_indptr", indptr_len, spec->batch_size + 1))) return rc;
    if ((rc = require_len("last_page_len", last_len, spec->batch_size))) return rc;
    if (!indptr || !last) return fail(LB_INVALID_ARGUMENT, "page table");
    if (indptr[0] != 0) return fail(LB_INVALID_PAGE_INDPTR_START, nullptr, indptr[0]);
    for (size_t request = 0; request < spec->batch_size; ++request) {
        const int32_t start = indptr[request], end = indptr[request + 1];
        if (end < start)
            return fail(LB_NON_MONOTONIC_PAGE_INDPTR, nullptr, (int64_t)request, start, end);
        if (end == start) return fail(LB_EMPTY_PAGED_REQUEST, nullptr, (int64_t)request);
        const int32_t length = last[request];
        if (length < 1 || length > (int32_t)LB_PAGE_SIZE)
            return fail(LB_INVALID_LAST_PAGE_LENGTH, nullptr, (int64_t)request, length,
                        LB_PAGE_SIZE);
    }
    if (indptr[spec->batch_size] < 0) return fail(LB_ELEMENT_COUNT_OVERFLOW);
    if ((rc = require_len("page_indices", indices_len, (size_t)indptr[spec->batch_size])))
        return rc;
    for (size_t position = 0; position < indices_len; ++position) {
        const int32_t index = indices[position];
        if (index < 0 || (size_t)index >= spec->max_num_pages)
            return fail(LB_PAGE_INDEX_OUT_OF_RANGE, nullptr, (int64_t)position, index,
                        (int64_t)spec->max_num_pages);
    }
    return LB_OK;
}

int lb_page_table_request_kv_len(const lb_paged_spec *spec, const int32_t *indptr,
                                 const int32_t *last, size_t request, size_t *kv_len) {
    if (request >= spec->batch_size) return 0;
    *kv_len = kv_len_of(indptr, last, request);
    return 1;
}

int lb_page_table_physical_page_for_token(const lb_paged_spec *spec, const int32_t *indptr,
                                          const int32_t *indices, const int32_t *last,
                                          size_t request, size_t token, size_t *page,
                                          size_t *offset) {
    if (request >= spec->batch_size) return 0;
    if (token >= kv_len_of(indptr, last, request)) return 0;
    *page = (size_t)indices[(size_t)indptr[request] + token / LB_PAGE_SIZE];
    *offset = token % LB_PAGE_SIZE;
    return 1;
}

lb_status lb_append_spec_validate_page_table(const lb_paged_spec *spec, const int32_t *indptr,
                                             size_t indptr_len, const int32_t *indices,
                                             size_t indices_len, const int32_t *last,
                                             size_t last_len) {
    lb_status rc = lb_paged_spec_validate_page_table(spec, indptr, indptr_len, indices,
                                                     indices_len, last, last_len);
    if (rc) return rc;
    std::vector<int64_t> slots(spec->batch_size);
    for (size_t request = 0; request < spec->batch_size; ++request) {
        size_t page, offset;
        lb_page_table_physical_page_for_token(spec, indptr, indices, last, request,
                                              kv_len_of(indptr, last, request) - 1, &page,
                                              &offset);
        slots[request] = (int64_t)(page * LB_PAGE_SIZE + offset);
    }
    // report the lexicographically first (first_request, second_request) pair, as the
    // reference's nested loops do
    for (size_t first = 0; first < spec->batch_size; ++first)
        for (size_t second = first + 1; second < spec->batch_size; ++second)
            if (slots[first] == slots[second])
                return fail(LB_DUPLICATE_PAGE_APPEND_SLOT, nullptr, (int64_t)first,
                            (int64_t)second, slots[first] / LB_PAGE_SIZE,
                            slots[first] % LB_PAGE_SIZE);
    return LB_OK;
}

size_t lb_append_extended_max_tokens(void) { return 16384; }

static lb_status tokens_spec(size_t tokens, size_t max_tokens, size_t batch, size_t max_pages,
                             size_t qh, size_t kvh, size_t head_dim, size_t page_size,
                             lb_append_tokens_spec *out) {
    if (!out) return fail(LB_INVALID_ARGUMENT, "out");
    if (tokens == 0) return fail(LB_ZERO_DIMENSION);
    if (tokens > max_tokens)
        return fail(LB_UNSUPPORTED_APPEND_TOKEN_COUNT, nullptr, (int64_t)max_tokens,
                    (int64_t)tokens);
    lb_status rc = lb_paged_spec_new(batch, max_pages, qh, kvh, head_dim, page_size, &out->paged);
    if (rc) return rc;
    size_t t;
    if (mul_overflow(tokens, qh, &t) || mul_overflow(t, head_dim, &t) ||
        mul_overflow(tokens, kvh, &t) || mul_overflow(t, head_dim, &t))
        return fail(LB_ELEMENT_COUNT_OVERFLOW);
    out->tokens = tokens;
    return LB_OK;
}

lb_status lb_append_tokens_spec_new(size_t tokens, size_t batch, size_t max_pages, size_t qh,
                                    size_t kvh, size_t head_dim, size_t page_size,
                                    lb_append_tokens_spec *out) {
    lb_status rc = tokens_spec(tokens, LB_APPEND_MAX_TOKENS, batch, max_pages, qh, kvh, head_dim,
                               page_size, out);
    if (rc == LB_OK) out->max_tokens = LB_APPEND_MAX_TOKENS;
    return rc;
}

lb_status lb_append_tokens_spec_new_extended(size_t tokens, size_t batch, size_t max_pages,
                                             size_t qh, size_t kvh, size_t head_dim,
                                             size_t page_size, lb_append_tokens_spec *out) {
    lb_status rc = tokens_spec(tokens, lb_append_extended_max_tokens(), batch, max_pages, qh, kvh,
                               head_dim, page_size, out);
    if (rc == LB_OK) out->max_tokens = 0;
    return rc;
}

lb_status lb_append_tokens_spec_validate_metadata(
    const lb_append_tokens_spec *spec, const int32_t *batch_indices, size_t batch_indices_len,
    const int32_t *positions, size_t positions_len, const int32_t *indptr, size_t indptr_len,
    const int32_t *indices, size_t indices_len, const int32_t *last, size_t last_len,
    int64_t *slots_out) {
    if (!spec) return fail(LB_INVALID_ARGUMENT, "spec");
    lb_status rc;
    if ((rc = require_len("batch_indices", batch_indices_len, spec->tokens))) return rc;
    if ((rc = require_len("positions", positions_len, spec->tokens))) return rc;
    if ((rc = lb_paged_spec_validate_page_table(&spec->paged, indptr, indptr_len, indices,
                                                indices_len, last, last_len)))
        return rc;
    std::vector<int64_t> slots(spec->tokens);
    for (size_t token = 0; token < spec->tokens; ++token) {
        const int32_t index = batch_indices[token];
        if (index < 0 || (size_t)index >= spec->paged.batch_size)
            return fail(LB_APPEND_BATCH_INDEX_OUT_OF_RANGE, nullptr, (int64_t)token, index,
                        (int64_t)spec->paged.batch_size);
        const size_t request = (size_t)index;
        const size_t kv_len = kv_len_of(indptr, last, request);
        const int32_t position = positions[token];
        if (position < 0 || (size_t)position >= kv_len)
            return fail(LB_APPEND_POSITION_OUT_OF_RANGE, nullptr, (int64_t)token, (int64_t)request,
                        position, (int64_t)kv_len);
        const size_t page = (size_t)indices[(size_t)indptr[request] + (size_t)position / LB_PAGE_SIZE];
        const int64_t slot = (int64_t)(page * LB_PAGE_SIZE + (size_t)position % LB_PAGE_SIZE);
        for (size_t first = 0; first < token; ++first)
            if (slots[first] == slot)
                return fail(LB_DUPLICATE_PAGE_APPEND_TOKEN_SLOT, nullptr, (int64_t)first,
                            (int64_t)token, slot / LB_PAGE_SIZE, slot % LB_PAGE_SIZE);
        slots[token] = slot;
    }
    if (slots_out)
        for (size_t token = 0; token < spec->tokens; ++token) {
            slots_out[token * 2] = slots[token] / LB_PAGE_SIZE;
            slots_out[token * 2 + 1] = slots[token] % LB_PAGE_SIZE;
        }
    return LB_OK;
}

int lb_split_partition_range(size_t length, size_t partitions, size_t partition, size_t *start,
                             size_t *end) {
    if (partitions == 0 || partition >= partitions) return 0;
    const size_t base = length / partitions, remainder = length % partitions;
    const size_t extra_before = partition < remainder ? partition : remainder;
    *start = partition * base + extra_before;
    *end = *start + base + (partition < remainder ? 1 : 0);
    return 1;
}

lb_status lb_paged_split_workspace_numel(const lb_paged_spec *spec, size_t partitions,
                                         size_t *numel) {
    if (!spec || !numel) return fail(LB_INVALID_ARGUMENT, "spec");
    if (partitions == 0 || partitions > spec->max_num_pages)
        return fail(LB_INVALID_PARTITION_COUNT, nullptr, (int64_t)partitions,
                    (int64_t)spec->max_num_pages);
    size_t t;
    if (mul_overflow(spec->batch_size, spec->num_query_heads, &t) ||
        mul_overflow(t, partitions, &t) || mul_overflow(t, LB_PARTIAL_STATE_WIDTH, &t) ||
        t > SIZE_MAX / sizeof(float))
        return fail(LB_ELEMENT_COUNT_OVERFLOW);
    *numel = t;
    return LB_OK;
}

int64_t lb_paged_split_state_offset(const lb_paged_spec *spec, size_t partitions, size_t request,
                                    size_t query_head, size_t partition) {
    if (request >= spec->batch_size || query_head >= spec->num_query_heads ||
        partition >= partitions)
        return -1;
    return (int64_t)(((request * spec->num_query_heads + query_head) * partitions + partition) *
                     LB_PARTIAL_STATE_WIDTH);
}

lb_status lb_paged_decode_choose(const lb_paged_spec *spec, uint32_t sm_count,
                                 const lb_paged_decode_options *options,
                                 lb_paged_decode_plan_info *info) {
    if (!spec || !info) return fail(LB_INVALID_ARGUMENT, "spec");
    DecodeChoice choice;
    lb_status rc = choose_decode(*spec, sm_count, 0, options, &choice);
    if (rc) return rc;
    info->algorithm = (int32_t)choice.algorithm;
    info->partitions = choice.partitions;
    info->heads_per_cta = choice.heads_per_cta;
    info->q_tiles = choice.q_tiles;
    info->q_blocks = choice.q_blocks;
    info->pages_per_stage = choice.pages_per_stage;
    info->stages = choice.stages;
    info->grid = choice.grid;
    info->block = choice.block;
    info->shared_bytes = choice.shared_bytes;
    info->merge_grid = choice.merge_grid;
    info->merge_block = choice.merge_block;
    info->commands = choice.algorithm == LB_DECODE_DIRECT ||
                             choice.algorithm == LB_DECODE_CLUSTER_SPLIT || choice.merged_in_kernel
                         ? 1
                         : 2;
    info->workspace_numel = choice.workspace_numel;
    info->workspace_bytes = choice.workspace_numel * sizeof(float);
    info->merged_in_kernel = choice.merged_in_kernel;
    info->reserved = 0;
    return LB_OK;
}

// Bf16RopePosIdsSpec::new, crates/loom-infer/src/rope/mod.rs:21-62 (same order of checks)
lb_status lb_rope_pos_ids_spec_new(size_t tokens, size_t query_heads, size_t key_heads,
                                   size_t head_dim, size_t rotary_dim, float rope_scale,
                                   float rope_theta, lb_rope_pos_ids_spec *out) {
    if (!out) return fail(LB_INVALID_ARGUMENT, "out");
    if (tokens == 0 || query_heads == 0 || key_heads == 0 || head_dim == 0)
        return fail(LB_ZERO_DIMENSION);
    if (rotary_dim == 0 || rotary_dim % 2 != 0 || rotary_dim > head_dim)
        return fail(LB_INVALID_ROTARY_DIMENSION, nullptr, (int64_t)rotary_dim, (int64_t)head_dim);
    if (!std::isfinite(rope_scale) || rope_scale <= 0.0f) return fail(LB_INVALID_ROPE_SCALE);
    if (!std::isfinite(rope_theta) || rope_theta <= 1.0f) return fail(LB_INVALID_ROPE_THETA);
    size_t t;
    if (mul_overflow(tokens, query_heads, &t) || mul_overflow(t, head_dim, &t) ||
        mul_overflow(tokens, key_heads, &t) || mul_overflow(t, head_dim, &t))
        return fail(LB_ELEMENT_COUNT_OVERFLOW);
    out->tokens = tokens;
    out->query_heads = query_heads;
    out->key_heads = key_heads;
    out->head_dim = head_dim;
    out->rotary_dim = rotary_dim;
    out->rope_scale = rope_scale;
    out->rope_theta = rope_theta;
    return LB_OK;
}

size_t lb_rope_pos_ids_spec_query_numel(const lb_rope_pos_ids_spec *spec) {
    return spec ? spec->tokens * spec->query_heads * spec->head_dim : 0;
}
size_t lb_rope_pos_ids_spec_key_numel(const lb_rope_pos_ids_spec *spec) {
    return spec ? spec->tokens * spec->key_heads * spec->head_dim : 0;
}

}
