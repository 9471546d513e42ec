// Shared by the paged-prefill kernels: the launch arguments and the mapping from a row tile to
// the request that owns it.
#pragma once

#include "decode_device.cuh"

namespace lb {
namespace dev {

struct PrefillArgs {
    const __nv_bfloat16 *query;
    const int32_t *qo_indptr, *indptr, *indices, *last;
    __nv_bfloat16 *output;
    float *lse;
    int32_t *status;
    int32_t batch, nnz_qo, max_pages, qh, kvh, indices_len, indices_min;
    int32_t mt, pps, stages, tiles;
    float scale_log2;
    // tiled kernel with the KV range of a tile cut into chunks: F32 states
    // [nnz_qo * qh][partitions][130] (the split-K state of the decode kernels); partitions == 1
    // writes O and LSE directly
    float *workspace;
    int32_t partitions;
    // a tile uses min(partitions, blocks of the tile / min_chunk_blocks) chunks (one when a
    // plan-chosen count would come out below three): the count follows the KV length actually
    // met, which a plan cannot know
    int32_t min_chunk_blocks;
    long long wait_cycles;  // limit of every bounded wait (tiled kernel)
    int32_t test_lost_copy; // tests of the give-up path: the barrier of the first K block expects
                            // 16 bytes more than its copies deliver
};

// Chunks a tile of `tile_blocks` 64-token blocks is cut into.  One chunk means the CTA writes O and
// LSE itself and the merge leaves the row alone.
// With a plan-chosen count (min_chunk_blocks > 1) a range of fewer than three times that many
// blocks is not worth the second command: 256 new tokens over 2048 (32 blocks) measured 40 us in
// two chunks against 35 us in one.
__device__ __forceinline__ int chunks_of_tile(int tile_blocks, int partitions, int min_chunk_blocks) {
    int wanted = tile_blocks / min_chunk_blocks;
    if (min_chunk_blocks > 1 && wanted < 3) wanted = 1;
    return wanted < 1 ? 1 : (wanted < partitions ? wanted : partitions);
}

// The request that owns row tile `tile` (tiles are numbered request by request; a request of
// qo_len tokens has ceil(qo_len * group / rows) of them) and the tile's index inside it; false
// when the tile is past the last one or a request up to and including the owner has an invalid
// query range (crates/loom-infer-cuda/src/attention/prefill.rs:303-317).  Every lane of the
// calling warp returns the same.  The owner's query range, page range and last-page length come
// back with it: lane l of a window loads the metadata of request r0 + l in the same round trip
// as the query ranges that are searched, and the owner's lane hands its values out.
struct TileOwner {
    int request, tile_in_request, qo_start, qo_end, page_start, page_end, tail;
};
__device__ __forceinline__ bool locate_tile(const PrefillArgs &a, int group, int rows, int tile,
                                            int lane, TileOwner &owner) {
    long long before = 0;
    for (int r0 = 0; r0 < a.batch; r0 += 32) {
        const int r = r0 + lane;
        int start = 0, end = 0, page_start = 0, page_end = 0, tail = 0;
        if (r < a.batch) {
            start = a.qo_indptr[r];
            end = a.qo_indptr[r + 1];
            page_start = a.indptr[r];
            page_end = a.indptr[r + 1];
            tail = a.last[r];
        }
        const bool valid = r >= a.batch || (start >= 0 && end > start && end <= a.nnz_qo);
        const long long mine =
            r < a.batch && valid ? ((long long)(end - start) * group + rows - 1) / rows : 0;
        long long inclusive = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const long long up = __shfl_up_sync(0xffffffffu, inclusive, d);
            if (lane >= d) inclusive += up;
        }
        const long long first = before + inclusive - mine;
        const unsigned bad = __ballot_sync(0xffffffffu, !valid);
        const unsigned hit =
            __ballot_sync(0xffffffffu, mine > 0 && tile >= first && tile < first + mine);
        if (hit) {
            const int source = __ffs(hit) - 1;
            if (bad && __ffs(bad) - 1 < source) return false;
            owner.request = r0 + source;
            owner.tile_in_request = tile - (int)__shfl_sync(0xffffffffu, first, source);
            owner.qo_start = __shfl_sync(0xffffffffu, start, source);
            owner.qo_end = __shfl_sync(0xffffffffu, end, source);
            owner.page_start = __shfl_sync(0xffffffffu, page_start, source);
            owner.page_end = __shfl_sync(0xffffffffu, page_end, source);
            owner.tail = __shfl_sync(0xffffffffu, tail, source);
            return true;
        }
        if (bad) return false;
        before += __shfl_sync(0xffffffffu, inclusive, 31);
    }
    return false;
}

// The guard of the prefill kernels (prefill.rs:289-347) in one round trip to the metadata: the
// global checks, every query range up to the owner of `tile`, the owner's page range and
// qo_len <= kv_len.  Also fetches the first 32 page ids of the table (`head_of_table`, lane l holds
// indices[l]) for the warp `want_head` names, so that a CTA whose first pages lie among them --
// short calls -- has its ids without another trip.
__device__ __forceinline__ bool prefill_guard(const PrefillArgs &a, int group, int rows, int tile,
                                              int lane, bool want_head, TileOwner &owner,
                                              int &head_of_table) {
    const int qo_first = a.qo_indptr[0], qo_total = a.qo_indptr[a.batch];
    const int table_first = a.indptr[0], table_end = a.indptr[a.batch];
    head_of_table = want_head && lane < a.indices_len ? a.indices[lane] : 0;
    const bool located = locate_tile(a, group, rows, tile, lane, owner);
    if (qo_first != 0 || qo_total != a.nnz_qo || !located) return false;
    // request_metadata_valid on the values at hand
    if (table_first != 0 || table_end < a.indices_min || table_end > a.indices_len ||
        owner.page_start < 0 || owner.page_end <= owner.page_start || owner.page_end > table_end ||
        owner.tail < 1 || owner.tail > kPage)
        return false;
    const long long kv_len = (long long)(owner.page_end - owner.page_start - 1) * kPage + owner.tail;
    return owner.qo_end - owner.qo_start <= kv_len;
}

// The request that owns query row `row`, with its query range, page range and last-page length
// (all loaded in the same round trip as the query ranges that are searched: lane l of a window
// loads the metadata of request r0 + l, the owner's lane hands its values out); false when no
// request does or a request up to and including the owner has an invalid query range (the guard
// of locate_tile, per row).
struct RowOwner {
    int request, qo_start, qo_end, page_start, page_end, tail;
};
__device__ __forceinline__ bool locate_row(const int32_t *qo_indptr, const int32_t *indptr,
                                           const int32_t *last, int batch, int nnz_qo, int row,
                                           int lane, RowOwner &owner) {
    for (int r0 = 0; r0 < batch; r0 += 32) {
        const int r = r0 + lane;
        int start = 0, end = 0, page_start = 0, page_end = 0, tail = 0;
        if (r < batch) {
            start = qo_indptr[r];
            end = qo_indptr[r + 1];
            page_start = indptr[r];
            page_end = indptr[r + 1];
            tail = last[r];
        }
        const bool valid = r >= batch || (start >= 0 && end > start && end <= nnz_qo);
        const unsigned bad = __ballot_sync(0xffffffffu, !valid);
        const unsigned hit = __ballot_sync(0xffffffffu, r < batch && valid && row >= start && row < end);
        if (hit) {
            const int source = __ffs(hit) - 1;
            if (bad && __ffs(bad) - 1 < source) return false;
            owner.request = r0 + source;
            owner.qo_start = __shfl_sync(0xffffffffu, start, source);
            owner.qo_end = __shfl_sync(0xffffffffu, end, source);
            owner.page_start = __shfl_sync(0xffffffffu, page_start, source);
            owner.page_end = __shfl_sync(0xffffffffu, page_end, source);
            owner.tail = __shfl_sync(0xffffffffu, tail, source);
            return true;
        }
        if (bad) return false;
    }
    return false;
}

} // namespace dev
} // namespace lb
