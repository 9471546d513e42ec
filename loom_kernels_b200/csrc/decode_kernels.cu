// Paged decode attention for sm_100a: BF16 NHD, head dim 128, page size 16 -- the direct and the
// fixed-partition split-K algorithms (one CTA per (request, head block, query block, chunk)).
//
// Replaces the reference's paged_batch_decode_bf16_nhd{,_token_parallel} kernels
// (crates/loom-infer-cuda/src/attention/decode.rs:210-371,395-678) and supplies the paged
// split-K partial + merge pair the reference only has for contiguous KV (:699-998).
//
// Shape of the kernel
//   work item  = (request, block of HC KV heads, query block, page chunk); one CTA each.
//   data path  = one warp issues TMA tile loads (cp.async.bulk.tensor.3d, 128-byte swizzle) into
//                a ring of shared-memory stages: one box per (page, K|V) covering the CTA's HC
//                heads, laid out [head half][16 tokens][64 dims] (up to 32 KB per instruction;
//                small boxes cap an SM near 45 GB/s, 32 KB boxes reach 80+).  Every page slot
//                of a stage has its own full/empty mbarrier pair.
//   math       = each consumer warp owns one (page slot, KV head) of every stage and the whole GQA
//                group of that KV head as the M=16 rows of mma.sync.m16n8k16 (BF16 in, F32 out):
//                S = Q K^T (16 MMAs), online softmax in registers (exp2 domain), O += P V
//                (16 MMAs).  K/V bytes are read from HBM once per KV head, not once per query
//                head.  The op is HBM-bound (<= 32 FLOP/B), so tensor cores only keep the
//                issue slots free for loads; tcgen05/TMEM tiles (M >= 64) would be empty.
//   epilogue   = warps that shared a KV head merge their states in shared memory; the CTA then
//                writes BF16 O + log2 LSE (direct) or the F32 state [m, n, wv[128]] (split-K).
//
// Device-resident metadata is never an error: an invalid request returns without writing
// (decode.rs:238-248,281-283,430-478).  Every mbarrier wait is bounded; on a timeout the CTA
// records a status word and writes nothing.
#include <cstring>

#include "decode_device.cuh"
#include "kernels.hpp"

namespace lb {
namespace {

using namespace dev;

constexpr int kMergeFloatsPerWarp = 68 * 32; // 64 accumulators + m[2] + l[2], lane-major

struct DecodeArgs {
    const __nv_bfloat16 *query;
    const int32_t *indptr, *indices, *last;
    __nv_bfloat16 *output;
    float *lse;
    float *workspace;
    int32_t *status;
    int32_t batch, max_pages, qh, kvh, indices_len, indices_min;
    int32_t hc, pps, mt, qb, partitions, stages;
    float scale_log2;
    long long workspace_numel; // F32 elements bound as the workspace (checked builds)
    int32_t skip_page;     // tests of the give-up path: 1 + the page whose bytes never all arrive
    long long wait_cycles; // limit of every bounded wait
    int32_t *counters;     // split plans that merge in this kernel: one word per item, zero
                           // between commands (a queue's synchronisation words)
    PeerOut peer;          // world == 0 unless the plan gathers its output
    PeerSignal signal;     // world == 0 unless this kernel is the last of a gathering command
};

// The work of one CTA.  A thread that has nothing (more) to do returns from here; every thread
// of the grid then meets again in the kernel below.
// kCluster: the `partitions` CTAs of one (request, head block, query block) form a thread-block
// cluster (the chunk is the CTA's rank in it) and their states are merged through distributed
// shared memory by the cluster's first CTA: split-K as one command, without a workspace.
// What the merge at the end of a split plan's kernel (a.counters) needs to know about this CTA.
struct CtaItem {
    int request, qb, hb;
    bool counted; // the CTA left a state (finished, empty or poisoned) for every row of its item
};

template <bool kGather, bool kCluster>
__device__ __forceinline__ void paged_decode_cta(const CUtensorMap &k_map, const CUtensorMap &v_map,
                                                 const DecodeArgs &a, PeerLocal &peer_local,
                                                 CtaItem &item_out) {
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    const int units = kComputeWarps / a.mt;
    const int stage_bytes = units * kUnitBytes;
    const int slot_bytes = a.hc * kUnitBytes; // one page of the CTA's heads: K box then V box
    // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits 7..9
    uint8_t *ring = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + a.stages * stage_bytes);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + a.stages * a.pps * 8;
    volatile int *flags = reinterpret_cast<volatile int *>(bars + 2 * a.stages * a.pps);
    // flags[0] = an out-of-range page index was seen; flags[1] = a bounded wait ran out

    // ---- work item --------------------------------------------------------------------------
    const int group = a.qh / a.kvh;
    const int head_blocks = a.kvh / a.hc;
    int item = blockIdx.x;
    int part = 0;
    if (kCluster) { // the CTAs of a cluster are consecutive blocks: the chunk varies fastest
        part = item % a.partitions;
        item /= a.partitions;
    }
    const int hb = item % head_blocks; item /= head_blocks;
    const int qb = item % a.qb; item /= a.qb;
    if (!kCluster) {
        part = item % a.partitions;
        item /= a.partitions;
    }
    const int request = item;
    item_out.request = request;
    item_out.qb = qb;
    item_out.hb = hb;
    item_out.counted = false;
    // (a CTA past the batch leaves at once, unless the plan gathers: there every CTA of the grid
    // is counted at the kernel's end)
    if (!kGather && request >= a.batch) return;

    // barriers: one thread each, before the first touch of global memory
    if (tid < a.stages * a.pps) {
        mbar_init(full0 + tid * 8, 1);
        mbar_init(empty0 + tid * 8, a.hc * a.mt);
        fence_barrier_init();
    }
    if (tid == 0) {
        flags[0] = 0;
        flags[1] = 0;
    }
    if (warp == kComputeWarps && lane == 0) {
        prefetch_tensormap(&k_map);
        prefetch_tensormap(&v_map);
    }
    __syncthreads(); // the barriers exist for every warp
    // everything above ran beside the previous command; global memory is touched from here on
    dependent_launch_wait();
    // a gathering plan: the peers' addresses and the epoch, fetched now for the kernel's last
    // instructions (read after the join below, or after the barrier that ends the kernel)
    if (kGather && warp == kComputeWarps - 1) peer_prefetch(a.peer, a.signal, lane, peer_local);
    if (kGather && request >= a.batch) return;
    // The first 32 page ids of the table travel with the request's metadata: when the pages this
    // CTA starts with lie among them (small batches, short contexts) the producer has its ids
    // one round trip earlier.
    int head_of_table = 0;
    if (warp == kComputeWarps && lane < a.indices_len) head_of_table = a.indices[lane];
    int page_start, page_end, tail;
    if (!request_metadata_valid(a.indptr, a.last, a.batch, a.indices_min, a.indices_len, request,
                                page_start, page_end, tail, a.status))
        return;
    const int num_pages = page_end - page_start;
    const int kv_len = (num_pages - 1) * kPage + tail;
    // balanced page partition (single_decode/mod.rs:171-185 applied to pages)
    const int base = num_pages / a.partitions, rem = num_pages % a.partitions;
    const int pg0 = part * base + min(part, rem);
    const int cnt = base + (part < rem ? 1 : 0);
    const int chunk_end_token = min((pg0 + cnt) * kPage, kv_len);
    const int rows_per_block = 16 * a.mt;

    if (!kCluster && cnt == 0) {
        // a chunk without pages: the empty state [0, 0, 0...] the merge skips
        const int row_lo = qb * rows_per_block;
        const int row_hi = min(group, row_lo + rows_per_block);
        const int rows = max(0, row_hi - row_lo);
        for (int i = tid; i < a.hc * rows * kStateWidth; i += blockDim.x) {
            const int e = i % kStateWidth;
            const int row = (i / kStateWidth) % rows;
            const int h = i / (kStateWidth * rows);
            const int qhead = (hb * a.hc + h) * group + row_lo + row;
            const size_t at =
                ((size_t)(request * a.qh + qhead) * a.partitions + part) * kStateWidth + e;
            if (in_bounds((long long)at, a.workspace_numel, a.status, kSiteWorkspace))
                a.workspace[at] = 0.0f;
        }
        item_out.counted = true;
        return;
    }


    const int n_iter = (cnt + a.pps - 1) / a.pps;

    // consumer identity (declared here so the epilogue after the join can use it)
    WarpState st;
    int dest_request = 0; // gathering plans: the row of the gathered result this request owns
    int producer_trips = 0; // producer lanes: iterations of the page loop that issued copies
    const int unit = warp / a.mt;      // consumer: which (page slot, head) of each stage
    const int mtile = warp % a.mt;     // consumer: which 16-row tile of the group
    const int page_slot0 = unit / a.hc;
    const int head_in_cta = unit % a.hc;

    if (warp == kComputeWarps) {
        // ================= producer warp: page-table walk + TMA issue =========================
        const int my_slot = lane >> 1;
        const int which = lane & 1; // 0: K box, 1: V box
        const bool lane_active = my_slot < a.pps;
        const int z = hb * a.hc * 2;
        const CUtensorMap *map = which == 0 ? &k_map : &v_map;
        bool bad_page = false;
        auto fetch_page = [&](int j) -> int { // the raw id (0 past the chunk)
            if (j >= cnt) return 0;
            const int at = page_start + pg0 + j;
            return in_bounds(at, a.indices_len, a.status, kSiteIndices) ? a.indices[at] : 0;
        };
        auto check_page = [&](int id) -> int {
            if (id < 0 || id >= a.max_pages) {
                bad_page = true;
                return 0;
            }
            return id;
        };
        auto load_page = [&](int j) -> int { return check_page(fetch_page(j)); };
        // the first two windows travel together; ids among the first 32 of the table are here
        const int first_index = page_start + pg0 + lane;
        int window = __shfl_sync(0xffffffffu, head_of_table, first_index & 31);
        if (lane >= cnt) window = 0;
        else if (first_index >= 32 &&
                 in_bounds(first_index, a.indices_len, a.status, kSiteIndices))
            window = a.indices[first_index];
        int window_next = fetch_page(32 + lane);
        window = check_page(window);
        window_next = check_page(window_next);
        const uint32_t my_full = full0 + my_slot * 8, my_empty = empty0 + my_slot * 8;
        const uint32_t my_tile =
            smem_u32(ring + my_slot * slot_bytes + which * (slot_bytes / 2));
        int stage = 0;
        uint32_t phase = 0;    // parity of the ring round being filled
        bool recycled = false; // the ring has wrapped: a slot must be handed back before reuse
        // A test of the give-up path: the barrier of one page (of the ring's first round) expects
        // 16 bytes more than its copies deliver, which is all a lost copy would look like -- the
        // page's consumers wait for bytes that never arrive.
        if (a.skip_page != 0 && lane_active && which == 0 && a.skip_page - 1 < cnt &&
            (a.skip_page - 1) % a.pps == my_slot && (a.skip_page - 1) / a.pps < a.stages)
            mbar_expect_more(my_full + ((a.skip_page - 1) / a.pps) * a.pps * 8, 16);
        int it = 0;
        for (; it < n_iter; ++it) {
            const int first = it * a.pps;
            if (it > 0 && (first & 31) == 0) {
                window = window_next;
                window_next = load_page(first + 32 + lane);
            }
            const int slot = first + my_slot;
            const int page_id = __shfl_sync(0xffffffffu, window, slot & 31);
            const bool has = lane_active && slot < cnt;
            const uint32_t bar_full = my_full + stage * a.pps * 8;
            bool ok = true;
            if (has && recycled)
                ok = mbar_wait(my_empty + stage * a.pps * 8, phase ^ 1, a.wait_cycles);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) flags[1] = 1;
                break;
            }
            if (has && which == 0) mbar_expect_tx(bar_full, slot_bytes);
            __syncwarp();
            if (has)
                tma_load_3d(my_tile + stage * stage_bytes, map, 0,
                            in_bounds(page_id, a.max_pages, a.status, kSitePage) ? page_id * kPage
                                                                                : 0,
                            z, bar_full);
            if (++stage == a.stages) {
                stage = 0;
                phase ^= 1;
                recycled = true;
            }
        }
        producer_trips = it;
        if (__any_sync(0xffffffffu, bad_page) && lane == 0) flags[0] = 1;
    } else {
        // ================= consumer warps ======================================================
        st.reset();
        if (kGather && a.peer.world != 0) dest_request = a.peer.dest_rows[request];
        const int kv_head = hb * a.hc + head_in_cta;
        const int row0 = qb * rows_per_block + mtile * 16;
        // the rows this warp reads: [row0, min(group, row0 + 16)) of the head's group
        const long long q_row = (long long)request * a.qh + (long long)kv_head * group + row0;
        const int q_rows = in_bounds(q_row, (long long)a.batch * a.qh, a.status, kSiteQuery,
                                     max(0, min(16, group - row0)))
                               ? group - row0
                               : 0;

        // my pages are page_slot0, page_slot0 + pps, ... of the chunk; stage and phase are
        // carried as counters (no division in the loop)
        const int my_pages = cnt > page_slot0 ? (cnt - page_slot0 + a.pps - 1) / a.pps : 0;
        int tokens_left = chunk_end_token - (pg0 + page_slot0) * kPage;
        const int tile_offset = page_slot0 * slot_bytes + head_in_cta * 2 * kBoxBytes;
        const uint32_t my_full = full0 + page_slot0 * 8, my_empty = empty0 + page_slot0 * 8;
        int stage = 0;
        uint32_t phase = 0;
        uint32_t qf[8][4];
        load_query_fragments(a.query + (size_t)q_row * kHeadDim, q_rows, lane, qf);
        for (int it = 0; it < my_pages; ++it) {
            const bool ok = mbar_wait(my_full + stage * a.pps * 8, phase, a.wait_cycles);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) flags[1] = 1;
                break;
            }
            uint8_t *k_tile = ring + stage * stage_bytes + tile_offset;
            const bool wrote = attend_page(k_tile, k_tile + slot_bytes / 2, min(kPage, tokens_left),
                                           qf, a.scale_log2, lane, st);
            __syncwarp();
            if (lane == 0) {
                if (wrote) fence_proxy_async();
                mbar_arrive(my_empty + stage * a.pps * 8);
            }
            tokens_left -= a.pps * kPage;
            if (++stage == a.stages) {
                stage = 0;
                phase ^= 1;
            }
        }
        st.finish_rows();
    }

    // ---- join: every TMA write has been consumed or abandoned; the ring becomes scratch ---------
    __syncthreads();
    const bool timed_out = flags[1] != 0;
    const bool invalid_page = flags[0] != 0;
    if (timed_out) {
        // nothing is published; the copies already on their way are waited for (bounded), so
        // that none lands in shared memory after this CTA has gone
        if (warp == kComputeWarps && (lane & 1) == 0 && (lane >> 1) < a.pps) {
            // pages of my slot whose copies were issued: one per trip of the producer loop while
            // the slot still had pages of the chunk
            const int slot = lane >> 1;
            const int mine = cnt > slot ? (cnt - slot + a.pps - 1) / a.pps : 0;
            drain_issued_copies(full0 + slot * 8, a.pps * 8, a.stages, min(producer_trips, mine),
                                a.wait_cycles);
        }
        __syncthreads();
        if (tid == 0 && a.status) atomicExch(a.status, 1);
        if (!kCluster && a.counters != nullptr) {
            // the item's chunks are counted at the kernel's end: this one leaves poisoned states,
            // so that the count stays whole and the rows keep their previous contents
            const int row_lo = qb * rows_per_block;
            const int rows = max(0, min(group, row_lo + rows_per_block) - row_lo);
            for (int i = tid; i < a.hc * rows; i += blockDim.x) {
                const int qhead = (hb * a.hc + i / rows) * group + row_lo + i % rows;
                const size_t at =
                    ((size_t)(request * a.qh + qhead) * a.partitions + part) * kStateWidth;
                if (in_bounds((long long)at, a.workspace_numel, a.status, kSiteWorkspace,
                              kStateWidth))
                    a.workspace[at + 1] = -1.0f;
            }
            item_out.counted = true;
        }
        if (!kCluster) return; // (a cluster's CTAs still meet at its barriers: a poisoned state)
    }

    // page slots that streamed pages of this chunk: slot s has pages iff s < cnt
    const int populated = timed_out ? 0 : min(a.pps, cnt);
    if (populated > 1) {
        // warps that streamed different pages of the same KV head merge their states
        float *scratch = reinterpret_cast<float *>(ring);
        if (warp < kComputeWarps && page_slot0 > 0 && page_slot0 < populated) {
            float *mine = scratch + warp * kMergeFloatsPerWarp;
#pragma unroll
            for (int nt = 0; nt < 16; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) mine[(nt * 4 + j) * 32 + lane] = st.acc[nt][j];
            mine[64 * 32 + lane] = st.row_max[0];
            mine[65 * 32 + lane] = st.row_max[1];
            mine[66 * 32 + lane] = st.row_sum[0];
            mine[67 * 32 + lane] = st.row_sum[1];
        }
        __syncthreads();
        if (warp < kComputeWarps && page_slot0 == 0) {
            for (int k = 1; k < populated; ++k) {
                const float *other = scratch + (warp + k * a.hc * a.mt) * kMergeFloatsPerWarp;
                const float om0 = other[64 * 32 + lane], om1 = other[65 * 32 + lane];
                const float ol0 = other[66 * 32 + lane], ol1 = other[67 * 32 + lane];
                const float n0 = fmaxf(st.row_max[0], om0), n1 = fmaxf(st.row_max[1], om1);
                const float w0 = ol0 == 0.0f ? 1.0f : exp2f(st.row_max[0] - n0);
                const float w1 = ol1 == 0.0f ? 1.0f : exp2f(st.row_max[1] - n1);
                const float ow0 = ol0 == 0.0f ? 0.0f : exp2f(om0 - n0);
                const float ow1 = ol1 == 0.0f ? 0.0f : exp2f(om1 - n1);
                if (ol0 != 0.0f) st.row_max[0] = n0;
                if (ol1 != 0.0f) st.row_max[1] = n1;
                st.row_sum[0] = st.row_sum[0] * w0 + ol0 * ow0;
                st.row_sum[1] = st.row_sum[1] * w1 + ol1 * ow1;
#pragma unroll
                for (int nt = 0; nt < 16; ++nt) {
                    st.acc[nt][0] = st.acc[nt][0] * w0 + other[(nt * 4 + 0) * 32 + lane] * ow0;
                    st.acc[nt][1] = st.acc[nt][1] * w0 + other[(nt * 4 + 1) * 32 + lane] * ow0;
                    st.acc[nt][2] = st.acc[nt][2] * w1 + other[(nt * 4 + 2) * 32 + lane] * ow1;
                    st.acc[nt][3] = st.acc[nt][3] * w1 + other[(nt * 4 + 3) * 32 + lane] * ow1;
                }
            }
        }
    }

    if (kCluster) {
        // every CTA leaves the state of its chunk in its own shared memory (beyond the scratch of
        // the slot merge, which other warps may still be reading) ...
        float *chunk_state = reinterpret_cast<float *>(ring) + kComputeWarps * kMergeFloatsPerWarp;
        const int valid_rows = min(rows_per_block, group - qb * rows_per_block);
        if (warp < kComputeWarps && page_slot0 == 0) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = mtile * 16 + (lane >> 2) + half * 8;
                if (row < valid_rows)
                    write_state_row(chunk_state +
                                        (size_t)(head_in_cta * rows_per_block + row) * kStateWidth,
                                    lane, half, st, invalid_page || timed_out);
            }
        }
        cluster_barrier();
        // ... and the cluster's first CTA merges them, one warp per row
        if (part == 0 && warp < kComputeWarps) {
            for (int r = warp; r < a.hc * valid_rows; r += kComputeWarps) {
                const int h = r / valid_rows, row = r - h * valid_rows;
                float top, norm;
                float4 acc;
                const bool ok = merge_cluster_row(
                    smem_u32(chunk_state + (size_t)(h * rows_per_block + row) * kStateWidth),
                    a.partitions, lane, top, norm, acc);
                const long long head = (long long)(hb * a.hc + h) * group + qb * rows_per_block + row;
                if (kGather && a.peer.world != 0) {
                    const long long out_row =
                        (long long)a.peer.dest_rows[request] * a.peer.gathered_qh +
                        a.peer.head_offset + head;
                    for (int p = 0; p < a.peer.world; ++p)
                        if (ok)
                            publish_merged(top, norm, acc, lane,
                                           static_cast<__nv_bfloat16 *>(peer_local.out[p]) +
                                               out_row * kHeadDim,
                                           peer_local.lse[p] + out_row);
                } else if (ok) {
                    const long long state = (long long)request * a.qh + head;
                    if (in_bounds(state, (long long)a.batch * a.qh, a.status, kSiteOutput))
                        publish_merged(top, norm, acc, lane, a.output + state * kHeadDim,
                                       a.lse + state);
                }
            }
        }
        cluster_barrier(); // nobody leaves while the first CTA still reads its shared memory
        return;
    }
    item_out.counted = true; // (every thread of the CTA passes here)
    if (warp >= kComputeWarps || page_slot0 != 0) return;

    // ---- epilogue ---------------------------------------------------------------------------------
    const int kv_head = hb * a.hc + head_in_cta;
    const int g0 = qb * rows_per_block + mtile * 16 + (lane >> 2);
    if (kGather && a.partitions == 1 && a.peer.world != 0) {
        // the finished rows go straight into every rank's copy of the gathered result
        const long long row0 = (long long)dest_request * a.peer.gathered_qh + a.peer.head_offset +
                               (long long)kv_head * group;
        const long long rows[2] = {g0 < group && !invalid_page ? row0 + g0 : -1,
                                   g0 + 8 < group && !invalid_page ? row0 + g0 + 8 : -1};
        write_final_rows_to_peers(peer_local, a.peer.world, rows, lane, st);
        return;
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int g = g0 + half * 8;
        if (g >= group) continue;
        const size_t state = (size_t)request * a.qh + (size_t)kv_head * group + g;
        if (a.partitions == 1) {
            if (invalid_page) continue; // the request keeps its previous output
            if (in_bounds((long long)state, (long long)a.batch * a.qh, a.status, kSiteOutput))
                write_final_row(a.output + state * kHeadDim, a.lse + state, lane, half, st);
        } else {
            const size_t at = (state * a.partitions + part) * kStateWidth;
            if (in_bounds((long long)at, a.workspace_numel, a.status, kSiteWorkspace, kStateWidth))
                write_state_row(a.workspace + at, lane, half, st, invalid_page);
        }
    }
}

// Split-K as one command: every chunk's CTA has left its states in the workspace; each counts
// itself on its item's word, and the one that finds the item complete merges the item's rows and
// writes O and LSE.  The word wraps to zero on the last count (atomicInc), so it is ready for
// the next command without anybody resetting it.  No CTA waits for another.
template <bool kGather>
__device__ __forceinline__ void merge_when_last(const DecodeArgs &a, const CtaItem &item) {
    __shared__ int is_last;
    const int head_blocks = a.kvh / a.hc;
    __syncthreads(); // every state of this CTA has been written ...
    if (threadIdx.x == 0) {
        __threadfence(); // ... and is visible to the GPU before the count is
        const unsigned word = ((unsigned)item.request * a.qb + item.qb) * head_blocks + item.hb;
        const unsigned seen = atomicInc(reinterpret_cast<unsigned *>(a.counters) + word,
                                        (unsigned)a.partitions - 1);
        is_last = seen == (unsigned)a.partitions - 1;
        if (is_last) __threadfence();
    }
    __syncthreads();
    if (!is_last) return;
    const int group = a.qh / a.kvh;
    const int rows_per_block = 16 * a.mt;
    const int row_lo = item.qb * rows_per_block;
    const int rows = max(0, min(group, row_lo + rows_per_block) - row_lo);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < a.hc * rows; r += kComputeWarps + 1) {
        const int qhead = (item.hb * a.hc + r / rows) * group + row_lo + r % rows;
        const long long state = (long long)item.request * a.qh + qhead;
        const float *first = a.workspace + (size_t)state * a.partitions * kStateWidth;
        auto state_of = [&](int p) { return first + (size_t)p * kStateWidth; };
        if (!in_bounds((state + 1) * a.partitions * kStateWidth - 1, a.workspace_numel, a.status,
                       kSiteWorkspace) ||
            !in_bounds(state, (long long)a.batch * a.qh, a.status, kSiteOutput))
            continue;
        if (kGather && a.peer.world != 0)
            merge_states_to_peers(state_of, a.partitions, lane, true, a.peer, item.request, qhead);
        else
            merge_states<8>(state_of, a.partitions, lane, true, a.output + state * kHeadDim,
                            a.lse + state);
    }
}

// kGather: the instantiation for plans that gather their output (the other one carries none of
// its registers or shared memory).
template <bool kGather, bool kCluster>
__global__ void __launch_bounds__((kComputeWarps + 1) * 32, 1)
paged_decode_kernel(const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const DecodeArgs a) {
    __shared__ PeerLocal peer_local;
    dependent_launch_release();
    CtaItem item;
    paged_decode_cta<kGather, kCluster>(k_map, v_map, a, peer_local, item);
    if (!kCluster && a.counters != nullptr && item.counted)
        merge_when_last<kGather>(a, item);
    if (!kGather || a.signal.world == 0 || a.signal.defer) return;
    __syncthreads(); // every row of this CTA has been stored; peer_local is complete
    if (threadIdx.x >= 32) return;
    peer_signal_and_wait(a.signal,
                         (int)threadIdx.x < a.signal.world ? peer_local.flags[threadIdx.x] : nullptr,
                         peer_local.flags[a.signal.rank], peer_local.epoch);
}

// Merges the split-K states of one (request, query head) per warp (merge_states).
__device__ __forceinline__ void split_merge_warp(const float *__restrict__ workspace,
                                                 __nv_bfloat16 *output, float *lse,
                                                 const int32_t *indptr, const int32_t *last,
                                                 int batch, int qh, int partitions,
                                                 int indices_min, int indices_len,
                                                 const PeerOut &peer, long long workspace_numel,
                                                 int32_t *status) {
    const int lane = threadIdx.x & 31;
    const int state = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (state >= batch * qh) return;
    if (!in_bounds((long long)(state + 1) * partitions * kStateWidth - 1, workspace_numel, status,
                   kSiteWorkspace))
        return;
    const int request = state / qh;
    dependent_launch_wait(); // the partial states are complete and visible
    // the guard's loads and the state loads travel together; the verdict is used at the end
    int page_start, page_end, tail;
    const bool valid = indptr == nullptr || // a bare state merge has no request metadata
                       request_metadata_valid(indptr, last, batch, indices_min, indices_len, request,
                                              page_start, page_end, tail);
    const float *st = workspace + (size_t)state * partitions * kStateWidth;
    auto state_of = [&](int p) { return st + (size_t)p * kStateWidth; };
    if (peer.world != 0) {
        merge_states_to_peers(state_of, partitions, lane, valid, peer, request,
                              state - request * qh);
        return;
    }
    merge_states(state_of, partitions, lane, valid, output + (size_t)state * kHeadDim, lse + state);
}

__global__ void __launch_bounds__(128)
split_merge_kernel(const float *__restrict__ workspace, __nv_bfloat16 *output, float *lse,
                   const int32_t *indptr, const int32_t *last, int batch, int qh, int partitions,
                   int indices_min, int indices_len, const PeerOut peer, const PeerSignal signal,
                   long long workspace_numel, int32_t *status) {
    dependent_launch_release();
    MergeSignalPrefetch handshake;
    if (signal.world != 0) {
        dependent_launch_wait();
        handshake.fetch(signal);
    }
    split_merge_warp(workspace, output, lse, indptr, last, batch, qh, partitions, indices_min,
                     indices_len, peer, workspace_numel, status);
    handshake.finish(signal);
}

template <bool kGather, bool kCluster>
int configure_one(size_t max_dynamic_shared) {
    // the opt-in limit covers static and dynamic shared memory together
    cudaFuncAttributes attributes;
    int rc = cudaFuncGetAttributes(&attributes, paged_decode_kernel<kGather, kCluster>);
    if (rc) return rc;
    return cudaFuncSetAttribute(paged_decode_kernel<kGather, kCluster>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)(max_dynamic_shared - attributes.sharedSizeBytes));
}

} // namespace

int configure_decode_kernels(size_t max_dynamic_shared) {
    int rc = configure_one<false, false>(max_dynamic_shared);
    if (!rc) rc = configure_one<true, false>(max_dynamic_shared);
    if (!rc) rc = configure_one<false, true>(max_dynamic_shared);
    if (!rc) rc = configure_one<true, true>(max_dynamic_shared);
    if (rc) return rc;
    return configure_stream_kernels(max_dynamic_shared);
}

int launch_paged_decode(const DecodeLaunch &launch, void *stream) {
    DecodeArgs args;
    args.query = static_cast<const __nv_bfloat16 *>(launch.query);
    args.indptr = launch.indptr;
    args.indices = launch.indices;
    args.last = launch.last;
    args.output = static_cast<__nv_bfloat16 *>(launch.output);
    args.lse = launch.lse;
    args.workspace = launch.workspace;
    args.status = launch.status;
    args.batch = launch.batch;
    args.max_pages = launch.max_pages;
    args.qh = launch.qh;
    args.kvh = launch.kvh;
    args.indices_len = launch.indices_len;
    args.indices_min = launch.indices_min;
    args.hc = launch.heads_per_cta;
    args.pps = launch.pages_per_stage;
    args.mt = launch.q_tiles;
    args.qb = launch.q_blocks;
    args.partitions = launch.partitions;
    args.stages = launch.stages;
    args.scale_log2 = launch.scale_log2;
    args.workspace_numel = launch.workspace_numel;
    args.skip_page = launch.test_skip_page;
    args.wait_cycles = launch.wait_cycles > 0 ? launch.wait_cycles : kWaitCycles;
    args.counters = launch.counters;
    args.peer = launch.peer;
    args.signal = launch.signal;
    CUtensorMap k_map, v_map;
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    memcpy(&k_map, launch.k_map, sizeof(k_map));
    memcpy(&v_map, launch.v_map, sizeof(v_map));
    const bool gather = launch.peer.world != 0 || launch.signal.world != 0;
    if (launch.cluster) {
        // the chunks of one item are one thread-block cluster (at most 8 CTAs: portable size)
        const unsigned cluster = (unsigned)launch.partitions;
        if (gather)
            return launch_dependent_cluster(paged_decode_kernel<true, true>, launch.grid,
                                            launch.block, launch.shared_bytes, cluster, stream,
                                            k_map, v_map, args);
        return launch_dependent_cluster(paged_decode_kernel<false, true>, launch.grid, launch.block,
                                        launch.shared_bytes, cluster, stream, k_map, v_map, args);
    }
    if (gather)
        return launch_dependent(paged_decode_kernel<true, false>, launch.grid, launch.block,
                                launch.shared_bytes, stream, k_map, v_map, args);
    return launch_dependent(paged_decode_kernel<false, false>, launch.grid, launch.block,
                            launch.shared_bytes, stream, k_map, v_map, args);
}

int launch_split_merge(const MergeLaunch &launch, void *stream) {
    return launch_dependent(split_merge_kernel, launch.grid, launch.block, 0, stream,
                            launch.workspace, static_cast<__nv_bfloat16 *>(launch.output),
                            launch.lse, launch.indptr, launch.last, launch.batch, launch.qh,
                            launch.partitions, launch.indices_min, launch.indices_len, launch.peer,
                            launch.signal, launch.workspace_numel, launch.status);
}

long long default_wait_cycles() { return kWaitCycles; }

} // namespace lb
