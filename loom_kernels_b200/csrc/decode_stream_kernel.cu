// Balanced paged decode for sm_100a: the same tile pipeline as paged_decode_kernel, but the work
// is cut by PAGES, not by requests.
//
// The reference's paged decode gives one CTA to one (request, query head)
// (crates/loom-infer-cuda/src/attention/decode.rs:225-233); with ragged batches or few requests
// the longest request then decides the run time.  Here every (page, head block) unit of the
// whole batch is laid on one line -- head block major, then request, then page -- and the line is
// cut into `workers` equal pieces (within one page), so every SM streams the same number of bytes
// whatever the request lengths are:
//
//     x = h * total_pages + prefix[r] + page          worker w owns [W*w/workers, W*(w+1)/workers)
//
// A worker = one page-slot lane of a CTA (HC*MT consumer warps + the shared producer warp).  Its
// range decomposes into segments, each inside one (request, head block) item.  A segment that
// covers its item completely is finished in place (BF16 O + log2 LSE); a cut segment leaves an
// unnormalised F32 state [max_log2, normaliser, wv[128]] (crates/loom-infer/src/attention/
// single_decode/mod.rs:10-13) in one of the worker's two workspace slots -- slot 0 if the
// segment begins where the worker begins, else slot 1 -- and balanced_merge_kernel, which
// recomputes the same cut, merges the states of an item in worker order with the arithmetic of
// single_decode_bf16_split_k_merge_reference (:343-379).
//
// Device-resident metadata is never an error: an invalid request contributes no pages and keeps
// its previous output; an out-of-range page index poisons its item.  All waits are bounded.
#include <cstring>

#include "decode_device.cuh"
#include "kernels.hpp"

namespace lb {
namespace {

using namespace dev;

struct StreamArgs {
    const __nv_bfloat16 *query;
    const int32_t *indptr, *indices, *last;
    __nv_bfloat16 *output;
    float *lse;
    float *workspace; // [workers][2][hc * rows][130] F32, then prefix[batch + 1] I32
    int32_t *status;
    int32_t batch, max_pages, qh, kvh, indices_len, indices_min;
    int32_t hc, pps, mt, qb, stages, workers;
    int32_t pw;   // producer warps: 1, or one per page slot (pps)
    int32_t rows; // state rows per KV head in a slot: min(group, 16 * mt)
    long long workspace_numel; // F32 elements bound as the workspace (checked builds)
    float scale_log2;
    long long wait_cycles; // limit of every bounded wait
    int32_t *counters;     // one zeroed word per (item, KV head of the CTA, row tile): cut items
                           // are merged by the warp that counts the last of their states
    PeerOut peer;          // world == 0 unless the plan gathers its output
    PeerSignal signal;     // world == 0 unless this kernel is the last of a gathering command
};

__device__ __forceinline__ size_t state_floats(int workers, int hc, int rows) {
    return (size_t)workers * 2 * hc * rows * kStateWidth;
}

// first index i in [0, n] with prefix[i] > y, minus one: the request that owns page y
__device__ __forceinline__ int owner_of(const int *prefix, int n, int y) {
    int lo = 0, hi = n; // invariant: prefix[lo] <= y < prefix[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= y) lo = mid;
        else hi = mid;
    }
    return lo;
}

// kGather: the instantiation for plans that gather their output (the other one carries none of
// its registers or shared memory).
// kMerge: the instantiation that merges cut items itself (a.counters); the plain one carries none
// of its registers (with the merge compiled into the one kernel the page loop spilled, and the
// ragged MQA family went from 110 to 123 us).
template <bool kGather, bool kMerge>
__device__ __forceinline__ void balanced_decode_cta(const CUtensorMap &k_map,
                                                    const CUtensorMap &v_map, const StreamArgs &a,
                                                    PeerLocal &peer_local) {
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    const int units = kComputeWarps / a.mt;
    const int stage_bytes = units * kUnitBytes;
    const int slot_bytes = a.hc * kUnitBytes;
    uint8_t *ring = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + a.stages * stage_bytes);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + a.stages * a.pps * 8;
    int *flags = reinterpret_cast<int *>(bars + 2 * a.stages * a.pps);
    volatile int *timeout_flag = flags;             // a bounded wait ran out
    volatile int *bad_slot = flags + 1;             // [stages * pps]: page id was out of range
    int *prefix = flags + 1 + a.stages * a.pps;     // [batch + 1] cumulative valid pages
    int *pstart = prefix + a.batch + 1;             // [batch] indptr[r]
    int *ptail = pstart + a.batch;                  // [batch] last_page_len[r]

    if (tid < a.stages * a.pps) {
        mbar_init(full0 + tid * 8, 1);
        mbar_init(empty0 + tid * 8, a.hc * a.mt);
        bad_slot[tid] = 0;
        fence_barrier_init();
    }
    if (tid == 0) {
        prefix[0] = 0;
        *timeout_flag = 0;
    }
    if (warp == kComputeWarps && lane == 0) {
        prefetch_tensormap(&k_map);
        prefetch_tensormap(&v_map);
    }
    // everything above ran beside the previous command; global memory is touched from here on
    dependent_launch_wait();
    // a gathering plan: the peers' addresses, fetched now for the row stores (the barriers of the
    // prefix computation below come before any of them)
    if (kGather && warp == kComputeWarps - 1) peer_prefetch(a.peer, a.signal, lane, peer_local);

    // ---- per-request guards (decode.rs:234-248), then the page prefix over valid requests ------
    const int global_end = a.indptr[a.batch];
    const bool global_ok =
        a.indptr[0] == 0 && global_end >= a.indices_min && global_end <= a.indices_len;
    for (int r = tid; r < a.batch; r += blockDim.x) {
        const int s = a.indptr[r], e = a.indptr[r + 1], t = a.last[r];
        const bool ok = global_ok && s >= 0 && e > s && e <= global_end && t >= 1 && t <= kPage;
        pstart[r] = s;
        ptail[r] = t;
        prefix[r + 1] = ok ? e - s : 0;
    }
    __syncthreads();
    if (warp == 0) {
        // inclusive scan of prefix[1..batch] by one warp: per-lane chunks, then a warp scan
        const int chunk = (a.batch + 31) / 32;
        const int lo = 1 + lane * chunk, hi = min(a.batch + 1, lo + chunk);
        int sum = 0;
        for (int i = lo; i < hi; ++i) sum += prefix[i];
        int offset = sum;
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, offset, d);
            if (lane >= d) offset += up;
        }
        int running = offset - sum;
        for (int i = lo; i < hi; ++i) {
            running += prefix[i];
            prefix[i] = running;
        }
    }
    __syncthreads();
    const int total = prefix[a.batch];
    const int group = a.qh / a.kvh;
    const int head_blocks = a.kvh / a.hc;
    const int items = head_blocks * a.qb;
    // little work uses fewer workers; a CTA none of whose page slots is a worker leaves at once
    const EvenCut cut((long long)(total > 0 ? total : 1) * items, a.workers);
    if (blockIdx.x == 0) {
        // the merge kernel reads the same prefix and the same cut
        int *out_prefix =
            reinterpret_cast<int *>(a.workspace + state_floats(a.workers, a.hc, a.rows));
        const bool room = in_bounds((long long)state_floats(a.workers, a.hc, a.rows) + a.batch + 5,
                                    a.workspace_numel + 1, a.status, kSiteWorkspace);
        for (int i = tid; room && i <= a.batch; i += blockDim.x) out_prefix[i] = prefix[i];
        if (tid == 0 && room) {
            out_prefix[a.batch + 1] = (int)(cut.q & 0xffffffffll);
            out_prefix[a.batch + 2] = (int)(cut.q >> 32);
            out_prefix[a.batch + 3] = cut.r;
            out_prefix[a.batch + 4] = cut.workers;
        }
    }
    if (total == 0) return;
    if ((int)blockIdx.x * a.pps >= cut.workers) return;

    const int rows_per_block = 16 * a.mt;
    int issued = 0; // producer lanes, set when the page loop ends: pages of my slot whose copies
                    // were issued

    if (warp >= kComputeWarps) {
        // ================= producer warps =========================================================
        // One warp serves all pps page slots of the CTA, or (a.pw == pps) every slot has a warp of
        // its own: with 4 KB boxes (one KV head per CTA) a single warp's loop -- look up, wait for
        // a free stage, arm, issue, for four slots in lock-step -- is what bounds the kernel, and
        // four independent loops are not.
        const int slots_here = a.pps / a.pw;                       // slots this warp serves
        const int slot_base = (warp - kComputeWarps) * slots_here; // the first of them
        const int my_slot = slot_base + (lane >> 1);
        const int which = lane & 1; // 0: K box, 1: V box
        const bool lane_active = (lane >> 1) < slots_here;
        const CUtensorMap *map = which == 0 ? &k_map : &v_map;
        // Page lookup is spread over the lanes: the warp's 32 lanes hold a window of 32 /
        // slots_here pages for each worker it serves; lane l looks after page (l % window) of
        // worker (l / window).  So the range of a worker (it starts at page y0 of item h0; one
        // 64-bit division) and every window refill cost one lane's work.
        const int window = 32 / slots_here;
        const int look_slot = slot_base + lane / window, look_j = lane & (window - 1);
        int h0 = 0, y0 = 0, count = 0;
        {
            const int w = blockIdx.x * a.pps + look_slot;
            if (w < cut.workers) {
                const long long begin = cut.begin(w);
                h0 = (int)(begin / total);
                y0 = (int)(begin - (long long)h0 * total);
                count = (int)(cut.begin(w + 1) - begin);
            }
        }
        int longest = count;
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1)
            longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, d));
        // (page id or -1, head block) of page first + look_j of my worker's range
        auto look_up = [&](int first, int &id, int &hb) {
            id = 0;
            hb = 0;
            const int j = first + look_j;
            if (j >= count) return;
            const unsigned pos = (unsigned)y0 + (unsigned)j; // one wrap at most, unless the item
            const int wraps = (int)(pos / (unsigned)total);  // line is short
            const int y = (int)(pos - (unsigned)wraps * (unsigned)total);
            const int r = owner_of(prefix, a.batch, y);
            const int at = pstart[r] + (y - prefix[r]);
            id = in_bounds(at, a.indices_len, a.status, kSiteIndices) ? a.indices[at] : -1;
            if (id < 0 || id >= a.max_pages) id = -1;
            hb = (h0 + wraps) / a.qb;
        };
        int win_id, win_hb, next_id = 0, next_hb = 0;
        look_up(0, win_id, win_hb);
        const int my_source = ((lane >> 1) & (slots_here - 1)) * window; // first lane of my worker's window
        const int my_count = __shfl_sync(0xffffffffu, count, my_source);
        const uint32_t my_full = full0 + my_slot * 8, my_empty = empty0 + my_slot * 8;
        const uint32_t my_tile =
            smem_u32(ring + my_slot * slot_bytes + which * (slot_bytes / 2));
        int stage = 0;
        uint32_t phase = 0;    // parity of the ring round being filled
        bool recycled = false; // the ring has wrapped: a slot must be handed back before reuse
        int j = 0;
        for (; j < longest; ++j) {
            if (j > 0 && (j & (window - 1)) == 0) {
                win_id = next_id;
                win_hb = next_hb;
                if (j + window < longest) look_up(j + window, next_id, next_hb);
            }
            const int source = my_source + (j & (window - 1));
            const int page_id = __shfl_sync(0xffffffffu, win_id, source);
            const int hb = __shfl_sync(0xffffffffu, win_hb, source);
            const bool has = lane_active && j < my_count;
            const uint32_t bar_full = my_full + stage * a.pps * 8;
            bool ok = true;
            if (has && recycled)
                ok = mbar_wait(my_empty + stage * a.pps * 8, phase ^ 1, a.wait_cycles);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) *timeout_flag = 1;
                break;
            }
            if (has && which == 0) {
                bad_slot[stage * a.pps + my_slot] = page_id < 0;
                mbar_expect_tx(bar_full, slot_bytes);
            }
            __syncwarp();
            if (has)
                tma_load_3d(my_tile + stage * stage_bytes, map, 0, max(page_id, 0) * kPage,
                            hb * a.hc * 2, bar_full);
            if (j == 0) {
                // the second window is fetched once the first pages are on their way
                if (window < longest) look_up(window, next_id, next_hb);
            }
            if (++stage == a.stages) {
                stage = 0;
                phase ^= 1;
                recycled = true;
            }
        }
        issued = lane_active ? min(j, my_count) : 0;
    } else {
        // ================= consumer warps: one (worker, KV head, 16-row tile) each ==================
        const int unit = warp / a.mt;
        const int mtile = warp % a.mt;
        const int my_slot = unit / a.hc;
        const int head_in_cta = unit % a.hc;
        const int w = blockIdx.x * a.pps + my_slot;
        const size_t slot_rows = (size_t)a.hc * a.rows;
        WarpState st;
        uint32_t qf[8][4];
        int h = 0, y = 0, remaining = 0;
        if (w < cut.workers) {
            const long long begin = cut.begin(w);
            h = (int)(begin / total);
            y = (int)(begin - (long long)h * total);
            remaining = (int)(cut.begin(w + 1) - begin);
        }
        bool first_segment = true;
        // ring position of the next page this worker consumes (counters, no division per page)
        const int tile_offset = my_slot * slot_bytes + head_in_cta * 2 * kBoxBytes;
        const uint32_t my_full = full0 + my_slot * 8, my_empty = empty0 + my_slot * 8;
        int stage = 0;
        uint32_t phase = 0;
        bool live = true;
        while (remaining > 0) {
            // ---- segment: the part of one (request, head block, query block) item in my range ---
            const int r = owner_of(prefix, a.batch, y);
            const int num_pages = prefix[r + 1] - prefix[r];
            const int first_page = y - prefix[r];
            const int seg_pages = min(num_pages - first_page, remaining);
            const int hb = h / a.qb, qb = h % a.qb;
            const int kv_head = hb * a.hc + head_in_cta;
            const int row0 = qb * rows_per_block + mtile * 16;
            const int dest_request = kGather && a.peer.world != 0 ? a.peer.dest_rows[r] : 0;
            const long long q_row = (long long)r * a.qh + (long long)kv_head * group + row0;
            const int q_rows = in_bounds(q_row, (long long)a.batch * a.qh, a.status, kSiteQuery,
                                         max(0, min(16, group - row0)))
                                   ? group - row0
                                   : 0;
            load_query_fragments(a.query + (size_t)q_row * kHeadDim, q_rows, lane, qf);
            st.reset();
            bool bad = false;
            const int tail = ptail[r];
            const int last_in_segment = num_pages - 1 - first_page; // p of the request's last page
            for (int p = 0; live && p < seg_pages; ++p) {
                const bool ok = mbar_wait(my_full + stage * a.pps * 8, phase, a.wait_cycles);
                if (__any_sync(0xffffffffu, !ok)) {
                    if (lane == 0) *timeout_flag = 1;
                    live = false;
                    break;
                }
                bad |= bad_slot[stage * a.pps + my_slot] != 0;
                uint8_t *k_tile = ring + stage * stage_bytes + tile_offset;
                const bool wrote =
                    attend_page(k_tile, k_tile + slot_bytes / 2, p == last_in_segment ? tail : kPage,
                                qf, a.scale_log2, lane, st);
                __syncwarp();
                if (lane == 0) {
                    if (wrote) fence_proxy_async();
                    mbar_arrive(my_empty + stage * a.pps * 8);
                }
                if (++stage == a.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            // (after a wait ran out the worker still walks its segments: each leaves a poisoned
            // state, so that the items it shares with other workers are counted whole)
            if (!live) bad = true;
            st.finish_rows();
            const bool complete = first_page == 0 && seg_pages == num_pages;
            const int which = first_segment ? 0 : 1;
            if (kGather && complete && a.peer.world != 0) {
                // finished in place: straight into every rank's copy of the gathered result
                const int g0 = qb * rows_per_block + mtile * 16 + (lane >> 2);
                const long long row0 = (long long)dest_request * a.peer.gathered_qh +
                                       a.peer.head_offset + (long long)kv_head * group;
                const long long rows[2] = {g0 < group && !bad ? row0 + g0 : -1,
                                           g0 + 8 < group && !bad ? row0 + g0 + 8 : -1};
                write_final_rows_to_peers(peer_local, a.peer.world, rows, lane, st);
            } else
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = mtile * 16 + (lane >> 2) + half * 8; // row within the query block
                const int g = qb * rows_per_block + row;
                if (g >= group) continue;
                if (complete) {
                    if (bad) continue; // the request keeps its previous output
                    const size_t state = (size_t)r * a.qh + (size_t)kv_head * group + g;
                    if (in_bounds((long long)state, (long long)a.batch * a.qh, a.status,
                                  kSiteOutput))
                        write_final_row(a.output + state * kHeadDim, a.lse + state, lane, half, st);
                } else {
                    float *slot = a.workspace +
                                  (((size_t)w * 2 + which) * slot_rows +
                                   (size_t)head_in_cta * a.rows + row) * kStateWidth;
                    if (in_bounds(slot - a.workspace, a.workspace_numel, a.status, kSiteWorkspace,
                                  kStateWidth))
                        write_state_row(slot, lane, half, st, bad);
                }
            }
            if (kMerge && !complete && a.counters != nullptr) {
                // The item is cut: its states are counted, and the warp that finds them all there
                // merges the rows of its tile and publishes them.  Nobody waits; the word wraps to
                // zero on the last count, ready for the next command.
                const long long start = (long long)h * total + prefix[r];
                const int w0 = cut.owner_fast(start), w1 = cut.owner_fast(start + num_pages - 1);
                const int n = w1 - w0 + 1;
                __syncwarp(); // every lane's part of the state has been written ...
                int last = 0;
                if (lane == 0) {
                    __threadfence(); // ... and is visible to the GPU before the count is
                    const unsigned word =
                        ((((unsigned)h * a.batch + r) * a.hc + head_in_cta) * a.mt + mtile);
                    last = atomicInc(reinterpret_cast<unsigned *>(a.counters) + word,
                                     (unsigned)n - 1) == (unsigned)n - 1;
                    if (last) __threadfence();
                }
                if (__shfl_sync(0xffffffffu, last, 0)) {
                    // every worker in [w0, w1] holds pages of this item; all but the first begin
                    // inside the item and used slot 0
                    const int first_slot = cut.begin(w0) != start ? 1 : 0;
                    const size_t slot_stride = slot_rows * kStateWidth;
                    const int tile_row0 = mtile * 16;
                    const int valid = max(0, min(16, group - qb * rows_per_block - tile_row0));
                    const float *base = a.workspace + (size_t)w0 * 2 * slot_stride +
                                        ((size_t)head_in_cta * a.rows + tile_row0) * kStateWidth;
                    auto state_of = [&](int row, int i) -> const float * {
                        return base + (size_t)row * kStateWidth +
                               ((size_t)i * 2 + (i == 0 ? first_slot : 0)) * slot_stride;
                    };
                    const long long head_row0 =
                        (long long)kv_head * group + qb * rows_per_block + tile_row0;
                    auto publish = [&](int row, float top, float norm, float4 acc) {
                        if (kGather && a.peer.world != 0) {
                            const long long at = (long long)dest_request * a.peer.gathered_qh +
                                                 a.peer.head_offset + head_row0 + row;
                            for (int p = 0; p < a.peer.world; ++p)
                                publish_merged(top, norm, acc, lane,
                                               static_cast<__nv_bfloat16 *>(peer_local.out[p]) +
                                                   at * kHeadDim,
                                               peer_local.lse[p] + at);
                        } else {
                            const long long at = (long long)r * a.qh + head_row0 + row;
                            if (in_bounds(at, (long long)a.batch * a.qh, a.status, kSiteOutput))
                                publish_merged(top, norm, acc, lane, a.output + at * kHeadDim,
                                               a.lse + at);
                        }
                    };
                    const bool inside = in_bounds(
                        (base - a.workspace) + (long long)((size_t)(w1 - w0) * 2 + 1) * slot_stride +
                            (long long)(valid > 0 ? valid - 1 : 0) * kStateWidth,
                        a.workspace_numel, a.status, kSiteWorkspace, kStateWidth);
                    if (inside && n <= 4) {
                        for (int row0 = 0; row0 < valid; row0 += 4)
                            merge_few_states_of_rows<4>(
                                [&](int row, int i) { return state_of(row0 + row, i); }, n,
                                min(4, valid - row0), lane,
                                [&](int row, float top, float norm, float4 acc) {
                                    publish(row0 + row, top, norm, acc);
                                });
                    } else if (inside) {
                        for (int row = 0; row < valid; ++row) {
                            float top, norm;
                            float4 acc;
                            if (merge_partial<8>([&](int i) { return state_of(row, i); }, n, lane,
                                                 top, norm, acc) &&
                                norm > 0.0f)
                                publish(row, top, norm, acc);
                        }
                    }
                }
            }
            first_segment = false;
            remaining -= seg_pages;
            y += seg_pages;
            if (y == total) { // the next head block starts again at the first request
                y = 0;
                ++h;
            }
        }
    }
    __syncthreads();
    if (*timeout_flag != 0) {
        // a wait ran out: the copies already on their way are waited for (bounded), so that none
        // lands in shared memory after this CTA has gone
        if (warp >= kComputeWarps && (lane & 1) == 0 && (lane >> 1) < a.pps / a.pw)
            drain_issued_copies(full0 + ((warp - kComputeWarps) * (a.pps / a.pw) + (lane >> 1)) * 8,
                                a.pps * 8, a.stages, issued,
                                a.wait_cycles);
        __syncthreads();
    }
    // (rows this kernel stored into other GPUs' memory are ordered by the stream before the merge
    // kernel, whose last CTA fences at system scope before it publishes the epoch)
    if (*timeout_flag != 0 && tid == 0 && a.status) atomicExch(a.status, 1);
}

template <bool kGather, bool kMerge>
__global__ void __launch_bounds__((kComputeWarps + kMaxProducerWarps) * 32, 1)
balanced_decode_kernel(const __grid_constant__ CUtensorMap k_map,
                       const __grid_constant__ CUtensorMap v_map, const StreamArgs a) {
    __shared__ PeerLocal peer_local;
    dependent_launch_release();
    balanced_decode_cta<kGather, kMerge>(k_map, v_map, a, peer_local);
    // a gathering plan that merges in this kernel: this is the command's last kernel
    if (!kGather || a.signal.world == 0 || a.signal.defer) return;
    __syncthreads(); // every row of this CTA has been stored; peer_local is complete
    if (threadIdx.x >= 32) return;
    peer_signal_and_wait(a.signal,
                         (int)threadIdx.x < a.signal.world ? peer_local.flags[threadIdx.x] : nullptr,
                         peer_local.flags[a.signal.rank], peer_local.epoch);
}

// One warp per (request, query head): finds the workers whose ranges cut this head's item and
// merges their states.  Items that one worker finished alone are skipped.
// kWarps = 1: one warp per item, four items per CTA.  kWarps = 4: the four warps of a CTA share
// the states of one item (small batches, where a long request is cut into many states).
template <int kWarps>
__device__ __forceinline__ void balanced_merge_warp(const float *__restrict__ workspace,
                                                    __nv_bfloat16 *output, float *lse, int batch,
                                                    int qh, int kvh, int hc, int mt, int qblocks,
                                                    int workers, int rows, const PeerOut &peer,
                                                    long long workspace_numel, int32_t *status) {
    const int lane = threadIdx.x & 31;
    const int part = kWarps == 1 ? 0 : (int)(threadIdx.x >> 5);
    const int state = kWarps == 1 ? blockIdx.x * 4 + (threadIdx.x >> 5) : blockIdx.x;
    if (state >= batch * qh) return;
    const int request = state / qh, qhead = state % qh;
    dependent_launch_wait(); // the states and the prefix are complete and visible
    const int *prefix =
        reinterpret_cast<const int *>(workspace + state_floats(workers, hc, rows));
    const int total = __ldcg(prefix + batch); // three independent loads, issued together
    const int page0 = __ldcg(prefix + request);
    const int num_pages = __ldcg(prefix + request + 1) - page0;
    if (num_pages == 0) return; // invalid request: nothing was computed, nothing is published
    const int group = qh / kvh;
    const int kv_head = qhead / group, g = qhead % group;
    const int rows_per_block = 16 * mt;
    const int hb = kv_head / hc, head_in_cta = kv_head % hc;
    const int qb = g / rows_per_block, row = g % rows_per_block;
    // the cut the decode kernel made (four more words behind the prefix, loaded with it)
    const EvenCut cut(((long long)__ldcg(prefix + batch + 2) << 32) |
                          (long long)(unsigned)__ldcg(prefix + batch + 1),
                      __ldcg(prefix + batch + 3), __ldcg(prefix + batch + 4));
    const long long start = (long long)(hb * qblocks + qb) * total + page0;
    const int w0 = cut.owner_fast(start), w1 = cut.owner_fast(start + num_pages - 1);
    if (w0 == w1) return; // finished in place by the decode kernel
    // every worker in [w0, w1] holds pages of this item (a worker is never empty); all but the
    // first begin inside the item and used slot 0
    const int first_slot = cut.begin(w0) != start ? 1 : 0;
    const size_t slot_stride = (size_t)hc * rows * kStateWidth;
    const float *base = workspace + (size_t)w0 * 2 * slot_stride +
                        ((size_t)head_in_cta * rows + row) * kStateWidth;
    // (the checked build: the last state this item reads lies inside the bound workspace)
    if (!in_bounds((base - workspace) + (long long)((size_t)(w1 - w0) * 2 + 1) * slot_stride,
                   workspace_numel, status, kSiteWorkspace, kStateWidth))
        return;
    auto state_of = [&](int i) -> const float * {
        return base + ((size_t)i * 2 + (i == 0 ? first_slot : 0)) * slot_stride;
    };
    if (peer.world != 0) {
        merge_states_to_peers<kWarps>(state_of, w1 - w0 + 1, lane, true, peer, request, qhead,
                                      part);
        return;
    }
    if (kWarps == 1)
        merge_states(state_of, w1 - w0 + 1, lane, true, output + (size_t)state * kHeadDim,
                        lse + state);
    else
        merge_states_shared<kWarps>(state_of, w1 - w0 + 1, lane, part,
                                    output + (size_t)state * kHeadDim, lse + state);
}

// (A form in which a warp takes four consecutive rows of one KV head -- one look-up of the cut
// for the four, their loads in flight together, a quarter of the warps -- measured the same
// 14.5 us on the 8192 rows of a ragged MQA batch and slower on small grids: the kernel's time is
// the instruction chain of one warp, about ten cycles per instruction, not the number of warps.)
// (Capping the one-warp form at 64 registers for eight CTAs per SM spilled and measured slower:
// 16.0 against 14.5 us on the 8192 rows of a ragged MQA batch.)
template <int kWarps>
__global__ void __launch_bounds__(128)
balanced_merge_kernel(const float *__restrict__ workspace, __nv_bfloat16 *output, float *lse,
                      int batch, int qh, int kvh, int hc, int mt, int qblocks, int workers,
                      int rows, const PeerOut peer, const PeerSignal signal,
                      long long workspace_numel, int32_t *status) {
    dependent_launch_release();
    MergeSignalPrefetch handshake;
    if (signal.world != 0) {
        dependent_launch_wait();
        handshake.fetch(signal);
    }
    balanced_merge_warp<kWarps>(workspace, output, lse, batch, qh, kvh, hc, mt, qblocks, workers,
                                rows, peer, workspace_numel, status);
    handshake.finish(signal);
}

int balanced_state_rows(const DecodeLaunch &launch) {
    const int group = launch.qh / launch.kvh;
    return group < 16 * launch.q_tiles ? group : 16 * launch.q_tiles;
}

} // namespace

template <bool kGather, bool kMerge>
static int configure_balanced(size_t max_dynamic_shared) {
    // the opt-in limit covers static and dynamic shared memory together
    cudaFuncAttributes attributes;
    const int rc = cudaFuncGetAttributes(&attributes, balanced_decode_kernel<kGather, kMerge>);
    if (rc) return rc;
    return cudaFuncSetAttribute(balanced_decode_kernel<kGather, kMerge>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)(max_dynamic_shared - attributes.sharedSizeBytes));
}

int configure_stream_kernels(size_t max_dynamic_shared) {
    int rc = configure_balanced<false, false>(max_dynamic_shared);
    if (!rc) rc = configure_balanced<true, false>(max_dynamic_shared);
    if (!rc) rc = configure_balanced<false, true>(max_dynamic_shared);
    if (!rc) rc = configure_balanced<true, true>(max_dynamic_shared);
    return rc;
}

int launch_balanced_decode(const DecodeLaunch &launch, void *stream) {
    StreamArgs args;
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
    args.stages = launch.stages;
    args.pw = launch.producer_warps > 0 ? launch.producer_warps : 1;
    args.workers = (int32_t)launch.grid * launch.pages_per_stage;
    args.rows = balanced_state_rows(launch);
    args.workspace_numel = launch.workspace_numel;
    args.scale_log2 = launch.scale_log2;
    args.wait_cycles = launch.wait_cycles > 0 ? launch.wait_cycles : kWaitCycles;
    args.counters = launch.counters;
    args.peer = launch.peer;
    args.signal = launch.signal;
    CUtensorMap k_map, v_map;
    memcpy(&k_map, launch.k_map, sizeof(k_map));
    memcpy(&v_map, launch.v_map, sizeof(v_map));
    const bool gather = launch.peer.world != 0, merge = launch.counters != nullptr;
    auto kernel = merge ? (gather ? balanced_decode_kernel<true, true> : balanced_decode_kernel<false, true>)
                        : (gather ? balanced_decode_kernel<true, false>
                                  : balanced_decode_kernel<false, false>);
    return launch_dependent(kernel, launch.grid, launch.block, launch.shared_bytes, stream, k_map,
                            v_map, args);
}

int launch_balanced_merge(const DecodeLaunch &launch, uint32_t grid, uint32_t block,
                          void *stream) {
    if (launch.merge_four_warps)
        return launch_dependent(balanced_merge_kernel<4>, grid, block, 0, stream,
                                (const float *)launch.workspace,
                                static_cast<__nv_bfloat16 *>(launch.output), launch.lse,
                                launch.batch, launch.qh, launch.kvh, launch.heads_per_cta,
                                launch.q_tiles, launch.q_blocks,
                                (int)launch.grid * launch.pages_per_stage,
                                balanced_state_rows(launch), launch.peer, launch.signal,
                                launch.workspace_numel, launch.status);
    return launch_dependent(balanced_merge_kernel<1>, grid, block, 0, stream,
                            (const float *)launch.workspace,
                            static_cast<__nv_bfloat16 *>(launch.output), launch.lse, launch.batch,
                            launch.qh, launch.kvh, launch.heads_per_cta, launch.q_tiles,
                            launch.q_blocks, (int)launch.grid * launch.pages_per_stage,
                            balanced_state_rows(launch), launch.peer, launch.signal,
                                launch.workspace_numel, launch.status);
}

} // namespace lb
