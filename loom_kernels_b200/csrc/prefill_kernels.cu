// Paged causal prefill for sm_100a: BF16 NHD, head dim 128, page size 16, ragged queries, the
// causal mask aligned bottom-right (query i of a request sees kv_index <= kv_len - qo_len + i).
//
// Replaces the reference's paged_prefill_bf16_nhd_causal{,_token_parallel8,_token_parallel16}
// kernels (crates/loom-infer-cuda/src/attention/prefill.rs:270-470,799-1170), which give every
// (query row, query head) a CTA of its own and so read a request's K/V once per row and head.
//
// Shape of the kernel
//   packed rows = for one KV head of one request the query rows are (token, head in group),
//                 row p = token * group + head: all of them read the same K/V.
//   work item   = (request, KV head, tile of 16 * MT packed rows); one CTA each.  The grid is an
//                 upper bound fixed by the plan (floor(nnz_qo * group / rows) + batch tiles per
//                 KV head); a CTA finds its request by a prefix sum over qo_indptr and returns
//                 if it is past the last tile.
//   data path   = the decode pipeline: one warp issues TMA page loads (K box + V box of the CTA's
//                 KV head, 128-byte swizzle) into a ring of stages with 8 / MT page slots each.
//   math        = consumer warp (slot s, tile m) streams pages s, s + slots, ... of the CTA for
//                 its 16 rows: S = Q K^T and O += P V on mma.sync.m16n8k16, online softmax in
//                 the log2 domain, the causal limit applied per row.  Warps that shared rows merge
//                 their states in shared memory; the CTA writes BF16 O + log2 LSE.
//
// Device-resident metadata is never an error: a row whose request fails the guard keeps its
// previous output (prefill.rs:289-347).  Every mbarrier wait is bounded; on a timeout the CTA
// records a status word and writes nothing.
#include <cstring>

#include "kernels.hpp"
#include "prefill_device.cuh"

namespace lb {
namespace {

using namespace dev;

constexpr int kMergeFloatsPerWarp = 68 * 32; // 64 accumulators + m[2] + l[2], lane-major

__global__ void __launch_bounds__((kComputeWarps + 1) * 32, 1)
paged_prefill_kernel(const __grid_constant__ CUtensorMap k_map,
                     const __grid_constant__ CUtensorMap v_map, const PrefillArgs a) {
    extern __shared__ uint8_t smem_raw[];
    dependent_launch_release();
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    const int slot_bytes = kUnitBytes; // one page of the CTA's KV head: K box then V box
    const int stage_bytes = a.pps * slot_bytes;
    uint8_t *ring = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + a.stages * stage_bytes);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + a.stages * a.pps * 8;
    volatile int *flags = reinterpret_cast<volatile int *>(bars + 2 * a.stages * a.pps);
    // flags[0] = an out-of-range page index was seen; flags[1] = a bounded wait ran out

    const int group = a.qh / a.kvh;
    const int rows_per_cta = 16 * a.mt;
    const int kv_head = blockIdx.x % a.kvh;
    // tiles late in a request see the most KV: they are started first
    const int tile = a.tiles - 1 - (int)(blockIdx.x / a.kvh);

    if (tid < a.stages * a.pps) {
        mbar_init(full0 + tid * 8, 1);
        mbar_init(empty0 + tid * 8, a.mt);
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
    TileOwner owner;
    int head_of_table;
    if (!prefill_guard(a, group, rows_per_cta, tile, lane, warp == kComputeWarps, owner,
                       head_of_table))
        return; // prefill.rs:289-347
    const int tile_in_request = owner.tile_in_request;
    const int page_start = owner.page_start, tail = owner.tail;
    const int qo_start = owner.qo_start;
    const int qo_len = owner.qo_end - qo_start;
    const int num_pages = owner.page_end - page_start;
    const int kv_len = (num_pages - 1) * kPage + tail;
    const int shift = kv_len - qo_len + 1; // row of token t sees logical tokens [0, shift + t)

    const long long rows_total = (long long)qo_len * group;
    const long long row_lo = (long long)tile_in_request * rows_per_cta;
    const long long row_hi = min(row_lo + rows_per_cta, rows_total); // > row_lo by construction
    const int cta_limit = shift + (int)((row_hi - 1) / group);       // tokens the last row sees
    const int cnt = (cta_limit + kPage - 1) / kPage;                 // pages this CTA streams

    WarpState st;
    const int unit = warp / a.mt;  // consumer: which page slot of each stage
    const int mtile = warp % a.mt; // consumer: which 16-row tile of the CTA
    const long long warp_row = row_lo + mtile * 16;

    int producer_trips = 0; // producer lanes: iterations of the page loop that issued copies
    if (warp == kComputeWarps) {
        // ================= producer warp: page-table walk + TMA issue =========================
        const int my_slot = lane >> 1;
        const int which = lane & 1; // 0: K box, 1: V box
        const bool lane_active = my_slot < a.pps;
        const CUtensorMap *map = which == 0 ? &k_map : &v_map;
        bool bad_page = false;
        auto load_page = [&](int j) -> int {
            const int id = j < cnt ? a.indices[page_start + j] : 0;
            if (id < 0 || id >= a.max_pages) {
                bad_page = true;
                return 0;
            }
            return id;
        };
        // the first window: ids among the first 32 of the table came with the guard
        int window = __shfl_sync(0xffffffffu, head_of_table, (page_start + lane) & 31);
        if (lane >= cnt) window = 0;
        else if (page_start + lane >= 32) window = a.indices[page_start + lane];
        if (window < 0 || window >= a.max_pages) {
            bad_page = true;
            window = 0;
        }
        int window_next = load_page(32 + lane);
        const uint32_t my_full = full0 + my_slot * 8, my_empty = empty0 + my_slot * 8;
        const uint32_t my_tile = smem_u32(ring + my_slot * slot_bytes + which * (slot_bytes / 2));
        const int n_iter = (cnt + a.pps - 1) / a.pps;
        int stage = 0;
        uint32_t phase = 0;
        bool recycled = false;
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
            if (has && recycled) ok = mbar_wait(my_empty + stage * a.pps * 8, phase ^ 1);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) flags[1] = 1;
                break;
            }
            if (has && which == 0) mbar_expect_tx(bar_full, slot_bytes);
            __syncwarp();
            if (has)
                tma_load_3d(my_tile + stage * stage_bytes, map, 0, page_id * kPage, kv_head * 2,
                            bar_full);
            if (++stage == a.stages) {
                stage = 0;
                phase ^= 1;
                recycled = true;
            }
        }
        producer_trips = it;
        // the reference validates every page of the request, also those past the causal limit
        // of a row (prefill.rs:333-340): the pages this CTA does not stream are range-checked
        for (int j = cnt + lane; j < num_pages; j += 32) {
            const int id = a.indices[page_start + j];
            if (id < 0 || id >= a.max_pages) bad_page = true;
        }
        if (__any_sync(0xffffffffu, bad_page) && lane == 0) flags[0] = 1;
    } else {
        // ================= consumer warps ======================================================
        st.reset();
        // the two packed rows of this lane, their tokens and causal limits
        const long long p0 = warp_row + (lane >> 2), p1 = p0 + 8;
        const bool valid0 = p0 < row_hi, valid1 = p1 < row_hi;
        const int token0 = valid0 ? (int)(p0 / group) : 0, token1 = valid1 ? (int)(p1 / group) : 0;
        const int head0 = kv_head * group + (valid0 ? (int)(p0 % group) : 0);
        const int head1 = kv_head * group + (valid1 ? (int)(p1 % group) : 0);
        const int see0 = valid0 ? shift + token0 : 0, see1 = valid1 ? shift + token1 : 0;
        uint32_t qf[8][4];
        {
            const uint32_t *q0 = reinterpret_cast<const uint32_t *>(
                a.query + ((size_t)(qo_start + token0) * a.qh + head0) * kHeadDim);
            const uint32_t *q1 = reinterpret_cast<const uint32_t *>(
                a.query + ((size_t)(qo_start + token1) * a.qh + head1) * kHeadDim);
            const int c = lane & 3;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                qf[kk][0] = valid0 ? q0[kk * 8 + c] : 0u;
                qf[kk][1] = valid1 ? q1[kk * 8 + c] : 0u;
                qf[kk][2] = valid0 ? q0[kk * 8 + 4 + c] : 0u;
                qf[kk][3] = valid1 ? q1[kk * 8 + 4 + c] : 0u;
            }
        }
        // tokens the last row of this warp sees: pages at or past it are only handed back
        int warp_limit = max(see0, see1);
        warp_limit = max(warp_limit, __shfl_xor_sync(0xffffffffu, warp_limit, 4));
        warp_limit = max(warp_limit, __shfl_xor_sync(0xffffffffu, warp_limit, 8));
        warp_limit = max(warp_limit, __shfl_xor_sync(0xffffffffu, warp_limit, 16));

        const int my_pages = cnt > unit ? (cnt - unit + a.pps - 1) / a.pps : 0;
        const int tile_offset = unit * slot_bytes;
        const uint32_t my_full = full0 + unit * 8, my_empty = empty0 + unit * 8;
        int page_token = unit * kPage; // first logical token of the page at hand
        int stage = 0;
        uint32_t phase = 0;
        for (int it = 0; it < my_pages; ++it) {
            const bool ok = mbar_wait(my_full + stage * a.pps * 8, phase);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) flags[1] = 1;
                break;
            }
            bool wrote = false;
            if (page_token < warp_limit) {
                uint8_t *k_tile = ring + stage * stage_bytes + tile_offset;
                wrote = attend_page<true>(k_tile, k_tile + slot_bytes / 2,
                                          min(kPage, kv_len - page_token), qf, a.scale_log2, lane,
                                          st, see0 - page_token, see1 - page_token);
            }
            __syncwarp();
            if (lane == 0) {
                if (wrote) fence_proxy_async();
                mbar_arrive(my_empty + stage * a.pps * 8);
            }
            page_token += a.pps * kPage;
            if (++stage == a.stages) {
                stage = 0;
                phase ^= 1;
            }
        }
        st.finish_rows();
    }

    // ---- join: every TMA write has been consumed or abandoned; the ring becomes scratch ---------
    __syncthreads();
    if (flags[1] != 0) {
        // a wait ran out: nothing is published; the copies already on their way are waited for
        // (bounded), so that none lands in shared memory after this CTA has gone
        if (warp == kComputeWarps && (lane & 1) == 0 && (lane >> 1) < a.pps) {
            const int slot = lane >> 1;
            const int mine = cnt > slot ? (cnt - slot + a.pps - 1) / a.pps : 0;
            drain_issued_copies(full0 + slot * 8, a.pps * 8, a.stages, min(producer_trips, mine),
                                kWaitCycles);
        }
        __syncthreads();
        if (tid == 0 && a.status) atomicExch(a.status, 1);
        return;
    }
    const bool invalid_page = flags[0] != 0;

    const int populated = min(a.pps, cnt);
    if (populated > 1) {
        // warps that streamed different pages for the same rows merge their states
        float *scratch = reinterpret_cast<float *>(ring);
        if (warp < kComputeWarps && unit > 0 && unit < populated) {
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
        if (warp < kComputeWarps && unit == 0) {
            for (int k = 1; k < populated; ++k) {
                const float *other = scratch + (warp + k * a.mt) * kMergeFloatsPerWarp;
                const float om0 = other[64 * 32 + lane], om1 = other[65 * 32 + lane];
                const float ol0 = other[66 * 32 + lane], ol1 = other[67 * 32 + lane];
                // a state without tokens (normaliser 0, maximum -inf) contributes nothing; the
                // slot-0 state always holds token 0, so its maximum is finite
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

    if (warp >= kComputeWarps || unit != 0 || invalid_page) return;

    // ---- epilogue ---------------------------------------------------------------------------------
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const long long p = warp_row + (lane >> 2) + half * 8;
        if (p >= row_hi) continue;
        const size_t state =
            (size_t)(qo_start + (int)(p / group)) * a.qh + kv_head * group + (int)(p % group);
        write_final_row(a.output + state * kHeadDim, a.lse + state, lane, half, st);
    }
}

} // namespace

int configure_prefill_kernels(size_t max_dynamic_shared) {
    return cudaFuncSetAttribute(paged_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)max_dynamic_shared);
}

int launch_paged_prefill(const PrefillLaunch &launch, void *stream) {
    PrefillArgs args;
    args.query = static_cast<const __nv_bfloat16 *>(launch.query);
    args.qo_indptr = launch.qo_indptr;
    args.indptr = launch.indptr;
    args.indices = launch.indices;
    args.last = launch.last;
    args.output = static_cast<__nv_bfloat16 *>(launch.output);
    args.lse = launch.lse;
    args.status = launch.status;
    args.batch = launch.batch;
    args.nnz_qo = launch.nnz_qo;
    args.max_pages = launch.max_pages;
    args.qh = launch.qh;
    args.kvh = launch.kvh;
    args.indices_len = launch.indices_len;
    args.indices_min = launch.indices_min;
    args.mt = launch.q_tiles;
    args.pps = launch.pages_per_stage;
    args.stages = launch.stages;
    args.tiles = launch.tiles;
    args.scale_log2 = launch.scale_log2;
    args.workspace = nullptr;
    args.partitions = 1;
    args.min_chunk_blocks = 1;
    args.wait_cycles = 0; // (the tiled kernel's)
    args.test_lost_copy = 0;
    CUtensorMap k_map, v_map;
    memcpy(&k_map, launch.k_map, sizeof(k_map));
    memcpy(&v_map, launch.v_map, sizeof(v_map));
    return launch_dependent(paged_prefill_kernel, launch.grid, launch.block, launch.shared_bytes,
                            stream, k_map, v_map, args);
}

} // namespace lb
