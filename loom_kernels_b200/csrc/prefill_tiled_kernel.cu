// Paged causal prefill on the 5th-generation tensor cores (tcgen05 + TMEM), for prompts long
// enough that the operator is bound by the tensor pipe rather than by latency.
//
// Same contract as paged_prefill_kernel (prefill_kernels.cu); replaces the same reference kernels
// (crates/loom-infer-cuda/src/attention/prefill.rs:270-470,799-1170).
//
// Shape of the kernel
//   work item  = (request, KV head, tile of 128 packed (token, head-in-group) rows); one CTA each,
//                192 threads: warps 0-3 own one row per thread (row t = TMEM lane t), warp 4 issues
//                the TMA loads, warp 5 allocates TMEM and issues the MMAs.  Two CTAs share an SM
//                (about 112 KB of shared memory and 256 TMEM columns each), so one CTA's MMAs run
//                under the other's softmax and every scheduler has two softmax warps.
//   per block  = 64 KV tokens (4 pages):
//                  S = Q K^T      8 x tcgen05.mma 128x64x16 (A = Q, B = K block, both K-major in
//                                 shared memory with the 128-byte swizzle), accumulator S in TMEM
//                  softmax        each thread pulls its S row out of TMEM (tcgen05.ld), masks it
//                                 with the row's causal limit where the block crosses it, and
//                                 writes P = 2^(S - m) as BF16 pairs back into TMEM
//                                 (tcgen05.st, double-buffered); the exponent base m follows the
//                                 running maximum lazily (only a rise of more than 8 rescales O
//                                 and the normaliser, through tcgen05.ld/st)
//                  O += P V       one tcgen05.mma 128x128x16 per page (A = P from TMEM, B = the V
//                                 page, which is MN-major: 64 dims contiguous per 128-byte row),
//                                 O in TMEM
//   pipelining = K and V blocks are double-buffered by TMA; the S MMAs of block j + 1 are issued
//                before the P V MMAs of block j, so the next scores are ready when the softmax
//                warps finish the current block.
//   shared mem = Q 32 KB | K 2 x 16 KB | V 2 x 16 KB | barriers
//   TMEM       = 256 columns: S (64 x F32) | P (2 x 32 columns of BF16 pairs) | O (128 x F32)
//   split KV   = a plan with partitions > 1 gives the 64-token blocks of a tile to that many CTAs
//                (the balanced rule of the split-K contract); each writes the unnormalised state
//                [max_log2, normaliser, weighted values] of its share into a workspace and
//                prefill_merge_kernel, a second command, merges them per (query row, head).
//
// Device-resident metadata is never an error (prefill.rs:289-347).  Every mbarrier wait is bounded
// (the plan's wait limit); after a timeout every role leaves its loop -- the producer after a
// bounded wait for the copies it has in flight, the MMA warp after a bounded wait for the MMAs it
// has issued (a commit on a barrier of its own) -- and only then the CTA frees its TMEM, records a
// status word and leaves without writing.
#include <cstring>

#include "kernels.hpp"
#include "prefill_device.cuh"
#include "tcgen05_device.cuh"

namespace lb {
namespace {

using namespace dev;

constexpr int kTileRows = 128;   // packed query rows per CTA = TMEM lanes
constexpr int kBlockTokens = 64; // KV tokens per block = 4 pages
constexpr int kBlockPages = kBlockTokens / kPage;
constexpr int kQHalfBytes = kTileRows * 128;   // 64 dims (128 bytes) of the 128 query rows
constexpr int kQBytes = 2 * kQHalfBytes;       // 32 KB
constexpr int kKHalfBytes = kBlockTokens * 128; // 64 dims of the block's token rows
constexpr int kKStageBytes = 2 * kKHalfBytes;  // 16 KB
constexpr int kVStageBytes = kBlockPages * 4096; // 16 KB: per page [half][16 tokens][64 dims]
constexpr int kStages = 2;
constexpr int kThreads = 192;
constexpr uint32_t kTmemColumns = 256;         // 64 (S) + 2 x 32 (P, double-buffered) + 128 (O)
constexpr uint32_t kTmemS = 0, kTmemP = 64, kTmemO = 128;
constexpr float kRescaleThreshold = 8.0f;      // log2 domain: P stays below 2^8

// shared-memory map (offsets from the 1024-byte aligned base of dynamic shared memory)
constexpr int kOffQ = 0;
constexpr int kOffK = kOffQ + kQBytes;
constexpr int kOffV = kOffK + kStages * kKStageBytes;
constexpr int kOffBars = kOffV + kStages * kVStageBytes;
// barriers: k_full[2] k_empty[2] v_full[2] v_empty[2] s_full s_free p_full[2] p_free[2] verdict
// q_full (the Q tile is in shared memory and TMEM is allocated)
constexpr int kBarKFull = 0, kBarKEmpty = 2, kBarVFull = 4, kBarVEmpty = 6, kBarSFull = 8,
              kBarSFree = 9, kBarPFull = 10, kBarPFree = 12, kBarVerdict = 14, kBarQFull = 15,
              kBarDrain = 16, kNumBars = 17;
constexpr int kOffMisc = kOffBars + kNumBars * 8; // tmem base address, flags
constexpr int kSharedBytes = kOffMisc + 24;
static_assert(2 * (kSharedBytes + 1024) <= 233472, "two CTAs must fit one SM");

constexpr uint32_t kIdescQK = idesc(kBlockTokens, false); // B = K block, K-major, N = 64 tokens
constexpr uint32_t kIdescPV = idesc(kHeadDim, true);      // B = V page, MN-major, N = 128 dims

__global__ void __launch_bounds__(kThreads, 2)
paged_prefill_tiled_kernel(const __grid_constant__ CUtensorMap k_half_map,
                           const __grid_constant__ CUtensorMap v_map, const PrefillArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    dependent_launch_release();
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    auto wait_on = [&](uint32_t bar, uint32_t parity) { return mbar_wait(bar, parity, a.wait_cycles); };
    uint8_t *base = smem_raw;
    const uint32_t base_u32 = smem_u32(base);
    const uint32_t bars = base_u32 + kOffBars;
    volatile uint32_t *misc = reinterpret_cast<volatile uint32_t *>(base + kOffMisc);
    // misc[0] = TMEM base address, misc[1] = an out-of-range page index was seen,
    // misc[2] = a bounded wait ran out

    const int group = a.qh / a.kvh;
    const int kv_head = blockIdx.x % a.kvh;
    // late (long) tiles start first; the chunks of a tile's KV range are neighbours in the grid
    const int tile = a.tiles - 1 - (int)(blockIdx.x / a.kvh) / a.partitions;

    if (tid == 0) {
        for (int i = 0; i < kNumBars; ++i)
            mbar_init(bars + i * 8, i == kBarQFull ? 5
                                    : i == kBarSFree || i == kBarPFull || i == kBarPFull + 1 ? 4
                                                                                             : 1);
        fence_barrier_init();
        misc[1] = 0;
        misc[2] = 0;
    }
    __syncthreads(); // the barriers exist for every warp, in particular for the producer's TMA
    if (warp == 4 && lane == 0) {
        prefetch_tensormap(&k_half_map);
        prefetch_tensormap(&v_map);
    }
    dependent_launch_wait();
    // ---- guards: CTA-uniform, before any TMEM is held ---------------------------------------------
    if ((base_u32 & 1023u) != 0) { // the swizzled tiles need the 1024-byte alignment asked for
        if (tid == 0 && a.status) atomicExch(a.status, 2);
        return;
    }
    // one round trip to the metadata (prefill.rs:289-347); the producer warp also gets the first 32
    // page ids of the table
    TileOwner owner;
    int head_of_table;
    if (!prefill_guard(a, group, kTileRows, tile, lane, warp == 4, owner, head_of_table)) return;
    const int tile_in_request = owner.tile_in_request;
    const int qo_start = owner.qo_start, qo_end = owner.qo_end;
    int page_start = owner.page_start;
    const int page_end = owner.page_end, tail = owner.tail;
    const int qo_len = qo_end - qo_start;
    const int request_pages = page_end - page_start;
    const long long kv_len_wide = (long long)(request_pages - 1) * kPage + tail;
    if (qo_len > kv_len_wide) return; // prefill.rs:343-347
    const int kv_len = (int)kv_len_wide;
    const int shift = kv_len - qo_len + 1; // the row of token t sees logical tokens [0, shift + t)
    const long long rows_total = (long long)qo_len * group;
    const long long row_lo = (long long)tile_in_request * kTileRows;
    const long long row_hi = min(row_lo + kTileRows, rows_total);
    const int cta_limit = shift + (int)((row_hi - 1) / group); // tokens the last row sees
    // this CTA's share of the tile's 64-token blocks: the balanced rule of the split-K contract
    // (crates/loom-infer/src/attention/single_decode/mod.rs:171-185)
    const int chunk = (int)(blockIdx.x / a.kvh) % a.partitions;
    const int tile_pages = (cta_limit + kPage - 1) / kPage; // pages the tile's last row sees
    const int tile_blocks = (tile_pages + kBlockPages - 1) / kBlockPages;
    const int chunks = chunks_of_tile(tile_blocks, a.partitions, a.min_chunk_blocks);
    if (chunk >= chunks) return; // the tile is too short for this many chunks: nothing to do
    const int block0 = chunk * (tile_blocks / chunks) + min(chunk, tile_blocks % chunks);
    const int blocks = tile_blocks / chunks + (chunk < tile_blocks % chunks ? 1 : 0);
    // from here on pages, blocks and tokens are counted from the start of the share
    page_start += block0 * kBlockPages;
    const int num_pages = request_pages - block0 * kBlockPages; // up to the request's last page
    const int cnt = min(tile_pages - block0 * kBlockPages, blocks * kBlockPages); // pages streamed
    const int shift_here = shift - block0 * kBlockTokens;

    // this thread's packed row (warps 0-3)
    const long long my_row = row_lo + tid;
    const bool row_valid = tid < kTileRows && my_row < row_hi;
    const int my_token = row_valid ? (int)(my_row / group) : 0;
    const int my_head = kv_head * group + (row_valid ? (int)(my_row % group) : 0);
    const size_t my_state = (size_t)(qo_start + my_token) * a.qh + my_head;
    // the state of this row and chunk in the workspace (plans with more than one chunk)
    auto partial_state = [&]() -> float * {
        const int chunk = (int)(blockIdx.x / a.kvh) % a.partitions;
        return a.workspace + (my_state * a.partitions + chunk) * kStateWidth;
    };

    // ---- TMEM, Q tile ---------------------------------------------------------------------------------
    // The producer warp does not wait for either: its first K/V boxes are in flight while the
    // other warps are here.
    if (warp == 5) {
        tmem_alloc(base_u32 + kOffMisc, kTmemColumns);
        tmem_relinquish();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + kBarQFull * 8);
    }
    if (tid < kTileRows) {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.query + my_state * kHeadDim);
#pragma unroll
        for (int chunk = 0; chunk < 16; ++chunk) {
            const uint4 value = row_valid ? __ldg(src + chunk) : make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4 *>(base + kOffQ + (chunk >> 3) * kQHalfBytes +
                                       swizzled(tid, chunk & 7)) = value;
        }
        fence_proxy_async(); // the MMAs read Q through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + kBarQFull * 8);
    }
    bool q_ready = true;
    if (warp != 4) {
        q_ready = __all_sync(0xffffffffu, wait_on(bars + kBarQFull * 8, 0));
        tc_fence_after();
    }
    const uint32_t tmem_base = misc[0]; // not used by the producer warp
    const uint32_t tmem_s = tmem_base + kTmemS; // scores of the block at hand
    const uint32_t tmem_p = tmem_base + kTmemP; // BF16 weights of the block, two per column
    const uint32_t tmem_o = tmem_base + kTmemO; // output accumulator

    if (warp == 4) {
        // ================= producer: page-table walk + TMA ==========================================
        // lanes 0-7: the two 64-dim halves of the K rows of page lane / 2 (2 KB boxes: the K block
        // must be one uniform 64-token operand); lanes 8-11: the V page lane - 8 (4 KB box)
        const bool is_k = lane < 8;
        const int slot = is_k ? lane >> 1 : lane - 8;
        const int half = lane & 1;
        const bool lane_active = lane < 12;
        bool bad_page = false;
        // Page ids travel in windows of 32 (one per lane): win0 holds the window of the block whose
        // values are loaded next, win1 the one after it, fetched a whole window ahead, so that no
        // load of the page table sits between a barrier and the TMA it releases.  An id out of
        // range is replaced by page 0 when it is used and poisons the request.
        auto load_window = [&](int w) -> int {
            const int page = w * 32 + lane;
            return page < cnt ? a.indices[page_start + page] : 0;
        };
        int first_window = 0;
        // the first window: ids among the first 32 of the table came with the guard
        int win0 = __shfl_sync(0xffffffffu, head_of_table, (page_start + lane) & 31);
        if (lane >= cnt) win0 = 0;
        else if (page_start + lane >= 32) win0 = a.indices[page_start + lane];
        int win1 = load_window(1);
        auto id_of_page = [&](int page) -> int {
            const int from0 = __shfl_sync(0xffffffffu, win0, page & 31);
            const int from1 = __shfl_sync(0xffffffffu, win1, page & 31);
            const int id = (page >> 5) == first_window ? from0 : from1;
            if (id < 0 || id >= a.max_pages) {
                bad_page = true;
                return 0;
            }
            return id;
        };
        auto pages_in = [&](int block) { return min(kBlockPages, cnt - block * kBlockPages); };
        auto load_k = [&](int block, int id) {
            const int stage = block & 1;
            if (lane == 0)
                mbar_expect_tx(bars + (kBarKFull + stage) * 8,
                               pages_in(block) * 4096 + (block == 0 && a.test_lost_copy ? 16 : 0));
            __syncwarp();
            if (is_k && block * kBlockPages + slot < cnt)
                tma_load_3d(base_u32 + kOffK + stage * kKStageBytes + half * kKHalfBytes + slot * 2048,
                            &k_half_map, 0, id * kPage, kv_head * 2 + half,
                            bars + (kBarKFull + stage) * 8);
        };
        auto load_v = [&](int block, int id) {
            const int stage = block & 1;
            if (lane == 8) mbar_expect_tx(bars + (kBarVFull + stage) * 8, pages_in(block) * 4096);
            __syncwarp();
            if (lane_active && !is_k && block * kBlockPages + slot < cnt)
                tma_load_3d(base_u32 + kOffV + stage * kVStageBytes + slot * 4096, &v_map, 0,
                            id * kPage, kv_head * 2, bars + (kBarVFull + stage) * 8);
        };
        // Keys run two blocks ahead of the scores that consume them, values follow the P V MMAs:
        // iteration j loads V(j) as soon as P V (j - 2) has freed its stage and K(j + 2) as soon
        // as S(j) has -- the order in which the MMA warp completes them.
        const int k_slot = lane >> 1, v_slot = lane - 8; // the page of a block this lane loads
        load_k(0, id_of_page(k_slot));
        if (blocks > 1) load_k(1, id_of_page(kBlockPages + k_slot));
        int k_issued = blocks > 1 ? 1 : 0, v_issued = -1; // the last blocks whose copies were issued
        bool gave_up = false;
        for (int j = 0; j < blocks; ++j) {
            const int stage = j & 1;
            const int v_id = id_of_page(j * kBlockPages + v_slot);
            const int k_id = id_of_page((j + 2) * kBlockPages + k_slot);
            bool ok = j < kStages || wait_on(bars + (kBarVEmpty + stage) * 8, ((j >> 1) + 1) & 1);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) misc[2] = 1;
                gave_up = true;
                break;
            }
            load_v(j, v_id);
            v_issued = j;
            if (j + 2 < blocks) {
                ok = wait_on(bars + (kBarKEmpty + stage) * 8, (j >> 1) & 1); // S(j) has completed
                if (__any_sync(0xffffffffu, !ok)) {
                    if (lane == 0) misc[2] = 1;
                    gave_up = true;
                    break;
                }
                load_k(j + 2, k_id);
                k_issued = j + 2;
            }
            if ((((j + 1) * kBlockPages) >> 5) != first_window) { // the values enter the next window
                ++first_window;
                win0 = win1;
                win1 = load_window(first_window + 1);
            }
        }
        if (gave_up && lane < 4) {
            // A wait ran out: before this CTA frees its TMEM and leaves, the copies already on
            // their way are waited for (bounded again), so that none lands in shared memory the
            // next CTA may own.  Lanes 0, 1: the K stages; lanes 2, 3: the V stages; each waits
            // for the last block issued into its stage.
            const int stage = lane & 1;
            const int issued = lane < 2 ? k_issued : v_issued;
            const int block = issued >= 0 && (issued & 1) != stage ? issued - 1 : issued;
            if (block >= 0)
                (void)wait_on(bars + ((lane < 2 ? kBarKFull : kBarVFull) + stage) * 8,
                              (block >> 1) & 1);
        }
        __syncwarp();
        // the reference validates every page of the request, also those past the causal limit of
        // a row (prefill.rs:333-340): the pages this CTA does not stream are range-checked
        for (int j = cnt + lane; j < num_pages; j += 32) {
            const int id = a.indices[page_start + j];
            if (id < 0 || id >= a.max_pages) bad_page = true;
        }
        if (__any_sync(0xffffffffu, bad_page) && lane == 0) misc[1] = 1;
        __syncwarp();
        // the verdict on the request's pages is final: the epilogue warps wait for it
        if (lane == 0) mbar_arrive(bars + kBarVerdict * 8);
    } else if (warp == 5) {
        // ================= MMA issue =================================================================
        // order: S(0), S(1), PV(0), S(2), PV(1), ... so that the scores of the next block are ready
        // when the softmax warps finish the current one
        // descriptors of the first tile of each operand; the others differ in the start address
        // field only (bytes >> 4, no carry out of its 14 bits inside shared memory)
        const uint64_t q_desc0 = smem_desc(base_u32 + kOffQ, 16, 1024);
        const uint64_t k_desc0 = smem_desc(base_u32 + kOffK, 16, 1024);
        const uint64_t v_desc0 = smem_desc(base_u32 + kOffV, 2048, 1024);
        auto issue_pv = [&](int i) -> bool {
            const int stage = i & 1, buffer = i & 1;
            bool ok = wait_on(bars + (kBarPFull + buffer) * 8, (i >> 1) & 1);
            ok = wait_on(bars + (kBarVFull + stage) * 8, (i >> 1) & 1) && ok;
            if (!ok) return false;
            tc_fence_after();
            const int pages_here = min(kBlockPages, cnt - i * kBlockPages);
            if (elect_one()) {
#pragma unroll
                for (int p = 0; p < kBlockPages; ++p) {
                    if (p < pages_here)
                        umma_bf16_ts(tmem_o, tmem_p + buffer * 32 + p * 8,
                                     v_desc0 + (uint64_t)((stage * kVStageBytes + p * 4096) >> 4),
                                     kIdescPV, (i > 0 || p > 0) ? 1u : 0u);
                }
                umma_commit(bars + (kBarPFree + buffer) * 8);
                umma_commit(bars + (kBarVEmpty + stage) * 8);
            }
            __syncwarp();
            return true;
        };
        bool ok = q_ready;
        for (int j = 0; j < blocks && ok; ++j) {
            const int stage = j & 1;
            ok = wait_on(bars + (kBarKFull + stage) * 8, (j >> 1) & 1);
            if (ok && j > 0) ok = wait_on(bars + kBarSFree * 8, (j - 1) & 1);
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    umma_bf16(tmem_s,
                              q_desc0 + (uint64_t)(((kk >> 2) * kQHalfBytes + (kk & 3) * 32) >> 4),
                              k_desc0 + (uint64_t)((stage * kKStageBytes + (kk >> 2) * kKHalfBytes +
                                                    (kk & 3) * 32) >> 4),
                              kIdescQK, kk > 0 ? 1u : 0u);
                umma_commit(bars + kBarSFull * 8);
                umma_commit(bars + (kBarKEmpty + stage) * 8);
            }
            __syncwarp();
            if (j > 0) ok = issue_pv(j - 1);
        }
        if (ok) ok = issue_pv(blocks - 1);
        if (!ok) {
            // a wait ran out: the MMAs already issued complete before the TMEM goes (the commit
            // arrives on the barrier when every earlier tcgen05 operation of the thread has)
            if (lane == 0) misc[2] = 1;
            if (elect_one()) umma_commit(bars + kBarDrain * 8);
            __syncwarp();
            (void)wait_on(bars + kBarDrain * 8, 0);
        }
    } else {
        // ================= softmax + epilogue: thread t owns packed row t ===========================
        // tokens of the share this row sees (none when negative)
        const int see = row_valid ? shift_here + my_token : 0;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float scale = a.scale_log2;
        float m_used = -INFINITY; // exponent base of P, O and the normaliser
        float l = 0.0f;
        bool ok = q_ready;
        for (int j = 0; q_ready && j < blocks; ++j) {
            ok = wait_on(bars + kBarSFull * 8, j & 1);
            if (__any_sync(0xffffffffu, !ok)) break;
            tc_fence_after();
            float s[kBlockTokens]; // raw dot products
            tmem_load64(tmem_s + lane_base, s);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + kBarSFree * 8); // S may be overwritten by block j + 1
            // the row's causal limit inside this block; columns past it (which also covers stale
            // or garbage key rows) are masked.  Most blocks lie wholly below the limit.
            const int limit = see - j * kBlockTokens;
            if (!__all_sync(0xffffffffu, limit >= kBlockTokens)) {
#pragma unroll
                for (int i = 0; i < kBlockTokens; ++i) s[i] = i < limit ? s[i] : -INFINITY;
            }
            // four chains of three-input maxima: 32 instructions, eight deep
            float chain[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) chain[c] = fmaxf(s[c * 16], s[c * 16 + 1]);
#pragma unroll
            for (int i = 2; i < 16; i += 2) {
#pragma unroll
                for (int c = 0; c < 4; ++c) chain[c] = max3(chain[c], s[c * 16 + i], s[c * 16 + i + 1]);
            }
            // scale > 0; -inf stays -inf
            const float mx = fmaxf(fmaxf(chain[0], chain[1]), fmaxf(chain[2], chain[3])) * scale;
            // the exponent base follows the maximum lazily: P <= 2^8 keeps BF16 P and the F32
            // normaliser exact enough, and most blocks skip the TMEM round trip of O
            const bool rescale = mx > m_used + kRescaleThreshold ||
                                 (m_used == -INFINITY && mx > -INFINITY);
            if (__any_sync(0xffffffffu, rescale)) {
                const float m_new = rescale ? mx : m_used;
                const float alpha = rescale ? fast_exp2(m_used - m_new) : 1.0f; // 0 from -inf
                l *= alpha;
                m_used = m_new;
                if (j > 0) {
                    // O holds blocks 0..j-1 once P V (j - 1) has completed
                    ok = wait_on(bars + (kBarPFree + ((j - 1) & 1)) * 8, ((j - 1) >> 1) & 1);
                    if (__any_sync(0xffffffffu, !ok)) break;
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float part[32];
                        tmem_load32(tmem_o + lane_base + c * 32, part);
#pragma unroll
                        for (int i = 0; i < 32; ++i) part[i] *= alpha;
                        tmem_store32(tmem_o + lane_base + c * 32, part);
                    }
                    tmem_store_wait();
                }
            }
            const float neg_base = m_used == -INFINITY ? 0.0f : -m_used;
            // The weights are double-buffered, and this buffer is free: P V (j - 2) was issued
            // before S(j) by the same elected thread, and the commit behind s_full(j), which this
            // warp has seen, covers every MMA that thread issued before it.
            float packed[kBlockTokens / 2]; // BF16 pairs (token 2c in the low half), as raw bits
            // the scaling and the row sum on pairs (fma / add .f32x2: one instruction per two
            // weights), the exponentials one by one
            const float2 scale2 = make_float2(scale, scale), base2 = make_float2(neg_base, neg_base);
            float2 sums[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f),
                              make_float2(0.f, 0.f)};
#pragma unroll
            for (int i = 0; i < kBlockTokens / 2; ++i) {
                const float2 x = fma2(make_float2(s[2 * i], s[2 * i + 1]), scale2, base2);
                const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                sums[i & 3] = add2(sums[i & 3], p);
                packed[i] = __uint_as_float(pack_bf16(p.x, p.y));
            }
            tmem_store32(tmem_p + (j & 1) * 32 + lane_base, packed);
            tmem_store_wait();
            const float2 total = add2(add2(sums[0], sums[1]), add2(sums[2], sums[3]));
            l += total.x + total.y;
            // rows of the request's last page past its length may hold anything (0 * NaN): zero
            // them in the V block before the MMA reads it
            const int last_page = num_pages - 1;
            const bool zero_tail = tail < kPage && last_page / kBlockPages == j && last_page < cnt;
            if (zero_tail) {
                ok = wait_on(bars + (kBarVFull + (j & 1)) * 8, (j >> 1) & 1);
                if (__any_sync(0xffffffffu, !ok)) break;
                uint8_t *v_page =
                    base + kOffV + (j & 1) * kVStageBytes + (last_page % kBlockPages) * 4096;
                for (int i = tid; i < (kPage - tail) * 16; i += kTileRows) {
                    const int row = tail + (i >> 4), c = i & 15;
                    *reinterpret_cast<uint4 *>(v_page + (c >> 3) * 2048 + row * 128 + (c & 7) * 16) =
                        make_uint4(0, 0, 0, 0);
                }
            }
            if (zero_tail) fence_proxy_async(); // the zeroed V rows become visible to the MMA
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + (kBarPFull + (j & 1)) * 8);
        }
        if (__any_sync(0xffffffffu, !ok)) {
            if (lane == 0) misc[2] = 1;
        } else {
            // every P V has completed once the last one has
            ok = wait_on(bars + (kBarPFree + ((blocks - 1) & 1)) * 8, ((blocks - 1) >> 1) & 1);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) misc[2] = 1;
            } else {
                tc_fence_after();
                const bool verdict = wait_on(bars + kBarVerdict * 8, 0); // the producer's page scan
                const bool settled = verdict && row_valid && misc[2] == 0;
                float *my_partial = chunks > 1 ? partial_state() : nullptr;
                const bool publish = settled && misc[1] == 0 && my_partial == nullptr;
                const float inv = 1.0f / l;
                uint4 *dst = reinterpret_cast<uint4 *>(a.output + my_state * kHeadDim);
                if (settled && my_partial != nullptr) {
                    // the unnormalised state of this chunk: [maximum, normaliser, weighted values];
                    // a row that saw nothing here is an empty state, a bad page id poisons it
                    *reinterpret_cast<float2 *>(my_partial) =
                        make_float2(l > 0.0f ? m_used : 0.0f, misc[1] != 0 ? -1.0f : l);
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float part[32];
                    tmem_load32(tmem_o + lane_base + c * 32, part);
                    if (settled && my_partial != nullptr) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            *reinterpret_cast<float2 *>(my_partial + 2 + c * 32 + 2 * i) =
                                make_float2(part[2 * i], part[2 * i + 1]);
                    }
                    if (publish) {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            dst[c * 4 + i] = make_uint4(
                                pack_bf16(part[i * 8] * inv, part[i * 8 + 1] * inv),
                                pack_bf16(part[i * 8 + 2] * inv, part[i * 8 + 3] * inv),
                                pack_bf16(part[i * 8 + 4] * inv, part[i * 8 + 5] * inv),
                                pack_bf16(part[i * 8 + 6] * inv, part[i * 8 + 7] * inv));
                    }
                }
                if (publish) a.lse[my_state] = m_used + log2f(l);
            }
        }
    }

    // ---- join: all tcgen05 work of this CTA has completed or been abandoned ------------------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 5) tmem_dealloc(tmem_base, kTmemColumns);
    if (tid == 0 && misc[2] != 0 && a.status) atomicExch(a.status, 1);
    // a chunk that gave up on a wait poisons its states, so that the merge publishes nothing
    if (misc[2] != 0 && chunks > 1 && row_valid) partial_state()[1] = -1.0f;
}

// Merges the chunk states of one (query row, query head) per warp and writes BF16 O + log2 LSE
// (merge_partial, publish_merged).  The row's request is checked again here -- the global checks,
// every query range up to the owner, its page range and qo_len <= kv_len (prefill.rs:289-347) --
// because a CTA of the main kernel that rejects a request writes no state; a bad page id arrives
// as a poisoned state.  The number of chunks of the row's tile is recomputed from the metadata
// as the main kernel computed it; a tile of one chunk was finished there.
__global__ void __launch_bounds__(128, 5)
prefill_merge_kernel(const float *__restrict__ workspace, __nv_bfloat16 *output, float *lse,
                     const int32_t *qo_indptr, const int32_t *indptr, const int32_t *last, int batch,
                     int nnz_qo, int qh, int kvh, int partitions, int min_chunk_blocks,
                     int indices_min, int indices_len) {
    dependent_launch_release();
    const int lane = threadIdx.x & 31;
    const long long state = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (state >= (long long)nnz_qo * qh) return;
    const int row = (int)(state / qh);
    dependent_launch_wait(); // the chunk states are complete and visible
    // one round trip for the metadata, one for the states
    const int qo_first = qo_indptr[0], qo_total = qo_indptr[batch];
    const int global_end = indptr[batch], first = indptr[0];
    RowOwner o;
    const bool located = locate_row(qo_indptr, indptr, last, batch, nnz_qo, row, lane, o);
    if (!located || qo_first != 0 || qo_total != nnz_qo) return;
    // request_metadata_valid and qo_len <= kv_len
    const int qo_len = o.qo_end - o.qo_start;
    const long long kv_len = (long long)(o.page_end - o.page_start - 1) * kPage + o.tail;
    if (first != 0 || global_end < indices_min || global_end > indices_len || o.page_start < 0 ||
        o.page_end <= o.page_start || o.page_end > global_end || o.tail < 1 || o.tail > kPage ||
        qo_len > kv_len)
        return;
    // the row's tile: 128 packed (token, head-in-group) rows of one KV head (32-bit arithmetic:
    // a plan admits at most 2^32 states)
    const unsigned group = (unsigned)(qh / kvh);
    const unsigned packed = (unsigned)(row - o.qo_start) * group + ((unsigned)state % (unsigned)qh) % group;
    const unsigned rows_total = (unsigned)qo_len * group;
    const unsigned tile_end = (packed / kTileRows + 1) * kTileRows;
    const unsigned row_hi = tile_end < rows_total ? tile_end : rows_total;
    const int tile_limit = (int)(kv_len - qo_len + 1) + (int)((row_hi - 1) / group); // tokens seen
    const int tile_pages = (tile_limit + kPage - 1) / kPage;
    const int chunks = chunks_of_tile((tile_pages + kBlockPages - 1) / kBlockPages, partitions,
                                      min_chunk_blocks);
    if (chunks == 1) return; // written by the main kernel
    const float *st = workspace + (size_t)state * partitions * kStateWidth;
    float top, norm;
    float4 acc;
    if (!merge_partial([&](int p) { return st + (size_t)p * kStateWidth; }, chunks, lane, top, norm,
                       acc))
        return; // a chunk met a page id out of range
    if (!(norm > 0.0f)) return;
    publish_merged(top, norm, acc, lane, output + (size_t)state * kHeadDim, lse + state);
}

} // namespace

int configure_prefill_tiled_kernel(size_t max_dynamic_shared) {
    if ((size_t)kSharedBytes > max_dynamic_shared) return cudaErrorInvalidValue;
    int rc = cudaFuncSetAttribute(paged_prefill_tiled_kernel,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, kSharedBytes);
    if (rc) return rc;
    // two CTAs per SM need the largest shared-memory carve-out
    return cudaFuncSetAttribute(paged_prefill_tiled_kernel,
                                cudaFuncAttributePreferredSharedMemoryCarveout,
                                cudaSharedmemCarveoutMaxShared);
}

int prefill_tiled_shared_bytes() { return kSharedBytes; }

int launch_paged_prefill_tiled(const PrefillLaunch &launch, void *stream) {
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
    args.mt = 8;
    args.pps = kBlockPages;
    args.stages = kStages;
    args.tiles = launch.tiles;
    args.scale_log2 = launch.scale_log2;
    args.workspace = launch.workspace;
    args.partitions = launch.partitions > 1 ? launch.partitions : 1;
    args.min_chunk_blocks = launch.min_chunk_blocks > 1 ? launch.min_chunk_blocks : 1;
    args.wait_cycles = launch.wait_cycles > 0 ? launch.wait_cycles : kWaitCycles;
    args.test_lost_copy = launch.test_lost_copy;
    CUtensorMap k_half_map, v_map;
    memcpy(&k_half_map, launch.k_map, sizeof(k_half_map));
    memcpy(&v_map, launch.v_map, sizeof(v_map));
    return launch_dependent(paged_prefill_tiled_kernel, launch.grid, kThreads, kSharedBytes, stream,
                            k_half_map, v_map, args);
}

int launch_prefill_merge(const PrefillLaunch &launch, void *stream) {
    const long long states = (long long)launch.nnz_qo * launch.qh;
    return launch_dependent(prefill_merge_kernel, (uint32_t)((states + 3) / 4), 128, 0, stream,
                            (const float *)launch.workspace,
                            static_cast<__nv_bfloat16 *>(launch.output), launch.lse,
                            launch.qo_indptr, launch.indptr, launch.last, launch.batch,
                            launch.nnz_qo, launch.qh, launch.kvh, launch.partitions,
                            launch.min_chunk_blocks > 1 ? launch.min_chunk_blocks : 1,
                            launch.indices_min, launch.indices_len);
}

} // namespace lb
