// Paged decode attention for sm_100a: BF16 NHD, head dim 128, page size 16.
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
//   math       = each consumer warp owns one unit slot of every stage and the whole GQA group
//                of that KV head as the M=16 rows of mma.sync.m16n8k16 (BF16 in, F32 out):
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
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.hpp"

namespace lb {
namespace {

constexpr int kHeadDim = 128;
constexpr int kPage = 16;
constexpr int kStateWidth = 130;
constexpr int kComputeWarps = 8;
constexpr int kUnitBytes = 8192;  // K (16 x 256 B) + V (16 x 256 B) of one (page, KV head)
constexpr int kBoxBytes = 2048;   // one TMA box: 16 tokens x 64 dims x 2 B
constexpr int kMergeFloatsPerWarp = 68 * 32; // 64 accumulators + m[2] + l[2], lane-major
constexpr long long kWaitCycles = 4000000000ll; // ~2 s at 2 GHz; waits normally take microseconds

struct DecodeArgs {
    const __nv_bfloat16 *query;
    const int32_t *indptr, *indices, *last;
    __nv_bfloat16 *output;
    float *lse;
    float *workspace;
    int32_t *status;
    int32_t batch, max_pages, qh, kvh, indices_len;
    int32_t hc, pps, mt, qb, partitions, stages;
    float scale_log2;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return done != 0;
}
// Bounded wait: false after kWaitCycles without the phase completing.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int spin = 0; spin < 256; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - start > kWaitCycles) return false;
    }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1,
                                            uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1,
                                                  uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// Per-request metadata guard, decode.rs:234-248 / :426-437.
__device__ __forceinline__ bool request_metadata_valid(const int32_t *indptr, const int32_t *last,
                                                       int batch, int indices_len, int request,
                                                       int &page_start, int &page_end, int &tail) {
    const int global_end = indptr[batch];
    page_start = indptr[request];
    page_end = indptr[request + 1];
    tail = last[request];
    return indptr[0] == 0 && global_end >= 0 && global_end == indices_len && page_start >= 0 &&
           page_end > page_start && page_end <= global_end && tail >= 1 && tail <= kPage;
}

__global__ void __launch_bounds__((kComputeWarps + 1) * 32, 1)
paged_decode_kernel(const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const DecodeArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    const int units = kComputeWarps / a.mt;
    const int stage_bytes = units * kUnitBytes;
    // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits 7..9
    uint8_t *ring = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int slot_bytes = a.hc * kUnitBytes; // one page of the CTA's heads: K box then V box
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + a.stages * stage_bytes);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + a.stages * a.pps * 8;
    volatile int *flags = reinterpret_cast<volatile int *>(bars + 2 * a.stages * a.pps);
    // flags[0] = an out-of-range page index was seen; flags[1] = a bounded wait ran out

    // ---- work item --------------------------------------------------------------------------
    const int group = a.qh / a.kvh;
    const int head_blocks = a.kvh / a.hc;
    int item = blockIdx.x;
    const int hb = item % head_blocks; item /= head_blocks;
    const int qb = item % a.qb; item /= a.qb;
    const int part = item % a.partitions;
    const int request = item / a.partitions;
    if (request >= a.batch) return;

    int page_start, page_end, tail;
    if (!request_metadata_valid(a.indptr, a.last, a.batch, a.indices_len, request, page_start,
                                page_end, tail))
        return;
    const int num_pages = page_end - page_start;
    const int kv_len = (num_pages - 1) * kPage + tail;
    // balanced page partition (single_decode/mod.rs:171-185 applied to pages)
    const int base = num_pages / a.partitions, rem = num_pages % a.partitions;
    const int pg0 = part * base + min(part, rem);
    const int cnt = base + (part < rem ? 1 : 0);
    const int chunk_end_token = min((pg0 + cnt) * kPage, kv_len);
    const int rows_per_block = 16 * a.mt;

    if (cnt == 0) {
        // a chunk without pages: the empty state [0, 0, 0...] the merge skips
        const int row_lo = qb * rows_per_block;
        const int row_hi = min(group, row_lo + rows_per_block);
        const int rows = max(0, row_hi - row_lo);
        for (int i = tid; i < a.hc * rows * kStateWidth; i += blockDim.x) {
            const int e = i % kStateWidth;
            const int row = (i / kStateWidth) % rows;
            const int h = i / (kStateWidth * rows);
            const int qhead = (hb * a.hc + h) * group + row_lo + row;
            a.workspace[((size_t)(request * a.qh + qhead) * a.partitions + part) * kStateWidth + e] =
                0.0f;
        }
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < a.stages * a.pps; ++i) {
            mbar_init(full0 + i * 8, 1);
            mbar_init(empty0 + i * 8, a.hc * a.mt);
        }
        flags[0] = 0;
        flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int n_iter = (cnt + a.pps - 1) / a.pps;

    // consumer state (declared here so the epilogue after the join can use it)
    float acc[16][4];
    float row_max[2] = {-INFINITY, -INFINITY};
    float row_sum[2] = {0.0f, 0.0f};
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
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&k_map) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&v_map) : "memory");
        }
        bool bad_page = false;
        auto load_page = [&](int j) -> int {
            if (j >= cnt) return 0;
            const int id = a.indices[page_start + pg0 + j];
            if (id < 0 || id >= a.max_pages) {
                bad_page = true;
                return 0;
            }
            return id;
        };
        int window = load_page(lane);
        int window_next = load_page(32 + lane);
        for (int it = 0; it < n_iter; ++it) {
            const int first = it * a.pps;
            if (it > 0 && (first & 31) == 0) {
                window = window_next;
                window_next = load_page(first + 32 + lane);
            }
            const int stage = it % a.stages;
            const int round = it / a.stages;
            const int slot = first + my_slot;
            const int page_id = __shfl_sync(0xffffffffu, window, slot & 31);
            const bool has = lane_active && slot < cnt;
            const uint32_t bar_full = full0 + (stage * a.pps + my_slot) * 8;
            const uint32_t bar_empty = empty0 + (stage * a.pps + my_slot) * 8;
            bool ok = true;
            if (has && round > 0) ok = mbar_wait(bar_empty, (round - 1) & 1);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) flags[1] = 1;
                break;
            }
#if defined(LB_PROBE) && LB_PROBE == 2
            if (has && which == 0) mbar_arrive(bar_full); // probe: no loads, consumers run on stale tiles
            continue;
#endif
            if (has && which == 0) mbar_expect_tx(bar_full, slot_bytes);
            __syncwarp();
            if (has)
                tma_load_3d(smem_u32(ring + stage * stage_bytes + my_slot * slot_bytes +
                                     which * (slot_bytes / 2)),
                            map, 0, page_id * kPage, z, bar_full);
        }
        if (__any_sync(0xffffffffu, bad_page) && lane == 0) flags[0] = 1;
    } else {
        // ================= consumer warps ======================================================
#pragma unroll
        for (int i = 0; i < 16; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

        const int kv_head = hb * a.hc + head_in_cta;
        const int g0 = qb * rows_per_block + mtile * 16 + (lane >> 2);
        const int g1 = g0 + 8;
        const bool valid0 = g0 < group, valid1 = g1 < group;
        uint32_t qf[8][4];
        {
            const uint32_t *q0 = reinterpret_cast<const uint32_t *>(
                a.query + ((size_t)request * a.qh + (size_t)kv_head * group + g0) * kHeadDim);
            const uint32_t *q1 = q0 + 8 * kHeadDim / 2;
            const int c = lane & 3;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                qf[kk][0] = valid0 ? q0[kk * 8 + c] : 0u;
                qf[kk][1] = valid1 ? q1[kk * 8 + c] : 0u;
                qf[kk][2] = valid0 ? q0[kk * 8 + 4 + c] : 0u;
                qf[kk][3] = valid1 ? q1[kk * 8 + 4 + c] : 0u;
            }
        }
        // per-lane ldmatrix row/column selectors (see the layout notes at the top of the file)
        const int k_tok = ((lane >> 4) << 3) + (lane & 7);
        const int k_hi = (lane >> 3) & 1;
        const int v_tok = (((lane >> 3) & 1) << 3) + (lane & 7);
        const int v_hi = lane >> 4;

        for (int it = 0; it < n_iter; ++it) {
            const int slot = it * a.pps + page_slot0;
            if (slot >= cnt) continue;
            const int stage = it % a.stages;
            const int round = it / a.stages;
            const uint32_t bar_full = full0 + (stage * a.pps + page_slot0) * 8;
            const uint32_t bar_empty = empty0 + (stage * a.pps + page_slot0) * 8;
            const bool ok = mbar_wait(bar_full, round & 1);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) flags[1] = 1;
                break;
            }
            uint8_t *slot_base = ring + stage * stage_bytes + page_slot0 * slot_bytes;
            uint8_t *v_rows = slot_base + slot_bytes / 2 + head_in_cta * 2 * kBoxBytes;
            const uint32_t k_tile = smem_u32(slot_base + head_in_cta * 2 * kBoxBytes);
            const uint32_t v_tile = smem_u32(v_rows);
            const int valid_tokens = min(kPage, chunk_end_token - (pg0 + slot) * kPage);
            if (valid_tokens < kPage) {
                // rows past the request's length hold whatever the pool holds; zero the V rows so
                // that 0 * garbage cannot produce NaN (their scores are masked below)
                for (int i = lane; i < (kPage - valid_tokens) * 16; i += 32) {
                    const int row = valid_tokens + (i >> 4);
                    const int c = i & 15;
                    *reinterpret_cast<uint4 *>(v_rows + (c >> 3) * kBoxBytes + row * 128 +
                                               (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }

#if defined(LB_PROBE) && LB_PROBE == 1
            __syncwarp(); // probe: no math, the tile is released at once
            if (lane == 0) mbar_arrive(bar_empty);
            row_sum[0] = 1.0f; row_sum[1] = 1.0f; row_max[0] = 0.0f; row_max[1] = 0.0f;
            continue;
#endif
            // ---- S = Q K^T : 16 rows x 16 tokens ------------------------------------------------
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const int chunk = ((kk & 3) << 1) + k_hi;
                const uint32_t addr = k_tile + (kk >> 2) * kBoxBytes + k_tok * 128 +
                                      ((chunk ^ (k_tok & 7)) << 4);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(addr, b0, b1, b2, b3);
                mma_bf16(s0, qf[kk], b0, b1);
                mma_bf16(s1, qf[kk], b2, b3);
            }
            // ---- online softmax (log2 domain) ---------------------------------------------------
            const int t0 = (lane & 3) * 2;
            float x00 = s0[0] * a.scale_log2, x01 = s0[1] * a.scale_log2;
            float x02 = s0[2] * a.scale_log2, x03 = s0[3] * a.scale_log2;
            float x10 = s1[0] * a.scale_log2, x11 = s1[1] * a.scale_log2;
            float x12 = s1[2] * a.scale_log2, x13 = s1[3] * a.scale_log2;
            if (valid_tokens < kPage) {
                if (t0 >= valid_tokens) { x00 = -INFINITY; x02 = -INFINITY; }
                if (t0 + 1 >= valid_tokens) { x01 = -INFINITY; x03 = -INFINITY; }
                if (t0 + 8 >= valid_tokens) { x10 = -INFINITY; x12 = -INFINITY; }
                if (t0 + 9 >= valid_tokens) { x11 = -INFINITY; x13 = -INFINITY; }
            }
            float m0 = fmaxf(fmaxf(x00, x01), fmaxf(x10, x11));
            float m1 = fmaxf(fmaxf(x02, x03), fmaxf(x12, x13));
            m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
            m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
            m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
            m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
            const float new0 = fmaxf(row_max[0], m0), new1 = fmaxf(row_max[1], m1);
            // token 0 of a page is always valid, so new0/new1 are finite
            const float alpha0 = exp2f(row_max[0] - new0), alpha1 = exp2f(row_max[1] - new1);
            row_max[0] = new0;
            row_max[1] = new1;
            const float p00 = exp2f(x00 - new0), p01 = exp2f(x01 - new0);
            const float p10 = exp2f(x10 - new0), p11 = exp2f(x11 - new0);
            const float p02 = exp2f(x02 - new1), p03 = exp2f(x03 - new1);
            const float p12 = exp2f(x12 - new1), p13 = exp2f(x13 - new1);
            row_sum[0] = row_sum[0] * alpha0 + ((p00 + p01) + (p10 + p11));
            row_sum[1] = row_sum[1] * alpha1 + ((p02 + p03) + (p12 + p13));
            uint32_t pf[4];
            pf[0] = pack_bf16(p00, p01);
            pf[1] = pack_bf16(p02, p03);
            pf[2] = pack_bf16(p10, p11);
            pf[3] = pack_bf16(p12, p13);
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) {
                acc[nt][0] *= alpha0;
                acc[nt][1] *= alpha0;
                acc[nt][2] *= alpha1;
                acc[nt][3] *= alpha1;
            }
            // ---- O += P V : 16 rows x 128 dims --------------------------------------------------
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int chunk = ((2 * j) & 7) + v_hi;
                const uint32_t addr = v_tile + (j >> 2) * kBoxBytes + v_tok * 128 +
                                      ((chunk ^ (v_tok & 7)) << 4);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(addr, b0, b1, b2, b3);
                mma_bf16(acc[2 * j], pf, b0, b1);
                mma_bf16(acc[2 * j + 1], pf, b2, b3);
            }
            __syncwarp();
            if (lane == 0) {
                if (valid_tokens < kPage)
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(bar_empty);
            }
        }
        row_sum[0] += __shfl_xor_sync(0xffffffffu, row_sum[0], 1);
        row_sum[0] += __shfl_xor_sync(0xffffffffu, row_sum[0], 2);
        row_sum[1] += __shfl_xor_sync(0xffffffffu, row_sum[1], 1);
        row_sum[1] += __shfl_xor_sync(0xffffffffu, row_sum[1], 2);
    }

    // ---- join: every TMA write has been consumed or abandoned; the ring becomes scratch ---------
    __syncthreads();
    const bool timed_out = flags[1] != 0;
    const bool invalid_page = flags[0] != 0;
    if (timed_out) {
        if (tid == 0 && a.status) atomicExch(a.status, 1);
        return;
    }

    if (a.pps > 1) {
        // warps that streamed different pages of the same KV head merge their states
        float *scratch = reinterpret_cast<float *>(ring);
        if (warp < kComputeWarps) {
            float *mine = scratch + warp * kMergeFloatsPerWarp;
#pragma unroll
            for (int nt = 0; nt < 16; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) mine[(nt * 4 + j) * 32 + lane] = acc[nt][j];
            mine[64 * 32 + lane] = row_max[0];
            mine[65 * 32 + lane] = row_max[1];
            mine[66 * 32 + lane] = row_sum[0];
            mine[67 * 32 + lane] = row_sum[1];
        }
        __syncthreads();
        if (warp < kComputeWarps && page_slot0 == 0) {
            for (int k = 1; k < a.pps; ++k) {
                const float *other = scratch + (warp + k * a.hc * a.mt) * kMergeFloatsPerWarp;
                const float om0 = other[64 * 32 + lane], om1 = other[65 * 32 + lane];
                const float ol0 = other[66 * 32 + lane], ol1 = other[67 * 32 + lane];
                const float n0 = fmaxf(row_max[0], om0), n1 = fmaxf(row_max[1], om1);
                const float w0 = ol0 == 0.0f ? 1.0f : exp2f(row_max[0] - n0);
                const float w1 = ol1 == 0.0f ? 1.0f : exp2f(row_max[1] - n1);
                const float ow0 = ol0 == 0.0f ? 0.0f : exp2f(om0 - n0);
                const float ow1 = ol1 == 0.0f ? 0.0f : exp2f(om1 - n1);
                if (ol0 != 0.0f) row_max[0] = n0;
                if (ol1 != 0.0f) row_max[1] = n1;
                row_sum[0] = row_sum[0] * w0 + ol0 * ow0;
                row_sum[1] = row_sum[1] * w1 + ol1 * ow1;
#pragma unroll
                for (int nt = 0; nt < 16; ++nt) {
                    acc[nt][0] = acc[nt][0] * w0 + other[(nt * 4 + 0) * 32 + lane] * ow0;
                    acc[nt][1] = acc[nt][1] * w0 + other[(nt * 4 + 1) * 32 + lane] * ow0;
                    acc[nt][2] = acc[nt][2] * w1 + other[(nt * 4 + 2) * 32 + lane] * ow1;
                    acc[nt][3] = acc[nt][3] * w1 + other[(nt * 4 + 3) * 32 + lane] * ow1;
                }
            }
        }
    }

    if (warp >= kComputeWarps || page_slot0 != 0) return;

    // ---- epilogue ---------------------------------------------------------------------------------
    const int kv_head = hb * a.hc + head_in_cta;
    const int g0 = qb * rows_per_block + mtile * 16 + (lane >> 2);
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int g = g0 + half * 8;
        if (g >= group) continue;
        const size_t state = (size_t)request * a.qh + (size_t)kv_head * group + g;
        const float m = row_max[half], l = row_sum[half];
        if (a.partitions == 1) {
            if (invalid_page) continue; // the request keeps its previous output
            uint32_t *out = reinterpret_cast<uint32_t *>(a.output + state * kHeadDim);
#pragma unroll
            for (int nt = 0; nt < 16; ++nt)
                out[nt * 4 + (lane & 3)] =
                    pack_bf16(acc[nt][half * 2] / l, acc[nt][half * 2 + 1] / l);
            if ((lane & 3) == 0) a.lse[state] = m + log2f(l);
        } else {
            float *ws = a.workspace + (state * a.partitions + part) * kStateWidth;
            if ((lane & 3) == 0) {
                ws[0] = m;
                ws[1] = invalid_page ? -1.0f : l; // a negative normaliser poisons the merge
            }
#pragma unroll
            for (int nt = 0; nt < 16; ++nt)
                *reinterpret_cast<float2 *>(ws + 2 + nt * 8 + col) =
                    make_float2(acc[nt][half * 2], acc[nt][half * 2 + 1]);
        }
    }
}

// Merges the split-K states of one (request, query head) per warp, in partition order, with
// the arithmetic of single_decode_bf16_split_k_merge_reference
// (crates/loom-infer/src/attention/single_decode/mod.rs:343-379); states with a zero
// normaliser (chunks without pages) are skipped as in decode.rs:635.
__global__ void __launch_bounds__(128)
split_merge_kernel(const float *__restrict__ workspace, __nv_bfloat16 *output, float *lse,
                   const int32_t *indptr, const int32_t *last, int batch, int qh, int partitions,
                   int indices_len) {
    const int lane = threadIdx.x & 31;
    const int state = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (state >= batch * qh) return;
    const int request = state / qh;
    int page_start, page_end, tail;
    if (!request_metadata_valid(indptr, last, batch, indices_len, request, page_start, page_end,
                                tail))
        return;
    const float *st = workspace + (size_t)state * partitions * kStateWidth;
    bool poisoned = false;
    for (int p = lane; p < partitions; p += 32) poisoned |= st[p * kStateWidth + 1] < 0.0f;
    if (__any_sync(0xffffffffu, poisoned)) return;

    float merged_max = st[0], merged_norm = st[1];
    float2 lo = *reinterpret_cast<const float2 *>(st + 2 + lane * 4);
    float2 hi = *reinterpret_cast<const float2 *>(st + 4 + lane * 4);
    for (int p = 1; p < partitions; ++p) {
        const float *s = st + p * kStateWidth;
        const float pm = s[0], pn = s[1];
        if (pn == 0.0f) continue;
        const float2 vlo = *reinterpret_cast<const float2 *>(s + 2 + lane * 4);
        const float2 vhi = *reinterpret_cast<const float2 *>(s + 4 + lane * 4);
        const float next = fmaxf(merged_max, pm);
        const float wm = exp2f(merged_max - next), wp = exp2f(pm - next);
        merged_norm = merged_norm * wm + pn * wp;
        lo.x = lo.x * wm + vlo.x * wp;
        lo.y = lo.y * wm + vlo.y * wp;
        hi.x = hi.x * wm + vhi.x * wp;
        hi.y = hi.y * wm + vhi.y * wp;
        merged_max = next;
    }
    uint2 packed;
    packed.x = pack_bf16(lo.x / merged_norm, lo.y / merged_norm);
    packed.y = pack_bf16(hi.x / merged_norm, hi.y / merged_norm);
    *reinterpret_cast<uint2 *>(output + (size_t)state * kHeadDim + lane * 4) = packed;
    if (lane == 0) lse[state] = merged_max + log2f(merged_norm);
}

} // namespace

int configure_decode_kernels(size_t max_dynamic_shared) {
    return cudaFuncSetAttribute(paged_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)max_dynamic_shared);
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
    args.hc = launch.heads_per_cta;
    args.pps = launch.pages_per_stage;
    args.mt = launch.q_tiles;
    args.qb = launch.q_blocks;
    args.partitions = launch.partitions;
    args.stages = launch.stages;
    args.scale_log2 = launch.scale_log2;
    CUtensorMap k_map, v_map;
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    memcpy(&k_map, launch.k_map, sizeof(k_map));
    memcpy(&v_map, launch.v_map, sizeof(v_map));
    paged_decode_kernel<<<launch.grid, launch.block, launch.shared_bytes,
                          static_cast<cudaStream_t>(stream)>>>(k_map, v_map, args);
    return cudaGetLastError();
}

int launch_split_merge(const MergeLaunch &launch, void *stream) {
    split_merge_kernel<<<launch.grid, launch.block, 0, static_cast<cudaStream_t>(stream)>>>(
        launch.workspace, static_cast<__nv_bfloat16 *>(launch.output), launch.lse, launch.indptr,
        launch.last, launch.batch, launch.qh, launch.partitions, launch.indices_len);
    return cudaGetLastError();
}

} // namespace lb
