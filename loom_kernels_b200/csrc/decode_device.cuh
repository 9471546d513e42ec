// Device-side building blocks shared by the paged-decode kernels: mbarrier / TMA / ldmatrix /
// mma.sync wrappers, the per-request metadata guard, and the per-page attention step.
//
// Shared-memory tile layout (what one TMA box leaves behind): for each KV head of the CTA, a
// K tile and a V tile of 4 KB each = two 2 KB halves (dims 0-63, dims 64-127); a half is 16 token
// rows of 128 bytes with the 128-byte swizzle (16-byte chunk c of row r sits at chunk c ^ (r & 7)).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "bounds_check.cuh"
#include "dependent_launch.cuh"
#include "kernels.hpp"

namespace lb {
namespace dev {

constexpr int kHeadDim = 128;
constexpr int kPage = 16;
constexpr int kStateWidth = 130;
constexpr int kComputeWarps = 8;
constexpr int kMaxProducerWarps = 4; // the balanced kernel: up to one producer warp per page slot
constexpr int kUnitBytes = 8192;  // K (16 x 256 B) + V (16 x 256 B) of one (page, KV head)
constexpr int kBoxBytes = 2048;   // half a tile: 16 tokens x 64 dims x 2 B
constexpr long long kWaitCycles = 4000000000ll; // ~2 s at 2 GHz; waits normally take microseconds

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
// Raises the byte count the current phase waits for, without arriving.
__device__ __forceinline__ void mbar_expect_more(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes)
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
// Bounded wait: false after `limit` cycles without the phase completing.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          long long limit = kWaitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int spin = 0; spin < 256; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - start > limit) return false;
    }
}
// After a wait ran out: before the CTA leaves, the lane that armed the `full` barriers of one
// page slot waits (bounded again) for the copies it issued last into every stage of the ring, so
// that no copy is still on its way into shared memory the next CTA may own.  `issued` = pages of
// this slot whose copies were issued, page k into stage k % stages in round k / stages.
__device__ __forceinline__ void drain_issued_copies(uint32_t slot_full0, int stage_stride,
                                                    int stages, int issued, long long limit) {
    for (int k = issued > stages ? issued - stages : 0; k < issued; ++k)
        (void)mbar_wait(slot_full0 + (k % stages) * stage_stride, (uint32_t)(k / stages) & 1u,
                        limit);
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
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
// 2^x on the special-function unit (relative error 2^-22; 2^0 = 1 and 2^-inf = 0 exactly)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// Per-request metadata guard of the reference's kernels
// (crates/loom-infer-cuda/src/attention/decode.rs:234-248 / :426-437).  The end of the table,
// page_indptr[batch], must lie in [indices_min, indices_len]: the reference's rule is
// indices_min == indices_len (the bound page_indices are exactly the table); a plan made with
// the capacity option passes 0, so that page_indices may be bound longer than the table in use.
__device__ __forceinline__ bool request_metadata_valid(const int32_t *indptr, const int32_t *last,
                                                       int batch, int indices_min, int indices_len,
                                                       int request, int &page_start, int &page_end,
                                                       int &tail, int32_t *status = nullptr) {
    if (!in_bounds(request, batch, status, kSiteIndptr)) return false; // indptr[request + 1], last
    const int global_end = indptr[batch];
    page_start = indptr[request];
    page_end = indptr[request + 1];
    tail = last[request];
    return indptr[0] == 0 && global_end >= indices_min && global_end <= indices_len &&
           page_start >= 0 &&
           page_end > page_start && page_end <= global_end && tail >= 1 && tail <= kPage;
}

// Online-softmax state of one warp: 16 query rows x 128 dims in MMA accumulator layout.  A lane
// owns rows lane/4 and lane/4 + 8; row_sum is a per-lane partial until finish_rows().
struct WarpState {
    float acc[16][4];
    float row_max[2];
    float row_sum[2];
    __device__ __forceinline__ void reset() {
#pragma unroll
        for (int i = 0; i < 16; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
        row_max[0] = row_max[1] = -INFINITY;
        row_sum[0] = row_sum[1] = 0.0f;
    }
    __device__ __forceinline__ void finish_rows() {
        row_sum[0] += __shfl_xor_sync(0xffffffffu, row_sum[0], 1);
        row_sum[0] += __shfl_xor_sync(0xffffffffu, row_sum[0], 2);
        row_sum[1] += __shfl_xor_sync(0xffffffffu, row_sum[1], 1);
        row_sum[1] += __shfl_xor_sync(0xffffffffu, row_sum[1], 2);
    }
};

// A-operand fragments of 16 query rows (rows >= `rows_valid` are zero): q points at row 0.
__device__ __forceinline__ void load_query_fragments(const __nv_bfloat16 *q, int rows_valid,
                                                     int lane, uint32_t (&qf)[8][4]) {
    const int r0 = lane >> 2, c = lane & 3;
    const bool valid0 = r0 < rows_valid, valid1 = r0 + 8 < rows_valid;
    const uint32_t *q0 = reinterpret_cast<const uint32_t *>(q + (size_t)r0 * kHeadDim);
    const uint32_t *q1 = q0 + 8 * kHeadDim / 2;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        qf[kk][0] = valid0 ? q0[kk * 8 + c] : 0u;
        qf[kk][1] = valid1 ? q1[kk * 8 + c] : 0u;
        qf[kk][2] = valid0 ? q0[kk * 8 + 4 + c] : 0u;
        qf[kk][3] = valid1 ? q1[kk * 8 + 4 + c] : 0u;
    }
}

// One page of one KV head: S = Q K^T (16 x 16), online softmax in the log2 domain, O += P V.
// k_tile / v_tile are the 4 KB tiles in shared memory; tokens >= valid_tokens are masked and
// their V rows zeroed first (pool rows past a request's length may hold anything, and
// 0 * garbage must not produce NaN).  Returns true when shared memory was written by this warp
// (the caller then fences before handing the tile back to the async proxy).
//
// kRowLimits (causal prefill): the two rows of a lane see only tokens below limit0 / limit1 of
// this page (any value; <= 0 masks the whole page for that row).  A row may then meet pages in
// which it sees nothing before it has seen any token, so its running maximum can still be
// -inf: the exponent base falls back to 0 and every weight of the row comes out as exactly 0.
template <bool kRowLimits = false>
__device__ __forceinline__ bool attend_page(uint8_t *k_ptr, uint8_t *v_ptr, int valid_tokens,
                                            const uint32_t (&qf)[8][4], float scale_log2,
                                            int lane, WarpState &st, int limit0 = kPage,
                                            int limit1 = kPage) {
    const uint32_t k_tile = smem_u32(k_ptr), v_tile = smem_u32(v_ptr);
    const bool partial = valid_tokens < kPage;
    if (partial) {
        for (int i = lane; i < (kPage - valid_tokens) * 16; i += 32) {
            const int row = valid_tokens + (i >> 4);
            const int c = i & 15;
            *reinterpret_cast<uint4 *>(v_ptr + (c >> 3) * kBoxBytes + row * 128 + (c & 7) * 16) =
                make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
    }
    // per-lane ldmatrix selectors: K matrices are (tokens 0-7 | 8-15) x (k chunk | k chunk + 1),
    // V matrices (transposed on load) are (tokens 0-7 | 8-15) x (dim chunk | dim chunk + 1)
    const int k_tok = ((lane >> 4) << 3) + (lane & 7);
    const int k_hi = (lane >> 3) & 1;
    const int v_tok = (((lane >> 3) & 1) << 3) + (lane & 7);
    const int v_hi = lane >> 4;

    // four accumulation chains of four MMAs each (dims 0-63 and 64-127 of tokens 0-7 and 8-15):
    // the dependent chain is what a warp waits on, so it is kept short and summed afterwards
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    float u0[4] = {0.f, 0.f, 0.f, 0.f}, u1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        const int chunk = (kk << 1) + k_hi;
        const uint32_t addr = k_tile + k_tok * 128 + ((chunk ^ (k_tok & 7)) << 4);
        uint32_t b0, b1, b2, b3, c0, c1, c2, c3;
        ldmatrix_x4(addr, b0, b1, b2, b3);
        ldmatrix_x4(addr + kBoxBytes, c0, c1, c2, c3);
        mma_bf16(s0, qf[kk], b0, b1);
        mma_bf16(s1, qf[kk], b2, b3);
        mma_bf16(u0, qf[kk + 4], c0, c1);
        mma_bf16(u1, qf[kk + 4], c2, c3);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s0[i] += u0[i];
        s1[i] += u1[i];
    }
    const int t0 = (lane & 3) * 2;
    float x00 = s0[0] * scale_log2, x01 = s0[1] * scale_log2;
    float x02 = s0[2] * scale_log2, x03 = s0[3] * scale_log2;
    float x10 = s1[0] * scale_log2, x11 = s1[1] * scale_log2;
    float x12 = s1[2] * scale_log2, x13 = s1[3] * scale_log2;
    if (kRowLimits) {
        const int lim0 = min(limit0, valid_tokens), lim1 = min(limit1, valid_tokens);
        if (t0 >= lim0) x00 = -INFINITY;
        if (t0 + 1 >= lim0) x01 = -INFINITY;
        if (t0 + 8 >= lim0) x10 = -INFINITY;
        if (t0 + 9 >= lim0) x11 = -INFINITY;
        if (t0 >= lim1) x02 = -INFINITY;
        if (t0 + 1 >= lim1) x03 = -INFINITY;
        if (t0 + 8 >= lim1) x12 = -INFINITY;
        if (t0 + 9 >= lim1) x13 = -INFINITY;
    } else if (partial) {
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
    // without row limits token 0 of a page is always valid, so the new maxima are finite
    const float new0 = fmaxf(st.row_max[0], m0), new1 = fmaxf(st.row_max[1], m1);
    const float base0 = kRowLimits && new0 == -INFINITY ? 0.0f : new0;
    const float base1 = kRowLimits && new1 == -INFINITY ? 0.0f : new1;
    const float alpha0 = fast_exp2(st.row_max[0] - base0), alpha1 = fast_exp2(st.row_max[1] - base1);
    st.row_max[0] = new0;
    st.row_max[1] = new1;
    const float p00 = fast_exp2(x00 - base0), p01 = fast_exp2(x01 - base0);
    const float p10 = fast_exp2(x10 - base0), p11 = fast_exp2(x11 - base0);
    const float p02 = fast_exp2(x02 - base1), p03 = fast_exp2(x03 - base1);
    const float p12 = fast_exp2(x12 - base1), p13 = fast_exp2(x13 - base1);
    st.row_sum[0] = st.row_sum[0] * alpha0 + ((p00 + p01) + (p10 + p11));
    st.row_sum[1] = st.row_sum[1] * alpha1 + ((p02 + p03) + (p12 + p13));
    uint32_t pf[4];
    pf[0] = pack_bf16(p00, p01);
    pf[1] = pack_bf16(p02, p03);
    pf[2] = pack_bf16(p10, p11);
    pf[3] = pack_bf16(p12, p13);
    // the running maxima settle after the first pages; then every alpha is exactly 1
    if (__any_sync(0xffffffffu, alpha0 != 1.0f || alpha1 != 1.0f)) {
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            st.acc[nt][0] *= alpha0;
            st.acc[nt][1] *= alpha0;
            st.acc[nt][2] *= alpha1;
            st.acc[nt][3] *= alpha1;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int chunk = ((2 * j) & 7) + v_hi;
        const uint32_t addr =
            v_tile + (j >> 2) * kBoxBytes + v_tok * 128 + ((chunk ^ (v_tok & 7)) << 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(addr, b0, b1, b2, b3);
        mma_bf16(st.acc[2 * j], pf, b0, b1);
        mma_bf16(st.acc[2 * j + 1], pf, b2, b3);
    }
    return partial;
}

// Writes the two rows a lane owns: BF16 O + log2 LSE (final) or the F32 state [m, n, wv[128]].
__device__ __forceinline__ void write_final_row(__nv_bfloat16 *out_row, float *lse_slot, int lane,
                                                int half, const WarpState &st) {
    const float l = st.row_sum[half];
    // one reciprocal instead of 32 divisions: the extra F32 rounding is far below a BF16 ulp
    const float inv = 1.0f / l;
    uint32_t *out = reinterpret_cast<uint32_t *>(out_row);
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
        out[nt * 4 + (lane & 3)] =
            pack_bf16(st.acc[nt][half * 2] * inv, st.acc[nt][half * 2 + 1] * inv);
    if ((lane & 3) == 0) *lse_slot = st.row_max[half] + log2f(l);
}
__device__ __forceinline__ void write_state_row(float *state, int lane, int half,
                                                const WarpState &st, bool poisoned) {
    if ((lane & 3) == 0) {
        state[0] = st.row_max[half];
        state[1] = poisoned ? -1.0f : st.row_sum[half]; // a negative normaliser poisons a merge
    }
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
        *reinterpret_cast<float2 *>(state + 2 + nt * 8 + col) =
            make_float2(st.acc[nt][half * 2], st.acc[nt][half * 2 + 1]);
}

// ---- output rows across GPUs ------------------------------------------------------------------------
//
// A command whose plan gathers its output writes every finished row straight into every rank's
// copy of one gathered result (peer-mapped device memory, plain stores over NVLink; this rank's
// own copy is one of them), instead of into a local buffer that a collective would then move.
// Row r of the local batch, local query head h lands at row
//     dest_rows[r] * gathered_qh + head_offset + h
// of the gathered [rows, 128] BF16 output and the gathered F32 LSE.
//
// The last kernel of a gathering command counts its CTAs; the last one to finish publishes a new
// epoch in every rank's flag array and then waits (bounded) until every rank has published the
// same epoch, so that the kernel -- and with it the command -- completes only when the gathered
// result is whole on this GPU.  Ranks are other GPUs running the same command; they never share
// a GPU with the waiter.
using ::lb::PeerOut;    // kernels.hpp: where the finished rows go when a plan gathers its output
using ::lb::PeerSignal; // kernels.hpp: the epoch the last kernel of such a command publishes

// acquire-release fence at system scope: orders this thread's earlier accesses -- and, through a
// CTA or warp barrier before it, those of the threads that met at the barrier -- before its later
// ones as seen from any GPU.  (Cheaper than the sequentially consistent membar.sys.)
__device__ __forceinline__ void fence_system() {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ void store_relaxed_system(uint32_t *address, uint32_t value) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t load_relaxed_system(const uint32_t *address) {
    uint32_t value;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}

// What a kernel fetches from the peer tables when it starts, so that its last instructions -- the
// row stores and the epoch -- do not wait on chains of dependent loads: the tables are device
// arrays of pointers, and the epoch and the row map are words in global memory.
struct PeerLocal {
    void *out[LB_PEER_MAX_RANKS];      // PeerOut::out
    float *lse[LB_PEER_MAX_RANKS];     // PeerOut::lse
    uint32_t *flags[LB_PEER_MAX_RANKS]; // PeerSignal::flags
    uint32_t epoch;                    // *PeerSignal::epoch when the kernel started
};

// One warp fills `local` (in shared memory); the CTA synchronises before anyone reads it.
__device__ __forceinline__ void peer_prefetch(const PeerOut &peer, const PeerSignal &signal,
                                              int lane, PeerLocal &local) {
    if (lane < peer.world) {
        local.out[lane] = peer.out[lane];
        local.lse[lane] = peer.lse[lane];
    }
    if (lane < signal.world) local.flags[lane] = signal.flags[lane];
    if (lane == 0 && signal.world != 0) local.epoch = *signal.epoch;
}

// Called by warp 0 of every CTA of the kernel, after a CTA barrier that follows the CTA's last row
// store.  Ordering, by the PTX memory model: the CTA barrier orders every thread's row stores
// before lane 0's counting atomic, which is a release at GPU scope (a system-scope fence per CTA
// costs about a microsecond each, and a kernel of a thousand small CTAs queues them up); the
// last CTA's atomic is an acquire of all of them, and its system-scope fence then orders every
// row of the grid -- and, through stream order, of the earlier kernels of the step -- before the
// epoch it publishes.  `flag_of_lane` is s.flags[lane], `my_flags` is s.flags[s.rank] and `epoch`
// is *s.epoch as the kernel found it (only this kernel's last CTA changes it), all fetched when
// the kernel started.
__device__ __forceinline__ void peer_signal_and_wait(const PeerSignal &s, uint32_t *flag_of_lane,
                                                     const uint32_t *my_flags, uint32_t epoch) {
    const int lane = threadIdx.x;
    unsigned last = 0;
    if (lane == 0) {
        unsigned counted;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;"
                     : "=r"(counted)
                     : "l"(s.done)
                     : "memory");
        last = counted == gridDim.x - 1 ? 1u : 0u;
    }
    if (!__shfl_sync(0xffffffffu, last, 0)) return;
    epoch += 1;
    if (lane == 0) {
        fence_system(); // every row of the step precedes the epoch, as seen from any GPU
        *s.done = 0; // the next kernel counts from zero (it starts after this one has completed)
        *s.epoch = epoch;
    }
    __syncwarp(); // lane 0's fence precedes every lane's flag store
    if (lane < s.world) store_relaxed_system(flag_of_lane + kPeerFlagsWord + s.rank, epoch);
    bool arrived = true;
    if (lane < s.world) {
        const uint32_t *mine = my_flags + kPeerFlagsWord + lane;
        arrived = (int32_t)(load_relaxed_system(mine) - epoch) >= 0;
        const long long start = clock64();
        while (!arrived) {
#pragma unroll 1
            for (int spin = 0; spin < 64 && !arrived; ++spin)
                arrived = (int32_t)(load_relaxed_system(mine) - epoch) >= 0;
            if (clock64() - start > s.wait_cycles) break;
        }
    }
    // the flags were read relaxed: this fence makes the peers' rows, which precede their epochs,
    // visible to everything that follows the kernel
    fence_system();
    if (__any_sync(0xffffffffu, !arrived) && lane == 0 && s.status) atomicExch(s.status, 2);
}

// 4 x 4 transpose of 32-bit words among the four lanes of a quad: afterwards lane c holds, in
// r[k], what lane k held in r[c].
__device__ __forceinline__ void quad_transpose(uint32_t (&r)[4], int lane) {
    const bool odd = lane & 1, upper = lane & 2;
#pragma unroll
    for (int k = 0; k < 4; k += 2) {
        const uint32_t other = __shfl_xor_sync(0xffffffffu, odd ? r[k] : r[k + 1], 1);
        if (odd) r[k] = other;
        else r[k + 1] = other;
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const uint32_t other = __shfl_xor_sync(0xffffffffu, upper ? r[k] : r[k + 2], 2);
        if (upper) r[k] = other;
        else r[k + 2] = other;
    }
}

// The two rows a lane owns (MMA accumulator layout), normalised, as BF16 into every rank's copy
// of the gathered result.  The four lanes of a quad first exchange their 4-byte pieces so that a
// lane owns whole 16-byte chunks: a row leaves as 16-byte stores, 64 contiguous bytes per quad.
// Every lane of the warp must call (the exchange is warp-wide); rows[half] < 0 stores nothing.
__device__ __forceinline__ void write_final_rows_to_peers(const PeerLocal &peer, int world,
                                                          const long long (&rows)[2], int lane,
                                                          const WarpState &st) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const float l = st.row_sum[half];
        const float inv = 1.0f / l;
        uint4 chunk[4]; // chunk[j] = bytes (4j + (lane & 3)) * 16 .. + 16 of the row
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t r[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                r[k] = pack_bf16(st.acc[4 * j + k][half * 2] * inv,
                                 st.acc[4 * j + k][half * 2 + 1] * inv);
            quad_transpose(r, lane);
            chunk[j] = make_uint4(r[0], r[1], r[2], r[3]);
        }
        if (rows[half] < 0) continue;
        const float lse = st.row_max[half] + log2f(l);
        for (int p = 0; p < world; ++p) {
            uint4 *row = reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(peer.out[p]) +
                                                   rows[half] * kHeadDim);
#pragma unroll
            for (int j = 0; j < 4; ++j) row[4 * j + (lane & 3)] = chunk[j];
            if ((lane & 3) == 0) peer.lse[p][rows[half]] = lse;
        }
    }
}

// ---- thread-block clusters: the chunks of one request reduced through distributed shared memory ----
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the shared::cluster window, of `local` (a shared::cta address) in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_address(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ float2 load_cluster_float2(uint32_t address) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];"
                 : "=f"(v.x), "=f"(v.y)
                 : "r"(address)
                 : "memory");
    return v;
}

// One warp merges the `parts` states [max_log2, normaliser, wv[128]] that the CTAs of its cluster
// hold for one row at shared-memory address `row_state` (the same address in every CTA): the
// algebra of merge_partial against the global maximum, the states read with plain
// ld.shared::cluster (no multicast).  Returns false when a state is poisoned or all are empty.
__device__ __forceinline__ bool merge_cluster_row(uint32_t row_state, int parts, int lane,
                                                  float &top, float &norm, float4 &acc) {
    constexpr int kMaxParts = 8;
    float part_max[kMaxParts], part_norm[kMaxParts];
    float2 lo[kMaxParts], hi[kMaxParts];
#pragma unroll
    for (int p = 0; p < kMaxParts; ++p) {
        part_max[p] = part_norm[p] = 0.0f;
        lo[p] = hi[p] = make_float2(0.f, 0.f);
        if (p < parts) {
            const uint32_t remote = cluster_address(row_state, (uint32_t)p);
            const float2 head = load_cluster_float2(remote);
            part_max[p] = head.x;
            part_norm[p] = head.y;
            lo[p] = load_cluster_float2(remote + 8 + lane * 16);
            hi[p] = load_cluster_float2(remote + 16 + lane * 16);
        }
    }
    top = -INFINITY;
    bool poisoned = false;
#pragma unroll
    for (int p = 0; p < kMaxParts; ++p) {
        poisoned |= part_norm[p] < 0.0f;
        if (part_norm[p] > 0.0f) top = fmaxf(top, part_max[p]);
    }
    norm = 0.0f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < kMaxParts; ++p) {
        const float weight = part_norm[p] > 0.0f ? exp2f(part_max[p] - top) : 0.0f;
        norm += part_norm[p] * weight;
        acc.x += lo[p].x * weight;
        acc.y += lo[p].y * weight;
        acc.z += hi[p].x * weight;
        acc.w += hi[p].y * weight;
    }
    return !poisoned && norm > 0.0f;
}

// Merges n unnormalised states [max_log2, normaliser, wv[128]] of one (request, query head) and
// writes BF16 O + log2 LSE.  state_of(i) returns the i-th state or nullptr for "no state";
// states with a zero normaliser (chunks without pages) are skipped as in the reference's device
// merge (crates/loom-infer-cuda/src/attention/decode.rs:635); a negative normaliser marks a chunk
// that met an out-of-range page, and then nothing is published.  Same algebra as
// single_decode_bf16_split_k_merge_reference (crates/loom-infer/src/attention/single_decode/
// mod.rs:343-379), evaluated against the global maximum so that the state loads are independent
// and pipeline instead of forming one dependent chain per state.
// `publish` is consulted only after every load has been issued, so a caller can hand in a
// predicate that itself depends on loads still in flight (the request guard) without putting a
// second memory round trip in front of the state loads.
constexpr int kMergeBatch = 16;  // states whose row loads are in flight together
constexpr int kMergeCached = 4;  // rounds of 32 states whose (max, normaliser) stay in registers

// The weighted sums of a merge, computed by one warp (per lane: four of the 128 dims; `norm` is
// complete in every lane).  Returns false when a state is poisoned.  Everything that does not
// depend on a value still in flight is issued first: the (max, normaliser) pairs of the first
// 128 states and the rows of the first 16, so that a merge of up to 16 states -- the common
// case -- costs one memory round trip, and a long request one more per 16 states.
// kBatch: states whose row loads are in flight together (16, or 8 where registers are scarce).
template <int kBatch = kMergeBatch, typename StateOf>
__device__ __forceinline__ bool merge_partial(StateOf state_of, int n, int lane, float &top,
                                              float &norm, float4 &acc) {
    if (n <= 4) {
        // the common case of a balanced plan (a request cut once or twice): a handful of
        // instructions instead of the batched loops below, whose cost does not depend on n
        float part_max[4], part_norm[4];
        float2 lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float *s = i < n ? state_of(i) : nullptr;
            part_max[i] = part_norm[i] = 0.0f;
            lo[i] = hi[i] = make_float2(0.f, 0.f);
            if (s != nullptr) {
                part_max[i] = __ldcg(s);
                part_norm[i] = __ldcg(s + 1);
                lo[i] = __ldcg(reinterpret_cast<const float2 *>(s + 2 + lane * 4));
                hi[i] = __ldcg(reinterpret_cast<const float2 *>(s + 4 + lane * 4));
            }
        }
        top = -INFINITY;
        bool poisoned = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            poisoned |= part_norm[i] < 0.0f;
            if (part_norm[i] > 0.0f) top = fmaxf(top, part_max[i]);
        }
        norm = 0.0f;
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float weight = part_norm[i] > 0.0f ? exp2f(part_max[i] - top) : 0.0f;
            norm += part_norm[i] * weight;
            acc.x += lo[i].x * weight;
            acc.y += lo[i].y * weight;
            acc.z += hi[i].x * weight;
            acc.w += hi[i].y * weight;
        }
        return !poisoned;
    }
    float my_norm[kMergeCached], my_max[kMergeCached];
#pragma unroll
    for (int k = 0; k < kMergeCached; ++k) {
        const float *s = k * 32 + lane < n ? state_of(k * 32 + lane) : nullptr;
        my_norm[k] = s ? __ldcg(s + 1) : 0.0f;
        my_max[k] = s ? __ldcg(s) : 0.0f;
    }
    float2 lo[kBatch], hi[kBatch];
    auto fetch_rows = [&](int base) { // rows of states base .. base + 15 (zero past n)
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const float *s = base + u < n ? state_of(base + u) : nullptr;
            lo[u] = hi[u] = make_float2(0.f, 0.f);
            if (s != nullptr) {
                lo[u] = __ldcg(reinterpret_cast<const float2 *>(s + 2 + lane * 4));
                hi[u] = __ldcg(reinterpret_cast<const float2 *>(s + 4 + lane * 4));
            }
        }
    };
    fetch_rows(0);

    top = -INFINITY;
    bool poisoned = false;
#pragma unroll
    for (int k = 0; k < kMergeCached; ++k) {
        poisoned |= my_norm[k] < 0.0f;
        if (my_norm[k] > 0.0f) top = fmaxf(top, my_max[k]);
    }
    for (int i = kMergeCached * 32 + lane; i < n; i += 32) { // beyond the cached rounds
        const float *s = state_of(i);
        if (s == nullptr) continue;
        const float part_norm = __ldcg(s + 1);
        poisoned |= part_norm < 0.0f;
        if (part_norm > 0.0f) top = fmaxf(top, __ldcg(s));
    }
    if (__any_sync(0xffffffffu, poisoned)) return false;
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, d));

    // 32 states per round: lane l holds the weight of state round * 32 + l
    norm = 0.0f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int round = 0; round * 32 < n; ++round) {
        float part_norm = 0.0f, part_max = 0.0f;
        if (round < kMergeCached) {
#pragma unroll
            for (int k = 0; k < kMergeCached; ++k)
                if (k == round) {
                    part_norm = my_norm[k];
                    part_max = my_max[k];
                }
        } else {
            const float *s = round * 32 + lane < n ? state_of(round * 32 + lane) : nullptr;
            part_norm = s ? __ldcg(s + 1) : 0.0f;
            part_max = s ? __ldcg(s) : 0.0f;
        }
        const float my_weight = part_norm > 0.0f ? exp2f(part_max - top) : 0.0f;
        norm += part_norm * my_weight;
#pragma unroll
        for (int half = 0; half < 32 / kBatch; ++half) {
            const int base = round * 32 + half * kBatch;
            if (base >= n) break;
            if (base > 0) fetch_rows(base); // the first batch is already here
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const float weight = __shfl_sync(0xffffffffu, my_weight, half * kBatch + u);
                acc.x += lo[u].x * weight;
                acc.y += lo[u].y * weight;
                acc.z += hi[u].x * weight;
                acc.w += hi[u].y * weight;
            }
        }
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) norm += __shfl_xor_sync(0xffffffffu, norm, d);
    return true;
}

// merge_partial shared out to the kWarps warps of a CTA that all work on ONE item: warp `part`
// merges a contiguous share of the n states, the shares are combined through shared memory, and
// warp 0 returns the result (the other warps return false).  A long request cut into ~90 states
// costs one warp six dependent rounds of loads; four warps need two.  Every thread of the CTA
// must call (CTA barrier inside).
template <int kWarps, typename StateOf>
__device__ __forceinline__ bool merge_partial_shared(StateOf state_of, int n, int lane, int part,
                                                     float &top, float &norm, float4 &acc) {
    __shared__ float4 share_acc[kWarps][32];
    __shared__ float share_top[kWarps], share_norm[kWarps];
    __shared__ int share_poisoned;
    const int lo = (int)((long long)n * part / kWarps);
    const int hi = (int)((long long)n * (part + 1) / kWarps);
    if (part == 0 && lane == 0) share_poisoned = 0;
    __syncthreads();
    const bool ok =
        merge_partial([&](int i) { return state_of(lo + i); }, hi - lo, lane, top, norm, acc);
    share_acc[part][lane] = acc;
    if (lane == 0) {
        share_top[part] = top;
        share_norm[part] = norm;
        if (!ok) share_poisoned = 1;
    }
    __syncthreads();
    if (part != 0 || share_poisoned) return false;
    top = -INFINITY;
#pragma unroll
    for (int k = 0; k < kWarps; ++k)
        if (share_norm[k] > 0.0f) top = fmaxf(top, share_top[k]);
    norm = 0.0f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < kWarps; ++k) {
        const float weight = share_norm[k] > 0.0f ? exp2f(share_top[k] - top) : 0.0f;
        const float4 other = share_acc[k][lane];
        norm += share_norm[k] * weight;
        acc.x += other.x * weight;
        acc.y += other.y * weight;
        acc.z += other.z * weight;
        acc.w += other.w * weight;
    }
    return true;
}

// BF16 O + log2 LSE of a merged row: lane l writes dims 4l .. 4l + 3.
__device__ __forceinline__ void publish_merged(float top, float norm, float4 acc, int lane,
                                               __nv_bfloat16 *out_row, float *lse_slot) {
    uint2 packed;
    packed.x = pack_bf16(acc.x / norm, acc.y / norm);
    packed.y = pack_bf16(acc.z / norm, acc.w / norm);
    *reinterpret_cast<uint2 *>(out_row + lane * 4) = packed;
    if (lane == 0) *lse_slot = top + log2f(norm);
}

template <int kBatch = kMergeBatch, typename StateOf>
__device__ __forceinline__ void merge_states(StateOf state_of, int n, int lane, bool publish,
                                             __nv_bfloat16 *out_row, float *lse_slot) {
    float top, norm;
    float4 acc;
    if (!merge_partial<kBatch>(state_of, n, lane, top, norm, acc) || !publish) return;
    if (!(norm > 0.0f)) return; // every state was empty: nothing to publish
    publish_merged(top, norm, acc, lane, out_row, lse_slot);
}

// kRows rows of at most four states each, merged by one warp with the loads of all of them in
// flight together (a warp that merges the sixteen rows of its tile one by one pays sixteen round
// trips to the L2; this pays four).  state_of(row, i) is state i of row `row` (row < rows);
// publish(row, top, norm, acc) receives every row that has a finite, unpoisoned result.  The
// arithmetic is merge_partial's short path.
template <int kRows, typename StateOf, typename Publish>
__device__ __forceinline__ void merge_few_states_of_rows(StateOf state_of, int n, int rows,
                                                         int lane, Publish publish) {
    float part_max[kRows][4], part_norm[kRows][4];
    float2 lo[kRows][4], hi[kRows][4];
#pragma unroll
    for (int row = 0; row < kRows; ++row)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            part_max[row][i] = part_norm[row][i] = 0.0f;
            lo[row][i] = hi[row][i] = make_float2(0.f, 0.f);
            if (row < rows && i < n) {
                const float *s = state_of(row, i);
                part_max[row][i] = __ldcg(s);
                part_norm[row][i] = __ldcg(s + 1);
                lo[row][i] = __ldcg(reinterpret_cast<const float2 *>(s + 2 + lane * 4));
                hi[row][i] = __ldcg(reinterpret_cast<const float2 *>(s + 4 + lane * 4));
            }
        }
#pragma unroll
    for (int row = 0; row < kRows; ++row) {
        if (row >= rows) break;
        float top = -INFINITY;
        bool poisoned = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            poisoned |= part_norm[row][i] < 0.0f;
            if (part_norm[row][i] > 0.0f) top = fmaxf(top, part_max[row][i]);
        }
        float norm = 0.0f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float weight =
                part_norm[row][i] > 0.0f ? exp2f(part_max[row][i] - top) : 0.0f;
            norm += part_norm[row][i] * weight;
            acc.x += lo[row][i].x * weight;
            acc.y += lo[row][i].y * weight;
            acc.z += hi[row][i].x * weight;
            acc.w += hi[row][i].y * weight;
        }
        if (!poisoned && norm > 0.0f) publish(row, top, norm, acc);
    }
}

// As merge_states, by the kWarps warps of a CTA for one item (every thread of the CTA calls).
template <int kWarps, typename StateOf>
__device__ __forceinline__ void merge_states_shared(StateOf state_of, int n, int lane, int part,
                                                    __nv_bfloat16 *out_row, float *lse_slot) {
    float top, norm;
    float4 acc;
    if (!merge_partial_shared<kWarps>(state_of, n, lane, part, top, norm, acc)) return;
    if (!(norm > 0.0f)) return;
    publish_merged(top, norm, acc, lane, out_row, lse_slot);
}

// As merge_states, into the row of `request`, query head `head` of every rank's copy of the
// gathered result.  The row map and the peers' addresses (lane p holds rank p's) are fetched
// before the states, so that the stores at the end wait for nothing.
template <int kWarps = 1, typename StateOf>
__device__ __forceinline__ void merge_states_to_peers(StateOf state_of, int n, int lane,
                                                      bool publish, const PeerOut &peer,
                                                      int request, int head, int part = 0) {
    const int dest = peer.dest_rows[request];
    __nv_bfloat16 *out_of_lane =
        lane < peer.world ? static_cast<__nv_bfloat16 *>(peer.out[lane]) : nullptr;
    float *lse_of_lane = lane < peer.world ? peer.lse[lane] : nullptr;
    float top, norm;
    float4 acc;
    bool ok;
    if (kWarps == 1) ok = merge_partial<8>(state_of, n, lane, top, norm, acc);
    else ok = merge_partial_shared<kWarps>(state_of, n, lane, part, top, norm, acc);
    ok = ok && publish && norm > 0.0f;
    const long long row = (long long)dest * peer.gathered_qh + peer.head_offset + head;
    for (int p = 0; p < peer.world; ++p) {
        __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(
            __shfl_sync(0xffffffffu, (unsigned long long)out_of_lane, p));
        float *lse = reinterpret_cast<float *>(
            __shfl_sync(0xffffffffu, (unsigned long long)lse_of_lane, p));
        if (ok) publish_merged(top, norm, acc, lane, out + row * kHeadDim, lse + row);
    }
}

// The epoch hand-shake of a merge kernel (CTAs of a few warps, no shared memory): warp 0 fetches
// what the hand-shake needs before the merge, every thread calls this after it.
struct MergeSignalPrefetch {
    uint32_t *flag_of_lane;
    const uint32_t *my_flags;
    uint32_t epoch;
    __device__ __forceinline__ void fetch(const PeerSignal &s) {
        flag_of_lane = nullptr;
        my_flags = nullptr;
        epoch = 0;
        if (s.world == 0 || threadIdx.x >= 32) return;
        if ((int)threadIdx.x < s.world) flag_of_lane = s.flags[threadIdx.x];
        my_flags = s.flags[s.rank];
        epoch = *s.epoch;
    }
    __device__ __forceinline__ void finish(const PeerSignal &s) const {
        // a command that leaves the epoch to a later command of the step has nothing to do: its
        // rows are ordered before that command's kernels by the stream
        if (s.world == 0 || s.defer) return;
        __syncthreads();
        if (threadIdx.x >= 32) return;
        peer_signal_and_wait(s, flag_of_lane, my_flags, epoch);
    }
};

// The even cut of `total` units over `workers` workers, evaluated without 64-bit division:
// begin(w) = floor(total * w / workers) = q * w + floor(r * w / workers) with total = q *
// workers + r.  Fewer workers than `max_workers` are used when there is little work, so that a
// worker never gets less than kMinUnitsPerWorker pages (fewer states to merge).
constexpr int kMinUnitsPerWorker = 4;
struct EvenCut {
    long long q;
    int r, workers;
    __device__ __forceinline__ EvenCut(long long total, int max_workers) {
        const long long wanted = total / kMinUnitsPerWorker;
        workers = wanted >= max_workers ? max_workers : (wanted < 1 ? 1 : (int)wanted);
        q = total / workers;
        r = (int)(total - q * workers);
    }
    // a cut computed earlier (the 64-bit division above costs a warp hundreds of instructions)
    __device__ __forceinline__ EvenCut(long long q_, int r_, int workers_)
        : q(q_), r(r_), workers(workers_) {}
    __device__ __forceinline__ long long begin(int w) const {
        return q * w + (long long)((unsigned)r * (unsigned)w / (unsigned)workers);
    }
    // the worker whose range [begin(w), begin(w + 1)) contains x: begin(w) <= x means
    // total * w / workers < x + 1, i.e. w <= ((x + 1) * workers - 1) / total
    __device__ __forceinline__ int owner(long long x) const {
        const long long total = q * workers + r;
        return (int)(((x + 1) * workers - 1) / total);
    }
    // the same without a 64-bit division: a double-precision estimate (exact to well below one
    // worker for any total this library accepts), then at most a step either way
    __device__ __forceinline__ int owner_fast(long long x) const {
        const double total = (double)q * (double)workers + (double)r;
        int w = (int)(((double)(x + 1) * (double)workers - 1.0) / total);
        w = w < 0 ? 0 : (w >= workers ? workers - 1 : w);
        while (w > 0 && begin(w) > x) --w;
        while (w + 1 < workers && begin(w + 1) <= x) ++w;
        return w;
    }
};

} // namespace dev
} // namespace lb
