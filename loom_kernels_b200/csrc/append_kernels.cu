// Fused NeoX RoPE (theta 10000, D128) + paged KV append for sm_100a.
//
// Replaces the reference's rope_paged_kv_append_bf16_neox_d128 and
// rope_paged_kv_append_tokens_bf16_neox_d128 kernels
// (crates/loom-infer-cuda/src/rope/mod.rs:119-230,259-405).  rope_append_kernel serves the
// one-token-per-request contract and the explicit <=64-token contract (the any-total extension
// is the validate + scatter pair further down):
//
//   0. a CTA starts on its tokens at once: the first token's Q/K/V rows are fetched into
//      registers and the sin/cos tables of its first eight tokens are computed, 64 threads per
//      token (from in-bounds loads only), while
//   1. every CTA validates the whole call against device-resident metadata (page table, token
//      mapping, physical-slot uniqueness via a shared-memory hash set) and returns without
//      writing when anything is invalid, so a call is all-or-nothing exactly like the
//      reference's guards (rope/mod.rs:140-182,290-343).  The validation is laid out for
//      memory-level parallelism: four independent loads per thread per step, and the in-bounds
//      levels of the token -> request -> page chain are issued before the page-table verdict;
//   2. the CTA then walks its tokens (token, token + grid, ...): 8 lanes per head row rotate Q
//      and K with 16-byte loads/stores (a rotation pair (i, i+64) lives in one thread), scatter
//      K and copy V rows to the token's page slot, while the next token's rows are already on
//      their way into a second register set.
//
// Angles use the host-computed inverse frequencies powf(10000, -2i/128) (constant memory), so
// they are bit-identical to the CPU reference (crates/loom-infer/src/rope/mod.rs:148-150);
// the rotation is evaluated without FMA contraction like the reference (:154-155).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "bounds_check.cuh"
#include "dependent_launch.cuh"
#include "kernels.hpp"

namespace lb {
namespace {

using dev::in_bounds;

constexpr int kHeadDim = 128;
constexpr int kPairs = 64;
constexpr int kPage = 16;
constexpr int kThreads = 512;
constexpr int kTables = kThreads / kPairs;        // sin/cos tables computed in one go
constexpr int kMaxTokensPerCta = 128;            // the plan sizes the grid so that no CTA gets more

__constant__ float c_inverse_frequency[kPairs];

struct AppendArgs {
    const uint4 *query, *key, *value;
    const int32_t *batch_indices, *positions, *indptr, *indices, *last;
    uint4 *query_output, *key_pages, *value_pages;
    int32_t tokens, batch, max_pages, qh, kvh, indices_len, indices_min, hash_slots;
    int32_t *status;         // the checked build records an index outside its operand here
    int32_t workspace_numel; // I32 elements bound as the workspace of an extended plan
};

// Levels 1-2 of the token -> request -> page chain, from in-bounds loads only: an out-of-range
// request reads request 0 instead.  `position` and `start` mean something only if the page table
// is valid; the verdict on the token is the return value (to be combined with the table's).
// One-token-per-request plans derive request and position from the page table.
__device__ __forceinline__ bool token_request(const AppendArgs &a, int token, int &position,
                                              int &start) {
    const bool explicit_tokens = a.batch_indices != nullptr;
    const int request_raw = explicit_tokens ? a.batch_indices[token] : token;
    const int position_raw = explicit_tokens ? a.positions[token] : 0;
    const bool ok = request_raw >= 0 && request_raw < a.batch && position_raw >= 0;
    const int request = ok ? request_raw : 0;
    start = a.indptr[request];
    const int pages = a.indptr[request + 1] - start;
    const int kv_len = (pages - 1) * kPage + a.last[request];
    position = explicit_tokens ? position_raw : kv_len - 1;
    return ok && position < kv_len;
}

// The position the rotation of `token` uses, from in-bounds loads only (it may be garbage when
// the call is invalid; nothing is written in that case).
__device__ __forceinline__ int speculative_position(const AppendArgs &a, int token) {
    if (a.batch_indices) return a.positions[token];
    return (a.indptr[token + 1] - a.indptr[token] - 1) * kPage + a.last[token] - 1;
}

// Outside the range of the reduction below (an angle of 2^32 or more, or a garbage position of a
// call that will be rejected): the library routine, kept out of line.
__device__ __noinline__ float2 sincos_any(double x) {
    double s, c;
    sincos(x, &s, &c);
    return make_float2((float)s, (float)c);
}

// (sin, cos) of an F32 angle in [0, 2^32), evaluated in double and rounded once, which reproduces the host
// libm's (near correctly rounded) sinf/cosf: absolute error below 2e-16 before the rounding.
// The angle is reduced by k * pi/2 with pi/2 split into three 20-bit pieces (k * piece is exact
// for k < 2^32) and a tail; both functions are then summed as Taylor series on [-pi/4, pi/4]
// (degrees 17 and 18: the first omitted terms are below 1e-19).  A third of the instructions of
// the general-purpose routine, no local memory, and short enough to leave registers for the rows.
__device__ __forceinline__ float2 sincos_in_range(double x) { // 0 <= x < 2^32
    const double k = rint(x * 0x1.45f306dc9c883p-1); // x * 2/pi
    double r = fma(-k, 0x1.921fa00000000p+0, x);
    r = fma(-k, 0x1.5444200000000p-20, r);
    r = fma(-k, 0x1.a308c00000000p-41, r);
    r = fma(-k, 0x1.313198a2e0370p-61, r);
    const double r2 = r * r;
    double s = 1.0 / 355687428096000.0;       //  1/17!
    s = fma(s, r2, -1.0 / 1307674368000.0);   // -1/15!
    s = fma(s, r2, 1.0 / 6227020800.0);       //  1/13!
    s = fma(s, r2, -1.0 / 39916800.0);        // -1/11!
    s = fma(s, r2, 1.0 / 362880.0);           //  1/9!
    s = fma(s, r2, -1.0 / 5040.0);            // -1/7!
    s = fma(s, r2, 1.0 / 120.0);              //  1/5!
    s = fma(s, r2, -1.0 / 6.0);               // -1/3!
    s = fma(s, r2, 1.0);
    s *= r;
    double c = -1.0 / 6402373705728000.0;     // -1/18!
    c = fma(c, r2, 1.0 / 20922789888000.0);   //  1/16!
    c = fma(c, r2, -1.0 / 87178291200.0);     // -1/14!
    c = fma(c, r2, 1.0 / 479001600.0);        //  1/12!
    c = fma(c, r2, -1.0 / 3628800.0);         // -1/10!
    c = fma(c, r2, 1.0 / 40320.0);            //  1/8!
    c = fma(c, r2, -1.0 / 720.0);             // -1/6!
    c = fma(c, r2, 1.0 / 24.0);               //  1/4!
    c = fma(c, r2, -0.5);
    c = fma(c, r2, 1.0);
    const int quadrant = (int)((long long)k & 3);
    const double sine = (quadrant & 1) ? c : s, cosine = (quadrant & 1) ? s : c;
    return make_float2((float)((quadrant & 2) ? -sine : sine),
                       (float)(((quadrant + 1) & 2) ? -cosine : cosine));
}

// Any F32 angle: the stand-alone RoPE takes theta and scale from the caller.
__device__ __forceinline__ float2 sincos_of_f32_angle(float angle) {
    const double x = (double)angle;
    return x >= 0.0 && x < 4294967296.0 ? sincos_in_range(x) : sincos_any(x);
}

// (sin, cos) of rotation pair `pair` at `position` for the append (theta 10000, scale 1); the
// F32 angle is exactly the reference's.  Positions are below 2^31 and the inverse frequencies
// at most 1, so the angle is always inside the reduction's range; the garbage position of a
// call that is going to be rejected yields garbage that is never stored.
__device__ __forceinline__ float2 pair_sincos(int position, int pair) {
    return sincos_in_range((double)__fmul_rn((float)position, c_inverse_frequency[pair]));
}

__device__ __forceinline__ uint32_t rotate_pack(uint32_t lo_bits, uint32_t hi_bits, float2 sc0,
                                                float2 sc1, uint32_t &hi_out) {
    // lo_bits holds components (i, i+1) of the first half, hi_bits (i+64, i+65)
    const float x0 = __uint_as_float(lo_bits << 16), x1 = __uint_as_float(lo_bits & 0xffff0000u);
    const float y0 = __uint_as_float(hi_bits << 16), y1 = __uint_as_float(hi_bits & 0xffff0000u);
    const float a0 = __fsub_rn(__fmul_rn(x0, sc0.y), __fmul_rn(y0, sc0.x));
    const float b0 = __fadd_rn(__fmul_rn(y0, sc0.y), __fmul_rn(x0, sc0.x));
    const float a1 = __fsub_rn(__fmul_rn(x1, sc1.y), __fmul_rn(y1, sc1.x));
    const float b1 = __fadd_rn(__fmul_rn(y1, sc1.y), __fmul_rn(x1, sc1.x));
    __nv_bfloat162 lo = __floats2bfloat162_rn(a0, a1);
    __nv_bfloat162 hi = __floats2bfloat162_rn(b0, b1);
    hi_out = *reinterpret_cast<uint32_t *>(&hi);
    return *reinterpret_cast<uint32_t *>(&lo);
}

// lane j of 8 owns dims [8j, 8j+8) (lo) and [64+8j, 64+8j+8) (hi) of the 128-wide row
__device__ __forceinline__ void rotate_row(uint4 lo, uint4 hi, uint4 *dst, int j,
                                           const float2 *sincos) {
    const float4 *sc = reinterpret_cast<const float4 *>(sincos + 8 * j);
    const float4 t0 = sc[0], t1 = sc[1], t2 = sc[2], t3 = sc[3];
    uint4 out_lo, out_hi;
    out_lo.x = rotate_pack(lo.x, hi.x, make_float2(t0.x, t0.y), make_float2(t0.z, t0.w), out_hi.x);
    out_lo.y = rotate_pack(lo.y, hi.y, make_float2(t1.x, t1.y), make_float2(t1.z, t1.w), out_hi.y);
    out_lo.z = rotate_pack(lo.z, hi.z, make_float2(t2.x, t2.y), make_float2(t2.z, t2.w), out_hi.z);
    out_lo.w = rotate_pack(lo.w, hi.w, make_float2(t3.x, t3.y), make_float2(t3.z, t3.w), out_hi.w);
    dst[j] = out_lo;
    dst[8 + j] = out_hi;
}

// The rows of one token a thread works on, fetched ahead of their use: row task tid (8 tasks
// per Q/K row) and V chunk tid.  Tokens with more rows than that take the remainder straight
// from memory.
struct TokenRows {
    uint4 lo, hi, v;
};

__device__ __forceinline__ const uint4 *row_source(const AppendArgs &a, int token, int row) {
    return row < a.qh ? a.query + ((size_t)token * a.qh + row) * (kHeadDim / 8)
                      : a.key + ((size_t)token * a.kvh + (row - a.qh)) * (kHeadDim / 8);
}
__device__ __forceinline__ uint4 *row_destination(const AppendArgs &a, int token, int slot,
                                                  int row) {
    return row < a.qh ? a.query_output + ((size_t)token * a.qh + row) * (kHeadDim / 8)
                      : a.key_pages + ((size_t)slot * a.kvh + (row - a.qh)) * (kHeadDim / 8);
}

__device__ __forceinline__ void fetch_token(const AppendArgs &a, int token, int tid,
                                            TokenRows &rows) {
    if (!in_bounds(token, a.tokens, a.status, dev::kSiteAppendToken)) return;
    if (tid < (a.qh + a.kvh) * 8) {
        const uint4 *src = row_source(a, token, tid >> 3);
        rows.lo = src[tid & 7];
        rows.hi = src[8 + (tid & 7)];
    }
    if (tid < a.kvh * 16) rows.v = a.value[(size_t)token * a.kvh * 16 + tid];
}

__device__ __forceinline__ void store_token(const AppendArgs &a, int token, int slot, int tid,
                                            const TokenRows &rows, const float2 *sincos) {
    const int row_tasks = (a.qh + a.kvh) * 8; // 8 lanes per 128-wide row
    const int copy_tasks = a.kvh * 16;        // V rows: 16 x 16-byte chunks per KV head
    if (!in_bounds(token, a.tokens, a.status, dev::kSiteAppendToken) ||
        !in_bounds(slot, (long long)a.max_pages * kPage, a.status, dev::kSiteAppendPool))
        return;
    if (tid < row_tasks)
        rotate_row(rows.lo, rows.hi, row_destination(a, token, slot, tid >> 3), tid & 7, sincos);
    for (int task = tid + kThreads; task < row_tasks; task += kThreads) {
        const uint4 *src = row_source(a, token, task >> 3);
        rotate_row(src[task & 7], src[8 + (task & 7)], row_destination(a, token, slot, task >> 3),
                   task & 7, sincos);
    }
    if (tid < copy_tasks) a.value_pages[(size_t)slot * copy_tasks + tid] = rows.v;
    for (int task = tid + kThreads; task < copy_tasks; task += kThreads)
        a.value_pages[(size_t)slot * copy_tasks + task] =
            a.value[(size_t)token * copy_tasks + task];
}

__global__ void __launch_bounds__(kThreads, 2) rope_append_kernel(const AppendArgs a) {
    extern __shared__ int hash_table[];
    __shared__ __align__(16) float2 sincos_table[kTables][kPairs]; // (sin, cos) per pair and token
    __shared__ int2 mine[kMaxTokensPerCta];                  // (position, slot) of my tokens
    dev::dependent_launch_release();
    const int tid = threadIdx.x;
    const int grid = (int)gridDim.x;
    for (int i = tid; i < a.hash_slots; i += kThreads) hash_table[i] = -1;
    dev::dependent_launch_wait(); // global memory is touched from here on

    // ---- 0. start on this CTA's first token while the call is being validated ---------------
    const int first_token = blockIdx.x;
    const int count = first_token < a.tokens ? (a.tokens - first_token + grid - 1) / grid : 0;
    TokenRows rows;
    if (count > 0) fetch_token(a, first_token, tid, rows);
    // The sin/cos tables of my first kTables tokens, 64 threads per token, taken from the top of
    // the CTA (the low threads carry the token mapping of small calls).  Double-precision
    // sin/cos is the slowest single step of a small call, so it starts first and runs beside
    // the validation; positions come from in-bounds loads and are confirmed by the validation.
    {
        const int r = kThreads - 1 - tid;
        if (r / kPairs < min(count, kTables))
            sincos_table[r / kPairs][r % kPairs] =
                pair_sincos(speculative_position(a, first_token + (r / kPairs) * grid), r % kPairs);
    }
    // levels 1-2 of the first four tokens of this thread (in-bounds whatever the metadata holds)
    int position[4], start[4];
    bool ok[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int token = u * kThreads + tid;
        position[u] = start[u] = 0;
        ok[u] = token < a.tokens ? token_request(a, token, position[u], start[u]) : true;
    }

    // ---- 1. whole-call validation (identical in every CTA) -----------------------------------
    // the table ends at page_indptr[batch], which must lie in [indices_min, indices_len] (equal
    // bounds unless the plan was made with the capacity option); entries past it are not read
    const int final_indptr = a.indptr[a.batch];
    bool invalid = a.indptr[0] != 0 || final_indptr < a.indices_min || final_indptr > a.indices_len;
    int table_end = a.indices_len; // known without a load unless the plan has the capacity option
    if (a.indices_min != a.indices_len) table_end = min(max(final_indptr, 0), a.indices_len);
    for (int request = tid; request < a.batch; request += kThreads) {
        const int begin = a.indptr[request], end = a.indptr[request + 1], tail = a.last[request];
        if (begin < 0 || end <= begin || end > table_end || tail < 1 || tail > kPage)
            invalid = true;
    }
    // (eight loads per thread per round: a table of up to 4096 pages -- the C2 calls have 2100 --
    // is one round trip, not two)
    for (int base = 0; base < table_end; base += 8 * kThreads) {
        int id[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int page = base + u * kThreads + tid;
            id[u] = page < table_end ? a.indices[page] : 0;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) invalid |= id[u] < 0 || id[u] >= a.max_pages;
    }
    if (__syncthreads_or(invalid)) return;

    // token mapping: the page lookups of four tokens per thread travel together, then the
    // physical slots go into the hash set (meeting the same key = two tokens share a slot)
    for (int base = 0; base < a.tokens; base += 4 * kThreads) {
        int slot[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int token = base + u * kThreads + tid;
            if (base > 0)
                ok[u] = token < a.tokens ? token_request(a, token, position[u], start[u]) : true;
            const bool live = token < a.tokens && ok[u];
            const int page = live ? start[u] + position[u] / kPage : 0;
            slot[u] = (in_bounds(page, a.indices_len, a.status, dev::kSiteIndices)
                           ? a.indices[page]
                           : 0) * kPage + position[u] % kPage;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int token = base + u * kThreads + tid;
            if (token >= a.tokens) continue;
            if (!ok[u]) {
                invalid = true;
                continue;
            }
            if (token >= first_token && (token - first_token) % grid == 0)
                mine[(token - first_token) / grid] = make_int2(position[u], slot[u]);
            unsigned h = ((unsigned)slot[u] * 2654435761u) & (unsigned)(a.hash_slots - 1);
            for (int probe = 0; probe < a.hash_slots; ++probe) {
                const int seen = atomicCAS(&hash_table[h], -1, slot[u]);
                if (seen == -1) break;
                if (seen == slot[u]) {
                    invalid = true;
                    break;
                }
                h = (h + 1) & (unsigned)(a.hash_slots - 1);
            }
        }
    }
    if (__syncthreads_or(invalid)) return;
    if (first_token >= a.tokens) return;

    // ---- 2. rotate + scatter: token k's rows are in registers and its table in shared memory
    //         when its turn comes; token k + 1 is fetched while token k is rotated ------------------
    for (int k = 0; k < count; ++k) {
        const int token = first_token + k * grid;
        if (k > 0 && k % kTables == 0) {
            // the next kTables tables (only calls with more than kTables tokens per CTA get here)
            __syncthreads();
            const int r = kThreads - 1 - tid;
            if (k + r / kPairs < count)
                sincos_table[r / kPairs][r % kPairs] = pair_sincos(mine[k + r / kPairs].x, r % kPairs);
            __syncthreads();
        }
        // two tokens per round with two register sets, so that a fetched row is never moved (a
        // register move would wait for the load it copies)
        TokenRows other;
        if (k + 1 < count) fetch_token(a, token + grid, tid, other);
        store_token(a, token, mine[k].y, tid, rows, sincos_table[k % kTables]);
        if (++k == count) break; // k is odd now: never a table boundary (kTables is even)
        if (k + 1 < count) fetch_token(a, token + 2 * grid, tid, rows);
        store_token(a, token + grid, mine[k].y, tid, other, sincos_table[k % kTables]);
    }
}

// ---- the any-total append as two commands ----------------------------------------------------------
//
// Calls with hundreds or thousands of tokens pay too much for a validation that every CTA
// repeats.  The extended plan therefore validates ONCE, in a kernel of its own, and leaves its
// findings in a small caller-bound I32 workspace:
//
//     workspace[0 .. 32)                verdict of validation CTA i (0 = nothing wrong)
//     workspace[32 + 2t], [33 + 2t]     (position, physical slot) of token t
//
// append_validate_kernel: CTA 0 maps the tokens (and checks slot uniqueness in a shared-memory
// hash set), the other CTAs share the page-table and request checks.  It waits for the work
// before it FIRST and only then releases its dependent, so that
// append_scatter_kernel (one CTA per token) may read its inputs, build the sin/cos table and rotate
// the rows in registers while the validation is still running; it waits for the verdict only
// before it stores.  All-or-nothing as before: any non-zero verdict and nothing is written.
constexpr int kVerdictSlots = 32;
constexpr int kValidateThreads = 1024;
constexpr int kScatterThreads = 256;

// The validation of one call by validator CTA `cta` of `ctas` (`threads` threads each): true when
// this CTA found something invalid.  CTA 0 maps the tokens into the workspace.
// kTokens: tokens whose dependent loads one thread keeps in flight per round of the mapping.
template <int kTokens>
__device__ __forceinline__ bool validate_call(const AppendArgs &a, int32_t *workspace, int cta,
                                              int ctas, int threads, int *hash_table) {
    const int tid = threadIdx.x;
    bool invalid = false;
    if (cta > 0 || ctas == 1) {
        // page-table and request checks, sliced over the scanning CTAs
        const int scanners = ctas == 1 ? 1 : ctas - 1;
        const int me = ctas == 1 ? 0 : cta - 1;
        const int final_indptr = a.indptr[a.batch]; // must lie in [indices_min, indices_len]
        invalid = a.indptr[0] != 0 || final_indptr < a.indices_min || final_indptr > a.indices_len;
        int table_end = a.indices_len;
        if (a.indices_min != a.indices_len) table_end = min(max(final_indptr, 0), a.indices_len);
        for (int request = me * threads + tid; request < a.batch;
             request += scanners * threads) {
            const int begin = a.indptr[request], end = a.indptr[request + 1];
            const int tail = a.last[request];
            if (begin < 0 || end <= begin || end > table_end || tail < 1 || tail > kPage)
                invalid = true;
        }
        for (int base = me * 4 * threads; base < table_end;
             base += scanners * 4 * threads) {
            int id[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int page = base + u * threads + tid;
                id[u] = page < table_end ? a.indices[page] : 0;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) invalid |= id[u] < 0 || id[u] >= a.max_pages;
        }
    }
    if (cta == 0) {
        for (int i = tid; i < a.hash_slots; i += threads) hash_table[i] = -1;
        if (tid >= ctas && tid < kVerdictSlots) workspace[tid] = 0; // unused verdicts
        __syncthreads();
        for (int base = 0; base < a.tokens; base += kTokens * threads) {
            int position[kTokens], start[kTokens], slot[kTokens];
            bool ok[kTokens];
#pragma unroll
            for (int u = 0; u < kTokens; ++u) {
                const int token = base + u * threads + tid;
                position[u] = start[u] = 0;
                ok[u] = token < a.tokens ? token_request(a, token, position[u], start[u]) : false;
            }
#pragma unroll
            for (int u = 0; u < kTokens; ++u) {
                // the table itself is being checked elsewhere: stay inside page_indices
                const long long page = (long long)start[u] + position[u] / kPage;
                ok[u] = ok[u] && page >= 0 && page < a.indices_len;
                slot[u] = a.indices[ok[u] ? (int)page : 0] * kPage + position[u] % kPage;
            }
#pragma unroll
            for (int u = 0; u < kTokens; ++u) {
                const int token = base + u * threads + tid;
                if (token >= a.tokens) continue;
                if (in_bounds(kVerdictSlots + 2 * token + 1, a.workspace_numel, a.status,
                              dev::kSiteAppendWorkspace)) {
                    workspace[kVerdictSlots + 2 * token] = position[u];
                    workspace[kVerdictSlots + 2 * token + 1] = slot[u];
                }
                if (!ok[u]) {
                    invalid = true;
                    continue;
                }
                unsigned h = ((unsigned)slot[u] * 2654435761u) & (unsigned)(a.hash_slots - 1);
                for (int probe = 0; probe < a.hash_slots; ++probe) {
                    const int seen = atomicCAS(&hash_table[h], -1, slot[u]);
                    if (seen == -1) break;
                    if (seen == slot[u]) {
                        invalid = true;
                        break;
                    }
                    h = (h + 1) & (unsigned)(a.hash_slots - 1);
                }
            }
        }
    }
    return invalid;
}

__global__ void __launch_bounds__(kValidateThreads)
append_validate_kernel(const AppendArgs a, int32_t *workspace) {
    extern __shared__ int hash_table[];
    dev::dependent_launch_wait();    // the inputs may come from the command before this one
    dev::dependent_launch_release(); // from here on everything before this command is complete
    const bool invalid = validate_call<4>(a, workspace, (int)blockIdx.x, (int)gridDim.x,
                                          kValidateThreads, hash_table);
    const int verdict = __syncthreads_or(invalid);
    if (threadIdx.x == 0) workspace[blockIdx.x] = verdict;
}

// One token of an any-total call, in two steps: fetch its rows, rotate-ready, into registers and
// build its sin/cos table (from in-bounds loads only, before the verdict is known), then store.
struct ScatterRows {
    uint4 lo[2], hi[2], v;
};

__device__ __forceinline__ void scatter_fetch(const AppendArgs &a, int token, int tid,
                                              ScatterRows &rows, float2 *table) {
    const int row_tasks = (a.qh + a.kvh) * 8, copy_tasks = a.kvh * 16;
    rows.v = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int task = tid + i * kScatterThreads;
        rows.lo[i] = rows.hi[i] = make_uint4(0, 0, 0, 0);
        if (task < row_tasks) {
            const uint4 *src = row_source(a, token, task >> 3);
            rows.lo[i] = src[task & 7];
            rows.hi[i] = src[8 + (task & 7)];
        }
    }
    if (tid < copy_tasks) rows.v = a.value[(size_t)token * copy_tasks + tid];
    if (tid < kPairs) table[tid] = pair_sincos(speculative_position(a, token), tid);
}

__device__ __forceinline__ void scatter_store(const AppendArgs &a, int token, int slot, int tid,
                                              const ScatterRows &rows, const float2 *table) {
    const int row_tasks = (a.qh + a.kvh) * 8, copy_tasks = a.kvh * 16;
    if (!in_bounds(slot, (long long)a.max_pages * kPage, a.status, dev::kSiteAppendPool)) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int task = tid + i * kScatterThreads;
        if (task < row_tasks)
            rotate_row(rows.lo[i], rows.hi[i], row_destination(a, token, slot, task >> 3), task & 7,
                       table);
    }
    for (int task = tid + 2 * kScatterThreads; task < row_tasks; task += kScatterThreads) {
        const uint4 *src = row_source(a, token, task >> 3);
        rotate_row(src[task & 7], src[8 + (task & 7)], row_destination(a, token, slot, task >> 3),
                   task & 7, table);
    }
    if (tid < copy_tasks) a.value_pages[(size_t)slot * copy_tasks + tid] = rows.v;
    for (int task = tid + kScatterThreads; task < copy_tasks; task += kScatterThreads)
        a.value_pages[(size_t)slot * copy_tasks + task] = a.value[(size_t)token * copy_tasks + task];
}

__global__ void __launch_bounds__(kScatterThreads, 8)
append_scatter_kernel(const AppendArgs a, const int32_t *workspace) {
    __shared__ __align__(16) float2 table[kPairs];
    dev::dependent_launch_release();
    const int tid = threadIdx.x;
    const int token = blockIdx.x;
    // The validation kernel released this one only after everything before the call had
    // completed, so the call's inputs are final: fetch, rotate and keep the result in registers.
    ScatterRows rows;
    scatter_fetch(a, token, tid, rows, table);
    __syncthreads();
    dev::dependent_launch_wait(); // the verdicts and this token's slot are final
    // the slot travels with the verdicts (one round trip, not two); it is used only if they agree
    const int slot = __ldcg(workspace + kVerdictSlots + 2 * token + 1);
    const int verdict = __syncthreads_or(tid < kVerdictSlots ? __ldcg(workspace + tid) : 0);
    if (verdict != 0) return;
    scatter_store(a, token, slot, tid, rows, table);
}

// ---- the any-total append as ONE command ---------------------------------------------------------
//
// The same two roles in one grid: the first `validators` CTAs validate (CTA 0 maps the tokens into
// the workspace), every other CTA owns tokens.  A token CTA fetches and prepares its first token
// while the validators work, then waits -- bounded -- for their verdicts on words of the queue
// (0 = not yet, 1 = nothing wrong, 2 = invalid) instead of for the end of a kernel, and stores.
// The plan sizes the grid so that every CTA is resident at once, so a waiting CTA never keeps a
// validator off the GPU.  The last CTA of the grid to finish hands the words back as zeros; the
// queue's stream orders the next command after that.
constexpr long long kVerdictWaitCycles = 4000000000ll; // ~2 s of SM clock

__device__ __forceinline__ int load_acquire_gpu(const int32_t *p) {
    int value;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(value) : "l"(p) : "memory");
    return value;
}

// (Four CTAs per SM: the validators' code shares the kernel's register budget and spills at the
// 32 registers that eight CTAs would leave; a token CTA holds two tokens ahead of the verdict
// instead, so a call of up to 2 x 4 x SMs tokens is still one round.)
constexpr int kFusedTokensAhead = 2;

__global__ void __launch_bounds__(kScatterThreads, 4)
append_fused_kernel(const AppendArgs a, int32_t *workspace, int32_t *words, int validators) {
    extern __shared__ int hash_table[];
    __shared__ __align__(16) float2 table[kFusedTokensAhead][kPairs];
    dev::dependent_launch_release();
    dev::dependent_launch_wait(); // global memory (and the queue's words) from here on
    const int tid = threadIdx.x;
    if ((int)blockIdx.x < validators) {
        // (eight tokens per thread: a quarter of the validation kernel's threads map a call of
        // up to 2048 tokens in one round of dependent loads all the same)
        const bool invalid = validate_call<8>(a, workspace, (int)blockIdx.x, validators,
                                              kScatterThreads, hash_table);
        // (the barrier orders every thread's workspace stores before the release below)
        const int verdict = __syncthreads_or(invalid);
        if (tid == 0) {
            __threadfence();
            atomicExch(words + blockIdx.x, verdict ? 2 : 1);
        }
    } else {
        const int token_ctas = (int)gridDim.x - validators;
        int token = (int)blockIdx.x - validators;
        ScatterRows rows[kFusedTokensAhead];
#pragma unroll
        for (int i = 0; i < kFusedTokensAhead; ++i)
            if (token + i * token_ctas < a.tokens)
                scatter_fetch(a, token + i * token_ctas, tid, rows[i], table[i]);
        int seen = 1;
        if (tid < validators) {
            const long long start = clock64();
            while ((seen = load_acquire_gpu(words + tid)) == 0) {
                if (clock64() - start > kVerdictWaitCycles) break;
                __nanosleep(64); // (hundreds of CTAs poll the same few words)
            }
        }
        // (the barrier also publishes the sin/cos table and carries the acquire to every thread)
        const int bad = __syncthreads_or(seen != 1);
        if (bad) {
            if (seen == 0 && a.status) atomicExch(a.status, 1); // a wait ran out
        } else {
            int slot[kFusedTokensAhead];
#pragma unroll
            for (int i = 0; i < kFusedTokensAhead; ++i)
                slot[i] = token + i * token_ctas < a.tokens
                              ? __ldcg(workspace + kVerdictSlots + 2 * (token + i * token_ctas) + 1)
                              : 0;
#pragma unroll
            for (int i = 0; i < kFusedTokensAhead; ++i)
                if (token + i * token_ctas < a.tokens)
                    scatter_store(a, token + i * token_ctas, slot[i], tid, rows[i], table[i]);
            // (a grid smaller than half the call: the rest one token at a time)
            for (token += kFusedTokensAhead * token_ctas; token < a.tokens; token += token_ctas) {
                __syncthreads(); // table[0] has been used by everybody
                scatter_fetch(a, token, tid, rows[0], table[0]);
                __syncthreads();
                scatter_store(a, token, __ldcg(workspace + kVerdictSlots + 2 * token + 1), tid,
                              rows[0], table[0]);
            }
        }
    }
    // the last CTA to get here leaves the words as it found them: zero
    __syncthreads();
    if (tid == 0) {
        const unsigned done =
            atomicInc(reinterpret_cast<unsigned *>(words) + kVerdictSlots, gridDim.x - 1);
        if (done == gridDim.x - 1)
            for (int v = 0; v < validators; ++v) words[v] = 0;
    }
}

// Stand-alone NeoX RoPE over contiguous NHD Q and K (the reference's rope_pos_ids_bf16_neox_d128,
// crates/loom-infer-cuda/src/rope/mod.rs:44-94): the same rotation as the append, output to
// separate Q/K buffers.  A CTA walks tokens blockIdx.x, blockIdx.x + grid, ...; 64 threads build
// the token's sin/cos table, 8 lanes per head row rotate.  A token with a negative position id is
// left unwritten (the reference's device guard, :64-67); other tokens are not affected.
constexpr int kRopeThreads = 256;

struct RopeArgs {
    const uint4 *query, *key;
    const int32_t *position_ids;
    uint4 *query_output, *key_output;
    int32_t tokens, qh, kh;
    float inverse_frequency[kPairs]; // powf(theta, -2i/128) / scale, computed on the host
};

__global__ void __launch_bounds__(kRopeThreads) rope_pos_ids_kernel(const RopeArgs a) {
    __shared__ __align__(16) float2 table[kPairs];
    dev::dependent_launch_release();
    const int tid = threadIdx.x;
    const int row_tasks = (a.qh + a.kh) * 8;
    dev::dependent_launch_wait();
    for (int token = blockIdx.x; token < a.tokens; token += gridDim.x) {
        const int position = a.position_ids[token];
        if (position < 0) continue; // uniform over the CTA
        __syncthreads();            // the previous token's table is no longer read
        if (tid < kPairs) {
            table[tid] = sincos_of_f32_angle(__fmul_rn((float)position, a.inverse_frequency[tid]));
        }
        __syncthreads();
        for (int task = tid; task < row_tasks; task += kRopeThreads) {
            const int row = task >> 3, j = task & 7;
            const bool is_query = row < a.qh;
            const size_t offset = is_query ? ((size_t)token * a.qh + row) * (kHeadDim / 8)
                                           : ((size_t)token * a.kh + (row - a.qh)) * (kHeadDim / 8);
            const uint4 *src = (is_query ? a.query : a.key) + offset;
            uint4 *dst = (is_query ? a.query_output : a.key_output) + offset;
            rotate_row(src[j], src[8 + j], dst, j, table);
        }
    }
}

} // namespace

int launch_rope_pos_ids(const RopeLaunch &launch, void *stream) {
    RopeArgs args;
    args.query = static_cast<const uint4 *>(launch.query);
    args.key = static_cast<const uint4 *>(launch.key);
    args.position_ids = launch.position_ids;
    args.query_output = static_cast<uint4 *>(launch.query_output);
    args.key_output = static_cast<uint4 *>(launch.key_output);
    args.tokens = launch.tokens;
    args.qh = launch.qh;
    args.kh = launch.kh;
    for (int i = 0; i < kPairs; ++i) args.inverse_frequency[i] = launch.inverse_frequency[i];
    return launch_dependent(rope_pos_ids_kernel, launch.grid, kRopeThreads, 0, stream, args);
}

int configure_append_kernels(size_t max_dynamic_shared, const float *inverse_frequency) {
    int rc = cudaMemcpyToSymbol(c_inverse_frequency, inverse_frequency, sizeof(float) * kPairs);
    if (rc) return rc;
    rc = cudaFuncSetAttribute(append_validate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)max_dynamic_shared);
    if (rc) return rc;
    return cudaFuncSetAttribute(rope_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)max_dynamic_shared);
}

int append_block_threads() { return kThreads; }
int append_max_tokens_per_cta() { return kMaxTokensPerCta; }

static AppendArgs append_args(const AppendLaunch &launch) {
    AppendArgs args;
    args.query = static_cast<const uint4 *>(launch.query);
    args.key = static_cast<const uint4 *>(launch.key);
    args.value = static_cast<const uint4 *>(launch.value);
    args.batch_indices = launch.batch_indices;
    args.positions = launch.positions;
    args.indptr = launch.indptr;
    args.indices = launch.indices;
    args.last = launch.last;
    args.query_output = static_cast<uint4 *>(launch.query_output);
    args.key_pages = static_cast<uint4 *>(launch.key_pages);
    args.value_pages = static_cast<uint4 *>(launch.value_pages);
    args.tokens = launch.tokens;
    args.batch = launch.batch;
    args.max_pages = launch.max_pages;
    args.qh = launch.qh;
    args.kvh = launch.kvh;
    args.indices_len = launch.indices_len;
    args.indices_min = launch.indices_min;
    args.hash_slots = launch.hash_slots;
    args.status = launch.status;
    args.workspace_numel = launch.workspace_numel;
    return args;
}

int launch_rope_append(const AppendLaunch &launch, void *stream) {
    return launch_dependent(rope_append_kernel, launch.grid, launch.block, launch.shared_bytes,
                            stream, append_args(launch));
}

int append_workspace_numel(size_t tokens) { return (int)(kVerdictSlots + 2 * tokens); }

int launch_append_validate(const AppendLaunch &launch, void *stream) {
    return launch_dependent(append_validate_kernel, launch.validate_grid, kValidateThreads,
                            launch.shared_bytes, stream, append_args(launch), launch.workspace);
}

int append_fused_ctas_per_sm(int *ctas, size_t shared_bytes) {
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(ctas, append_fused_kernel,
                                                         kScatterThreads, shared_bytes);
}

int launch_append_fused(const AppendLaunch &launch, void *stream) {
    return launch_dependent(append_fused_kernel, launch.grid, kScatterThreads, launch.shared_bytes,
                            stream, append_args(launch), launch.workspace, launch.words,
                            (int)launch.validate_grid);
}

int launch_append_scatter(const AppendLaunch &launch, void *stream) {
    return launch_dependent(append_scatter_kernel, (unsigned)launch.tokens, kScatterThreads, 0,
                            stream, append_args(launch),
                            static_cast<const int32_t *>(launch.workspace));
}

} // namespace lb
