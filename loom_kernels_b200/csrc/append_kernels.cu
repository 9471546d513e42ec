// Fused NeoX RoPE (theta 10000, D128) + paged KV append for sm_100a.
//
// Replaces the reference's rope_paged_kv_append_bf16_neox_d128 and
// rope_paged_kv_append_tokens_bf16_neox_d128 kernels
// (crates/loom-infer-cuda/src/rope/mod.rs:119-230,259-405).  One kernel serves the
// one-token-per-request contract, the explicit <=64-token contract and the extended
// any-total variant:
//
//   1. every CTA validates the whole call against device-resident metadata (page table, token
//      mapping, physical-slot uniqueness via a shared-memory hash set) and returns without
//      writing when anything is invalid, so a call is all-or-nothing exactly like the
//      reference's guards (rope/mod.rs:140-182,290-343);
//   2. a CTA then walks its tokens: 64 threads compute the token's sin/cos table once, and
//      8 lanes per head row rotate Q and K with 16-byte loads/stores (a rotation pair
//      (i, i+64) lives in one thread), scatter K and copy V rows to the token's page slot.
//
// Angles use the host-computed inverse frequencies powf(10000, -2i/128) (constant memory), so
// they are bit-identical to the CPU reference (crates/loom-infer/src/rope/mod.rs:148-150);
// the rotation is evaluated without FMA contraction like the reference (:154-155).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.hpp"

namespace lb {
namespace {

constexpr int kHeadDim = 128;
constexpr int kPairs = 64;
constexpr int kPage = 16;
constexpr int kThreads = 256;

__constant__ float c_inverse_frequency[kPairs];

struct AppendArgs {
    const uint4 *query, *key, *value;
    const int32_t *batch_indices, *positions, *indptr, *indices, *last;
    uint4 *query_output, *key_pages, *value_pages;
    int32_t tokens, batch, max_pages, qh, kvh, indices_len, hash_slots;
};

// (request, position) of a token; one-token-per-request plans derive both from the page table.
__device__ __forceinline__ bool token_slot(const AppendArgs &a, int token, int &position,
                                           int &slot) {
    int request, pos;
    if (a.batch_indices) {
        request = a.batch_indices[token];
        pos = a.positions[token];
        if (request < 0 || request >= a.batch || pos < 0) return false;
    } else {
        request = token;
        pos = -1;
    }
    const int start = a.indptr[request];
    const int pages = a.indptr[request + 1] - start;
    const int kv_len = (pages - 1) * kPage + a.last[request];
    if (pos < 0) pos = kv_len - 1;
    if (pos >= kv_len) return false;
    position = pos;
    slot = a.indices[start + pos / kPage] * kPage + pos % kPage;
    return true;
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

__device__ __forceinline__ void rotate_row(const uint4 *src, uint4 *dst, int j,
                                           const float2 *sincos) {
    // lane j of 8 owns dims [8j, 8j+8) and [64+8j, 64+8j+8) of the 128-wide row
    const uint4 lo = src[j], hi = src[8 + j];
    const float2 *sc = sincos + 8 * j;
    uint4 out_lo, out_hi;
    out_lo.x = rotate_pack(lo.x, hi.x, sc[0], sc[1], out_hi.x);
    out_lo.y = rotate_pack(lo.y, hi.y, sc[2], sc[3], out_hi.y);
    out_lo.z = rotate_pack(lo.z, hi.z, sc[4], sc[5], out_hi.z);
    out_lo.w = rotate_pack(lo.w, hi.w, sc[6], sc[7], out_hi.w);
    dst[j] = out_lo;
    dst[8 + j] = out_hi;
}

__global__ void __launch_bounds__(kThreads) rope_append_kernel(const AppendArgs a) {
    extern __shared__ int hash_table[];
    __shared__ float2 sincos_table[kPairs]; // (sin, cos) per rotation pair of the current token
    const int tid = threadIdx.x;

    // ---- 1. whole-call validation (identical in every CTA) -----------------------------------
    for (int i = tid; i < a.hash_slots; i += kThreads) hash_table[i] = -1;
    bool invalid = false;
    if (tid == 0) {
        const int final_indptr = a.indptr[a.batch];
        invalid = a.indptr[0] != 0 || final_indptr < 0 || final_indptr != a.indices_len;
    }
    for (int request = tid; request < a.batch; request += kThreads) {
        const int start = a.indptr[request], end = a.indptr[request + 1], tail = a.last[request];
        if (start < 0 || end <= start || end > a.indices_len || tail < 1 || tail > kPage)
            invalid = true;
    }
    for (int page = tid; page < a.indices_len; page += kThreads) {
        const int id = a.indices[page];
        if (id < 0 || id >= a.max_pages) invalid = true;
    }
    if (__syncthreads_or(invalid)) return;

    for (int token = tid; token < a.tokens; token += kThreads) {
        int position, slot;
        if (!token_slot(a, token, position, slot)) {
            invalid = true;
            continue;
        }
        // open-addressing insert; meeting the same key means two tokens share a physical slot
        unsigned h = ((unsigned)slot * 2654435761u) & (unsigned)(a.hash_slots - 1);
        for (int probe = 0; probe < a.hash_slots; ++probe) {
            const int seen = atomicCAS(&hash_table[h], -1, slot);
            if (seen == -1) break;
            if (seen == slot) {
                invalid = true;
                break;
            }
            h = (h + 1) & (unsigned)(a.hash_slots - 1);
        }
    }
    if (__syncthreads_or(invalid)) return;

    // ---- 2. rotate + scatter -------------------------------------------------------------------
    const int heads = a.qh + a.kvh;
    const int row_tasks = heads * 8;   // 8 lanes per 128-wide row
    const int copy_tasks = a.kvh * 16; // V rows: 16 x 16-byte chunks
    for (int token = blockIdx.x; token < a.tokens; token += gridDim.x) {
        int position = 0, slot = 0;
        token_slot(a, token, position, slot);
        __syncthreads(); // the previous token's table is no longer read
        if (tid < kPairs) {
            // The F32 angle is exactly the reference's; sin/cos are evaluated in double and
            // rounded once, which reproduces the host libm's (near correctly rounded) sinf/cosf.
            const float angle = __fmul_rn((float)position, c_inverse_frequency[tid]);
            double s, c;
            sincos((double)angle, &s, &c);
            sincos_table[tid] = make_float2((float)s, (float)c);
        }
        __syncthreads();
        for (int task = tid; task < row_tasks; task += kThreads) {
            const int row = task >> 3, j = task & 7;
            if (row < a.qh) {
                const size_t offset = ((size_t)token * a.qh + row) * (kHeadDim / 8);
                rotate_row(a.query + offset, a.query_output + offset, j, sincos_table);
            } else {
                const int kv_head = row - a.qh;
                const size_t src = ((size_t)token * a.kvh + kv_head) * (kHeadDim / 8);
                const size_t dst = ((size_t)slot * a.kvh + kv_head) * (kHeadDim / 8);
                rotate_row(a.key + src, a.key_pages + dst, j, sincos_table);
            }
        }
        for (int task = tid; task < copy_tasks; task += kThreads) {
            const int kv_head = task >> 4, c = task & 15;
            a.value_pages[((size_t)slot * a.kvh + kv_head) * 16 + c] =
                a.value[((size_t)token * a.kvh + kv_head) * 16 + c];
        }
    }
}

} // namespace

int configure_append_kernels(size_t max_dynamic_shared, const float *inverse_frequency) {
    int rc = cudaMemcpyToSymbol(c_inverse_frequency, inverse_frequency, sizeof(float) * kPairs);
    if (rc) return rc;
    return cudaFuncSetAttribute(rope_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)max_dynamic_shared);
}

int launch_rope_append(const AppendLaunch &launch, void *stream) {
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
    args.hash_slots = launch.hash_slots;
    rope_append_kernel<<<launch.grid, launch.block, launch.shared_bytes,
                         static_cast<cudaStream_t>(stream)>>>(args);
    return cudaGetLastError();
}

} // namespace lb
