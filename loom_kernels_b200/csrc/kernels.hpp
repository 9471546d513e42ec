// Launch descriptors shared between the providers (host) and the kernel translation units.
#pragma once

#include <cstddef>
#include <cstdint>

#include "loom_b200.h"

namespace lb {

// Where finished rows go when a plan gathers its output over the ranks of a peer group: row r of
// the local batch, local query head h is row dest_rows[r] * gathered_qh + head_offset + h of the
// gathered [rows, 128] BF16 output and F32 LSE, in every rank's copy.  world == 0: no gather.
struct PeerOut {
    void *const *out;         // device array [world]: every rank's copy of the gathered O
    float *const *lse;        // device array [world]: every rank's copy of the gathered LSE
    const int32_t *dest_rows; // [batch]
    int32_t world, gathered_qh, head_offset;
};

// A rank's signal block is an array of 32-bit words in peer-mapped memory: word 0 counts finished
// CTAs, word 1 is the epoch, and the flags the other ranks write start at this word.
constexpr int kPeerFlagsWord = 32;

// What the last kernel of a gathering command needs to publish its epoch to every rank and to
// wait for theirs.  world == 0: nothing to signal.
struct PeerSignal {
    uint32_t *done;         // this GPU: CTAs of the running kernel that have finished
    uint32_t *epoch;        // this GPU: epochs published so far
    uint32_t *const *flags; // device array [world]: every rank's signal block (flags at word
                            // kPeerFlagsWord, one per sender)
    int32_t *status;        // set to 2 when the wait for the other ranks ran out
    int32_t rank, world;
    int32_t defer;          // 1: store the rows only; a later command of the step publishes the epoch
    long long wait_cycles;
};

// One paged-decode launch.  Every pointer is a device pointer of the queue's device.
struct DecodeLaunch {
    alignas(64) unsigned char k_map[128]; // CUtensorMap over K pages, see decode_kernels.cu
    alignas(64) unsigned char v_map[128]; // CUtensorMap over V pages
    const void *query;       // bf16 [batch, qh, 128]
    const int32_t *indptr;   // [batch + 1]
    const int32_t *indices;  // [indices_len]
    const int32_t *last;     // [batch]
    void *output;            // bf16 [batch, qh, 128]
    float *lse;              // [batch, qh]
    float *workspace;        // [batch, qh, partitions, 130] when partitions > 1
    int32_t *status;         // optional device status word (0 = ok)
    int32_t batch, max_pages, qh, kvh, indices_len;
    int32_t indices_min; // page_indptr[batch] must lie in [indices_min, indices_len]
    int32_t heads_per_cta, pages_per_stage, q_tiles, q_blocks, partitions, stages;
    int32_t cluster;        // 1: the chunks of an item are one thread-block cluster (one command)
    float scale_log2;
    uint32_t grid, block, shared_bytes;
    long long wait_cycles;  // limit of every bounded wait of the kernel, in SM clock cycles
    long long workspace_numel; // F32 elements bound as the workspace (the checked build's bound)
    int32_t test_skip_page; // tests of the give-up path: 1 + the page of a CTA's chunk whose
                            // bytes never all arrive (0 = none)
    int32_t producer_warps; // balanced plans: 1, or one per page slot
    int32_t merge_four_warps; // balanced plans: the merge gives every row a CTA of four warps
    int32_t *counters;      // one zeroed word per item when the split is merged in the kernel
    PeerOut peer;           // zeroed unless the plan gathers its output
    PeerSignal signal;      // zeroed unless this launch is the last kernel of a gathering command
};

struct MergeLaunch {
    const float *workspace;
    void *output;
    float *lse;
    const int32_t *indptr;
    const int32_t *last;
    int32_t batch, qh, partitions, indices_len, indices_min;
    uint32_t grid, block;
    PeerOut peer;
    PeerSignal signal;
    long long workspace_numel; // F32 elements of `workspace` (the checked build's bound)
    int32_t *status;           // optional device status word
};

// One fused RoPE + paged append launch.
struct AppendLaunch {
    const void *query, *key, *value;          // bf16 [tokens, qh|kvh, 128]
    const int32_t *batch_indices, *positions; // [tokens]; null for one-token-per-request
    const int32_t *indptr, *indices, *last;
    void *query_output, *key_pages, *value_pages;
    int32_t tokens, batch, max_pages, qh, kvh, indices_len, indices_min;
    int32_t hash_slots; // power of two >= 2 * tokens
    uint32_t grid, block, shared_bytes;
    // two-command (extended) plans only: I32 workspace of append_workspace_numel(tokens) and
    // the CTAs of the validation kernel (1, or 1 token CTA + page-table scanners)
    int32_t *workspace;
    uint32_t validate_grid;
    int32_t workspace_numel; // I32 elements of `workspace` (the checked build's bound)
    int32_t *status;         // optional device status word (the checked build; a wait that ran out)
    int32_t *words;          // one-command extended plans: the queue's synchronisation words
};

// Each returns a CUDA error code (0 = success).
int configure_decode_kernels(size_t max_dynamic_shared);
int configure_stream_kernels(size_t max_dynamic_shared);
// Balanced algorithm: launch.grid CTAs, launch.grid * pages_per_stage workers; launch.workspace
// holds [workers][2][heads_per_cta * min(group, 16 * q_tiles)][130] floats, then batch + 1 ints.
int launch_balanced_decode(const DecodeLaunch &launch, void *stream);
int launch_balanced_merge(const DecodeLaunch &launch, uint32_t grid, uint32_t block, void *stream);
long long default_wait_cycles(); // ~2 s of SM clock
int launch_paged_decode(const DecodeLaunch &launch, void *stream);
int launch_split_merge(const MergeLaunch &launch, void *stream);
int configure_append_kernels(size_t max_dynamic_shared, const float *inverse_frequency);
int launch_rope_append(const AppendLaunch &launch, void *stream);
int append_workspace_numel(size_t tokens);
int launch_append_validate(const AppendLaunch &launch, void *stream);
int launch_append_scatter(const AppendLaunch &launch, void *stream);
// One-command form: launch.grid = launch.validate_grid validators + token CTAs, all resident at once.
int launch_append_fused(const AppendLaunch &launch, void *stream);
int append_fused_ctas_per_sm(int *ctas, size_t shared_bytes); // occupancy of that kernel
// One stand-alone RoPE launch over contiguous NHD Q and K.
struct RopeLaunch {
    const void *query, *key;   // bf16 [tokens, heads, 128]
    const int32_t *position_ids;
    void *query_output, *key_output;
    int32_t tokens, qh, kh;
    float inverse_frequency[64];
    uint32_t grid;
};
int launch_rope_pos_ids(const RopeLaunch &launch, void *stream);
// One paged causal prefill launch.
struct PrefillLaunch {
    alignas(64) unsigned char k_map[128]; // CUtensorMap over K pages, box = one page of one KV head
    alignas(64) unsigned char v_map[128];
    const void *query;          // bf16 [nnz_qo, qh, 128]
    const int32_t *qo_indptr;   // [batch + 1]
    const int32_t *indptr;      // [batch + 1]
    const int32_t *indices;     // [indices_len]
    const int32_t *last;        // [batch]
    void *output;               // bf16 [nnz_qo, qh, 128]
    float *lse;                 // [nnz_qo, qh]
    int32_t *status;
    int32_t batch, nnz_qo, max_pages, qh, kvh, indices_len, indices_min;
    int32_t q_tiles, pages_per_stage, stages, tiles;
    float scale_log2;
    uint32_t grid, block, shared_bytes;
    // tiled plans that cut a tile's KV range into chunks: F32 states [nnz_qo * qh][partitions][130]
    float *workspace;
    int32_t partitions;
    int32_t min_chunk_blocks; // a tile uses min(partitions, its blocks / min_chunk_blocks) chunks
    long long wait_cycles;    // tiled kernel: limit of its bounded waits (0 = the default)
    int32_t test_lost_copy;   // tiled kernel, tests of the give-up path only
};
int configure_prefill_kernels(size_t max_dynamic_shared);
int launch_paged_prefill(const PrefillLaunch &launch, void *stream);
// The tcgen05 kernel: 128-row tiles; launch.k_map must have the box {64 dims, 16 tokens, 1 half}
// (the K rows of a block form one uniform operand), launch.v_map the box {64, 16, 2}.
int configure_prefill_tiled_kernel(size_t max_dynamic_shared);
int prefill_tiled_shared_bytes();
int launch_paged_prefill_tiled(const PrefillLaunch &launch, void *stream);
int launch_prefill_merge(const PrefillLaunch &launch, void *stream); // second command of a split plan
int append_block_threads();       // threads per CTA the append kernel is built for
int append_max_tokens_per_cta();  // tokens one CTA can own (grid floor = tokens / this)

} // namespace lb
