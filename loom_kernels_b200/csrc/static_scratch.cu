// Split-K paged decode for callers that cannot allocate device memory.
//
// The regular split-K plan needs a caller-owned F32 workspace for its partial states.  Some hosts
// have no way to produce one: a plug-in that is handed device pointers by its engine but is
// forbidden to call cudaMalloc itself (the engine gave all device memory to its own pool at
// start-up), or a latency-critical loop that must never enter the allocator.  For them this file
// keeps the states in a fixed array that lives inside the library image on every GPU that loads
// it, and exposes one entry point that uses it.  Nothing here calls cudaMalloc, cudaFree or any
// routine that allocates.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "kernels.hpp"
#include "runtime.hpp"

namespace {

// 16 384 states of 130 floats = 8 519 680 bytes, held by every GPU that loads the library until
// the process exits.  Enough for batch 8 x 64 query heads x 16 partitions with room to spare.
constexpr size_t kMaxStates = 16384;
constexpr size_t kScratchFloats = kMaxStates * LB_PARTIAL_STATE_WIDTH;
static __device__ __align__(256) float g_split_scratch[kScratchFloats];
// Set to 1 by a CTA of this entry point's kernels that gave up on a bounded wait (its rows are then
// missing from the result); read and cleared by lb_paged_decode_split_noalloc_status.
static __device__ int32_t g_split_status;

constexpr int kMaxDevices = 64;
struct DeviceSetup {
    bool ready = false;       // set only by a set-up on a real device, never under the fake driver
    float *scratch = nullptr; // device address of g_split_scratch on this GPU
    int32_t *status = nullptr; // device address of g_split_status on this GPU
    int sm_count = 0;
    size_t smem_optin = 0;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex; // the one-time set-up of a GPU may be raced by two host threads

// In host code `g_split_scratch` names a host-side stand-in, not device memory: the device
// address has to be asked for, once per GPU, with that GPU current.
int set_up_device(int device, DeviceSetup &setup) {
    int previous = -1;
    int rc = cudaGetDevice(&previous);
    if (rc) return rc;
    if (previous != device && (rc = cudaSetDevice(device))) return rc;
    void *address = nullptr, *status = nullptr;
    rc = cudaGetSymbolAddress(&address, g_split_scratch);
    if (!rc) rc = cudaGetSymbolAddress(&status, g_split_status);
    if (!rc) rc = lb::configure_decode_kernels(setup.smem_optin);
    if (previous != device) cudaSetDevice(previous);
    if (rc) return rc;
    if (address == nullptr || status == nullptr) return (int)cudaErrorInvalidSymbol;
    setup.scratch = static_cast<float *>(address);
    setup.status = static_cast<int32_t *>(status);
    setup.ready = true;
    return 0;
}

} // namespace

extern "C" {

size_t lb_paged_decode_split_noalloc_max_states(void) { return kMaxStates; }

lb_status lb_paged_decode_split_noalloc(const lb_paged_spec *spec, uint32_t partitions,
                                        void *stream, const void *query, const void *key_pages,
                                        const void *value_pages, const int32_t *page_indptr,
                                        const int32_t *page_indices, size_t page_indices_len,
                                        const int32_t *last_page_len, void *output, float *lse) {
    using namespace lb;
    if (!spec || !query || !key_pages || !value_pages || !page_indptr || !page_indices ||
        !last_page_len || !output || !lse)
        return fail(LB_INVALID_ARGUMENT, "null pointer");
    if (partitions < 2)
        return fail(LB_INVALID_PARTITION_COUNT, nullptr, partitions, (int64_t)spec->max_num_pages);
    lb_paged_spec checked;
    lb_status rc = lb_paged_spec_new(spec->batch_size, spec->max_num_pages, spec->num_query_heads,
                                     spec->num_kv_heads, LB_HEAD_DIM, LB_PAGE_SIZE, &checked);
    if (rc) return rc;
    if (page_indices_len < checked.batch_size)
        return fail(LB_PAGE_INDICES_TOO_SHORT, nullptr, (int64_t)checked.batch_size,
                    (int64_t)page_indices_len);
    if (page_indices_len > 0x7fffffffu || checked.max_num_pages > (size_t)0x7fffffff / LB_PAGE_SIZE ||
        checked.num_kv_heads > 0x7fffffffu / LB_HEAD_DIM)
        return fail(LB_STATE_COUNT_OUT_OF_RANGE, nullptr, (int64_t)page_indices_len);

    int device = 0;
    int error = driver().stream_device(stream, &device);
    if (error) return fail(LB_DRIVER, "stream_device", error);
    if (device < 0 || device >= kMaxDevices) return fail(LB_INVALID_ARGUMENT, "device", device);
    // Under the fake driver (host-only tests) nothing is cached: there is no device and no
    // address, and a later call on the real driver must still do its set-up.
    DeviceSetup fake_setup;
    const bool fake = driver().is_fake();
    DeviceSetup &setup = fake ? fake_setup : g_setup[device];
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!setup.ready) {
            int major = 0, minor = 0;
            size_t l2 = 0;
            if ((error = driver().device_props(device, &setup.sm_count, &major, &minor,
                                               &setup.smem_optin, &l2)))
                return fail(LB_DRIVER, "device_props", error);
            if (major != 10) return fail(LB_UNSUPPORTED_DEVICE, nullptr, major * 10 + minor);
            if (!fake && (error = set_up_device(device, setup)))
                return fail(LB_DRIVER, "cudaGetSymbolAddress", error);
        }
    }
    if (!fake && (setup.scratch == nullptr || setup.status == nullptr))
        return fail(LB_DRIVER, "static scratch address", (int)cudaErrorInvalidSymbol);
    // every operand must be device memory of the stream's GPU (BufferContextMismatch in the plan
    // path, crates/loom-infer-cuda/src/command/binding.rs:109-123)
    for (const void *p : {query, key_pages, value_pages, (const void *)page_indptr,
                          (const void *)page_indices, (const void *)last_page_len,
                          (const void *)output, (const void *)lse}) {
        int owner = -1;
        bool is_device = false;
        if ((error = driver().pointer_device(p, &owner, &is_device)) || !is_device)
            return fail(LB_INVALID_ARGUMENT, "not a device pointer", error);
        if (owner != device) return fail(LB_BUFFER_CONTEXT_MISMATCH, nullptr, owner, device);
    }

    lb_paged_decode_options options;
    memset(&options, 0, sizeof(options));
    options.partitions = partitions;
    DecodeChoice c;
    if ((rc = choose_decode(checked, (uint32_t)setup.sm_count, setup.smem_optin, &options, &c)))
        return rc;
    if (c.workspace_numel > kScratchFloats)
        return fail(LB_STATIC_SCRATCH_EXCEEDED, nullptr, (int64_t)c.workspace_numel,
                    (int64_t)kScratchFloats);
    for (const void *p : {query, key_pages, value_pages, (const void *)output})
        if ((uintptr_t)p % 16 != 0)
            return fail(LB_MISALIGNED_BUFFER, "operand", (int64_t)(uintptr_t)p, 16);

    DecodeLaunch launch;
    memset(&launch, 0, sizeof(launch));
    const uint64_t dims[3] = {64, (uint64_t)checked.max_num_pages * LB_PAGE_SIZE,
                              (uint64_t)checked.num_kv_heads * 2};
    const uint64_t strides[2] = {(uint64_t)checked.num_kv_heads * LB_HEAD_DIM * 2, 128};
    const uint32_t box[3] = {64, 16, c.heads_per_cta * 2};
    error = driver().encode_tensor_map_3d(device, launch.k_map, key_pages, dims, strides, box);
    if (!error)
        error = driver().encode_tensor_map_3d(device, launch.v_map, value_pages, dims, strides, box);
    if (error) return fail(LB_LAUNCH_CONTRACT, "tensor_map", error);
    launch.query = query;
    launch.indptr = page_indptr;
    launch.indices = page_indices;
    launch.last = last_page_len;
    launch.output = output;
    launch.lse = lse;
    launch.workspace = setup.scratch;
    launch.status = setup.status;
    launch.workspace_numel = (long long)c.workspace_numel;
    launch.batch = (int32_t)checked.batch_size;
    launch.max_pages = (int32_t)checked.max_num_pages;
    launch.qh = (int32_t)checked.num_query_heads;
    launch.kvh = (int32_t)checked.num_kv_heads;
    launch.indices_len = (int32_t)page_indices_len;
    launch.indices_min = launch.indices_len;
    launch.heads_per_cta = (int32_t)c.heads_per_cta;
    launch.pages_per_stage = (int32_t)c.pages_per_stage;
    launch.q_tiles = (int32_t)c.q_tiles;
    launch.q_blocks = (int32_t)c.q_blocks;
    launch.partitions = (int32_t)c.partitions;
    launch.stages = (int32_t)c.stages;
    launch.scale_log2 = checked.softmax_scale * 1.44269504088896340736f;
    launch.grid = c.grid;
    launch.block = c.block;
    launch.shared_bytes = c.shared_bytes;
    if ((error = driver().launch(device, [&]() { return launch_paged_decode(launch, stream); })))
        return fail(LB_DRIVER, "launch", error);
    MergeLaunch merge;
    memset(&merge, 0, sizeof(merge));
    merge.workspace = setup.scratch;
    merge.workspace_numel = (long long)c.workspace_numel;
    merge.status = setup.status;
    merge.output = output;
    merge.lse = lse;
    merge.indptr = page_indptr;
    merge.last = last_page_len;
    merge.batch = launch.batch;
    merge.qh = launch.qh;
    merge.partitions = launch.partitions;
    merge.indices_len = launch.indices_len;
    merge.indices_min = launch.indices_min;
    merge.grid = c.merge_grid;
    merge.block = c.merge_block;
    if ((error = driver().launch(device, [&]() { return launch_split_merge(merge, stream); })))
        return fail(LB_DRIVER, "launch", error);
    return LB_OK;
}

lb_status lb_paged_decode_split_noalloc_status(int device, int32_t *status) {
    using namespace lb;
    if (!status || device < 0 || device >= kMaxDevices) return fail(LB_INVALID_ARGUMENT, "status");
    *status = 0;
    int32_t *word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_setup[device].ready) return LB_OK; // no call has run on this GPU yet
        word = g_setup[device].status;
    }
    if (driver().is_fake()) return LB_OK;
    const int error = driver().configure(device, [&]() -> int {
        int e = cudaMemcpy(status, word, sizeof(int32_t), cudaMemcpyDeviceToHost);
        if (e) return e;
        return cudaMemset(word, 0, sizeof(int32_t));
    });
    if (error) return fail(LB_DRIVER, "noalloc_status", error);
    return LB_OK;
}

int lb_test_noalloc_is_set_up(int device) {
    if (device < 0 || device >= kMaxDevices) return 0;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    return g_setup[device].ready ? 1 : 0;
}

}
