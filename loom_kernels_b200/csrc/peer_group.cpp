// Output rows across the GPUs of one node: the ranks of a job (one process per GPU), device memory
// every rank can store into, and the all-gather of output rows as a command of the scope.
//
// The reference is a single-GPU operator layer (crates/loom-infer-cuda/src/command/binding.rs:
// 109-123 rejects buffers of another device).  Paged decode shards by request (or by KV head) with
// no exchange step; what crosses GPUs is only the finished output rows, when the caller wants one
// contiguous result.  Two ways to get it, both under the scope's one completion fence:
//
//   * lb_output_gather_enqueue: the communication library's all-gather (NCCL) enqueued on the
//     queue's own stream and recorded the way the reference records a vendor-library call
//     (record_external_submission, crates/loom-infer-cuda/src/command/submission.rs:240-272):
//     one command, counted by submitted(), capturable; a failure poisons scope and queue.
//   * lb_paged_decode_enqueue_gathered: no collective kernel at all.  The decode (or merge)
//     kernel stores every finished row straight into every rank's copy of a peer buffer and its
//     last CTA publishes an epoch and waits for the other ranks' (decode_device.cuh).
//
// NCCL is resolved with dlopen at first use, so a single-GPU host never loads it.  Peer buffers
// are plain cudaMalloc allocations shared through CUDA IPC handles, which the ranks exchange over
// the group's own communicator.  Only plain stores cross GPUs: no TMA load and no multicast load
// ever reads a peer's memory.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "kernels.hpp"
#include "peer_group.hpp"
#include "runtime.hpp"

using namespace lb;

namespace {

// ---- the communication library, by name --------------------------------------------------------

typedef struct ncclComm *ncclComm_t;
struct NcclUniqueId {
    char internal[128];
};
enum { kNcclUint8 = 1, kNcclInt32 = 2, kNcclFloat16 = 6, kNcclFloat32 = 7, kNcclBfloat16 = 9 };

struct NcclApi {
    int (*GetUniqueId)(NcclUniqueId *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Broadcast)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    bool loaded = false;
};

NcclApi g_nccl;
std::mutex g_nccl_mutex;

lb_status load_nccl() {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.loaded) return LB_OK;
    void *handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!handle) handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!handle) return fail(LB_EXTERNAL_COMMAND, "nccl: library not found", -1);
    auto resolve = [&](const char *name) { return dlsym(handle, name); };
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))resolve("ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))resolve("ncclCommInitRank");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))resolve("ncclCommDestroy");
    g_nccl.CommAbort = (decltype(g_nccl.CommAbort))resolve("ncclCommAbort");
    g_nccl.AllGather = (decltype(g_nccl.AllGather))resolve("ncclAllGather");
    g_nccl.Broadcast = (decltype(g_nccl.Broadcast))resolve("ncclBroadcast");
    g_nccl.GroupStart = (decltype(g_nccl.GroupStart))resolve("ncclGroupStart");
    g_nccl.GroupEnd = (decltype(g_nccl.GroupEnd))resolve("ncclGroupEnd");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.CommDestroy || !g_nccl.AllGather ||
        !g_nccl.Broadcast || !g_nccl.GroupStart || !g_nccl.GroupEnd)
        return fail(LB_EXTERNAL_COMMAND, "nccl: symbol missing", -2);
    g_nccl.loaded = true;
    return LB_OK;
}

int nccl_dtype(int dtype) {
    switch (dtype) {
    case LB_F32: return kNcclFloat32;
    case LB_F16: return kNcclFloat16;
    case LB_BF16: return kNcclBfloat16;
    case LB_I32: return kNcclInt32;
    default: return kNcclUint8;
    }
}

size_t dtype_bytes(int dtype) {
    switch (dtype) {
    case LB_F32: case LB_I32: return 4;
    case LB_F16: case LB_BF16: return 2;
    default: return 1;
    }
}

constexpr size_t kExchangeBytes = 128; // one rank's record in a handle exchange
constexpr size_t kSignalWords = 256;   // [done, epoch, status, ..., flags at word 32]
static_assert(kPeerFlagsWord + LB_PEER_MAX_RANKS <= (int)kSignalWords, "signal block size");

struct DeviceScope { // binds the group's device for the calling thread
    int previous = -1;
    bool changed = false;
    explicit DeviceScope(int device) {
        if (cudaGetDevice(&previous) == cudaSuccess && previous != device)
            changed = cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceScope() {
        if (changed) cudaSetDevice(previous);
    }
};

} // namespace

struct lb_peer_buffer {
    lb_peer_group *group = nullptr;
    size_t bytes = 0;
    void *local = nullptr;
    std::vector<void *> address; // [world] address, in this process, of every rank's copy
    void **table = nullptr;      // the same, as a device array the kernels read
};

struct lb_peer_group {
    int device = 0, rank = 0, world = 1;
    bool fake = false;
    ncclComm_t comm = nullptr;
    cudaStream_t stream = nullptr; // set-up traffic only (handle exchanges)
    uint8_t *exchange = nullptr;   // device: (1 + world) records of kExchangeBytes
    lb_peer_buffer *signal = nullptr;
    int clock_khz = 0;
};

namespace {

// Every rank contributes kExchangeBytes; all[r] receives rank r's.  Collective.
lb_status exchange_records(lb_peer_group *g, const void *mine, std::vector<uint8_t> &all) {
    all.assign((size_t)g->world * kExchangeBytes, 0);
    int rc = cudaMemcpy(g->exchange, mine, kExchangeBytes, cudaMemcpyHostToDevice);
    if (rc) return fail(LB_DRIVER, "peer exchange", rc);
    const int nccl = g_nccl.AllGather(g->exchange, g->exchange + kExchangeBytes, kExchangeBytes,
                                      kNcclUint8, g->comm, g->stream);
    if (nccl) return fail(LB_EXTERNAL_COMMAND, "nccl", nccl);
    if ((rc = cudaStreamSynchronize(g->stream))) return fail(LB_DRIVER, "peer exchange", rc);
    if ((rc = cudaMemcpy(all.data(), g->exchange + kExchangeBytes, all.size(),
                         cudaMemcpyDeviceToHost)))
        return fail(LB_DRIVER, "peer exchange", rc);
    return LB_OK;
}

lb_status create_buffer(lb_peer_group *g, size_t bytes, lb_peer_buffer **out) {
    lb_peer_buffer *b = new lb_peer_buffer();
    b->group = g;
    b->bytes = bytes;
    b->address.assign((size_t)g->world, nullptr);
    if (g->fake) { // host-only tests: addresses that the fake driver takes for device memory
        static uintptr_t next = 0x50000000;
        b->local = (void *)next;
        next += (bytes + 0xfffff) & ~(uintptr_t)0xfffff;
        for (int r = 0; r < g->world; ++r) b->address[r] = b->local;
        *out = b;
        return LB_OK;
    }
    DeviceScope scope(g->device);
    auto destroy = [&](lb_status status) {
        lb_peer_buffer_destroy(b);
        return status;
    };
    int rc = cudaMalloc(&b->local, bytes);
    if (rc) {
        delete b;
        return fail(LB_DRIVER, "peer buffer", rc);
    }
    b->address[g->rank] = b->local;
    if ((rc = cudaMemset(b->local, 0, bytes)) || (rc = cudaDeviceSynchronize()))
        return destroy(fail(LB_DRIVER, "peer buffer", rc));
    if (g->world > 1) {
        uint8_t mine[kExchangeBytes] = {0};
        cudaIpcMemHandle_t handle;
        static_assert(sizeof(handle) <= kExchangeBytes, "IPC handle size");
        if ((rc = cudaIpcGetMemHandle(&handle, b->local)))
            return destroy(fail(LB_DRIVER, "cudaIpcGetMemHandle", rc));
        memcpy(mine, &handle, sizeof(handle));
        std::vector<uint8_t> all;
        lb_status status = exchange_records(g, mine, all);
        if (status) return destroy(status);
        for (int r = 0; r < g->world; ++r) {
            if (r == g->rank) continue;
            memcpy(&handle, all.data() + (size_t)r * kExchangeBytes, sizeof(handle));
            if ((rc = cudaIpcOpenMemHandle(&b->address[r], handle, cudaIpcMemLazyEnablePeerAccess)))
                return destroy(fail(LB_DRIVER, "cudaIpcOpenMemHandle", rc));
        }
    }
    if ((rc = cudaMalloc((void **)&b->table, (size_t)g->world * sizeof(void *))) ||
        (rc = cudaMemcpy(b->table, b->address.data(), (size_t)g->world * sizeof(void *),
                         cudaMemcpyHostToDevice)))
        return destroy(fail(LB_DRIVER, "peer buffer", rc));
    *out = b;
    return LB_OK;
}

} // namespace

namespace lb {

PeerSignal peer_signal_of(const lb_peer_group *g, long long wait_cycles) {
    PeerSignal s;
    memset(&s, 0, sizeof(s));
    if (!g || !g->signal) return s;
    uint32_t *words = static_cast<uint32_t *>(g->signal->local);
    s.done = words;
    s.epoch = words + 1;
    s.status = reinterpret_cast<int32_t *>(words + 2);
    s.flags = reinterpret_cast<uint32_t *const *>(g->signal->table);
    s.rank = g->rank;
    s.world = g->world;
    s.wait_cycles = wait_cycles;
    return s;
}

void *const *peer_buffer_table(const lb_peer_buffer *b) { return b ? b->table : nullptr; }
int peer_group_device(const lb_peer_group *g) { return g->device; }
int peer_group_clock_khz(const lb_peer_group *g) { return g->clock_khz; }

} // namespace lb

extern "C" {

lb_status lb_peer_group_unique_id(uint8_t *id) {
    if (!id) return fail(LB_INVALID_ARGUMENT, "id");
    memset(id, 0, LB_PEER_ID_BYTES);
    if (driver().is_fake()) return LB_OK;
    lb_status status = load_nccl();
    if (status) return status;
    NcclUniqueId unique;
    static_assert(sizeof(unique) == LB_PEER_ID_BYTES, "unique id size");
    const int nccl = g_nccl.GetUniqueId(&unique);
    if (nccl) return fail(LB_EXTERNAL_COMMAND, "nccl", nccl);
    memcpy(id, &unique, sizeof(unique));
    return LB_OK;
}

lb_status lb_peer_group_create(int device, int world, int rank, const uint8_t *id,
                               lb_peer_group **out) {
    if (!out || !id) return fail(LB_INVALID_ARGUMENT, "out");
    *out = nullptr;
    if (world < 1 || world > LB_PEER_MAX_RANKS || rank < 0 || rank >= world)
        return fail(LB_INVALID_ARGUMENT, "rank", rank, world);
    lb_peer_group *g = new lb_peer_group();
    g->device = device;
    g->world = world;
    g->rank = rank;
    g->fake = driver().is_fake();
    driver().device_clock_khz(device, &g->clock_khz);
    lb_status status = LB_OK;
    if (!g->fake) {
        if ((status = load_nccl())) {
            delete g;
            return status;
        }
        DeviceScope scope(device);
        NcclUniqueId unique;
        memcpy(&unique, id, sizeof(unique));
        int rc = cudaStreamCreateWithFlags(&g->stream, cudaStreamNonBlocking);
        if (!rc) rc = cudaMalloc((void **)&g->exchange, (size_t)(1 + world) * kExchangeBytes);
        if (rc) {
            lb_peer_group_destroy(g);
            return fail(LB_DRIVER, "peer group", rc);
        }
        const int nccl = g_nccl.CommInitRank(&g->comm, world, unique, rank);
        if (nccl) {
            g->comm = nullptr;
            lb_peer_group_destroy(g);
            return fail(LB_EXTERNAL_COMMAND, "nccl", nccl);
        }
    }
    if ((status = create_buffer(g, kSignalWords * sizeof(uint32_t), &g->signal))) {
        g->signal = nullptr;
        lb_peer_group_destroy(g);
        return status;
    }
    *out = g;
    return LB_OK;
}

void lb_peer_group_destroy(lb_peer_group *g) {
    if (!g) return;
    if (g->signal) lb_peer_buffer_destroy(g->signal);
    if (!g->fake) {
        DeviceScope scope(g->device);
        if (g->comm) g_nccl.CommDestroy(g->comm);
        if (g->exchange) cudaFree(g->exchange);
        if (g->stream) cudaStreamDestroy(g->stream);
    }
    delete g;
}

int lb_peer_group_rank(const lb_peer_group *g) { return g ? g->rank : -1; }
int lb_peer_group_world(const lb_peer_group *g) { return g ? g->world : 0; }

lb_status lb_peer_buffer_create(lb_peer_group *g, size_t bytes, lb_peer_buffer **out) {
    if (!g || !out) return fail(LB_INVALID_ARGUMENT, "group");
    *out = nullptr;
    if (bytes == 0) return fail(LB_ZERO_DIMENSION);
    return create_buffer(g, bytes, out);
}

void lb_peer_buffer_destroy(lb_peer_buffer *b) {
    if (!b) return;
    if (!b->group->fake) {
        DeviceScope scope(b->group->device);
        for (int r = 0; r < (int)b->address.size(); ++r)
            if (r != b->group->rank && b->address[r]) cudaIpcCloseMemHandle(b->address[r]);
        if (b->table) cudaFree(b->table);
        if (b->local) cudaFree(b->local);
    }
    delete b;
}

void *lb_peer_buffer_local(const lb_peer_buffer *b) { return b ? b->local : nullptr; }
size_t lb_peer_buffer_bytes(const lb_peer_buffer *b) { return b ? b->bytes : 0; }

// ---- the all-gather of output rows as a command ----------------------------------------------------

struct lb_output_gather_plan {
    const lb_peer_group *group = nullptr;
    int dtype = LB_BF16;
    size_t row_numel = 0, total_rows = 0;
    std::vector<size_t> rows; // per rank
    bool equal = true;
};

lb_status lb_output_gather_plan_create(const lb_peer_group *g, int dtype,
                                       const size_t *rows_per_rank, size_t row_numel,
                                       lb_output_gather_plan **out) {
    if (!g || !rows_per_rank || !out) return fail(LB_INVALID_ARGUMENT, "group");
    *out = nullptr;
    if (dtype < LB_F32 || dtype > LB_U8) return fail(LB_UNSUPPORTED_DTYPE, nullptr, dtype);
    if (row_numel == 0) return fail(LB_ZERO_DIMENSION);
    lb_output_gather_plan *plan = new lb_output_gather_plan();
    plan->group = g;
    plan->dtype = dtype;
    plan->row_numel = row_numel;
    for (int r = 0; r < g->world; ++r) {
        size_t numel;
        if (__builtin_mul_overflow(rows_per_rank[r], row_numel, &numel) ||
            __builtin_add_overflow(plan->total_rows, rows_per_rank[r], &plan->total_rows)) {
            delete plan;
            return fail(LB_ELEMENT_COUNT_OVERFLOW);
        }
        plan->rows.push_back(rows_per_rank[r]);
        plan->equal &= rows_per_rank[r] == rows_per_rank[0];
    }
    size_t total;
    if (plan->total_rows == 0 || __builtin_mul_overflow(plan->total_rows, row_numel, &total)) {
        const bool empty = plan->total_rows == 0;
        delete plan;
        return fail(empty ? LB_ZERO_DIMENSION : LB_ELEMENT_COUNT_OVERFLOW);
    }
    *out = plan;
    return LB_OK;
}

void lb_output_gather_plan_destroy(lb_output_gather_plan *plan) { delete plan; }

lb_status lb_output_gather_enqueue(const lb_output_gather_plan *plan, lb_scope *scope,
                                   const lb_output_gather_args *args) {
    if (!plan || !scope || !args) return fail(LB_INVALID_ARGUMENT, "plan");
    const lb_peer_group *g = plan->group;
    if (scope->queue->device != g->device)
        return fail(LB_BUFFER_CONTEXT_MISMATCH, nullptr, g->device, scope->queue->device);
    lb_status rc = require_command_capacity(*scope, 1);
    if (rc) return rc;
    OperandRequest requests[2] = {{args->local, (uint8_t)plan->dtype, false},
                                  {args->gathered, (uint8_t)plan->dtype, true}};
    Operand op[2];
    if ((rc = resolve(*scope, requests, 2, op))) return rc;
    const size_t mine = plan->rows[(size_t)g->rank] * plan->row_numel;
    if (op[0].numel != mine)
        return fail(LB_ENQUEUE_LENGTH_MISMATCH, "local", (int64_t)mine, (int64_t)op[0].numel);
    if (op[1].numel != plan->total_rows * plan->row_numel)
        return fail(LB_ENQUEUE_LENGTH_MISMATCH, "gathered",
                    (int64_t)(plan->total_rows * plan->row_numel), (int64_t)op[1].numel);
    cudaStream_t stream = static_cast<cudaStream_t>(scope->queue->stream);
    const int type = nccl_dtype(plan->dtype);
    const size_t scale = type == kNcclUint8 ? dtype_bytes(plan->dtype) : 1; // bytes when untyped
    return submit_external(*scope, "nccl", [&]() -> int {
        if (plan->equal)
            return g_nccl.AllGather(op[0].ptr, op[1].ptr, mine * scale, type, g->comm, stream);
        // unequal counts: one broadcast per rank, fused into one launch by the group call
        int error = g_nccl.GroupStart();
        if (error) return error;
        uint8_t *cursor = static_cast<uint8_t *>(op[1].ptr);
        for (int r = 0; r < g->world && !error; ++r) {
            const size_t numel = plan->rows[(size_t)r] * plan->row_numel;
            if (numel)
                error = g_nccl.Broadcast(r == g->rank ? op[0].ptr : cursor, cursor, numel * scale,
                                         type, r, g->comm, stream);
            cursor += numel * dtype_bytes(plan->dtype);
        }
        const int end = g_nccl.GroupEnd();
        return error ? error : end;
    });
}

}
