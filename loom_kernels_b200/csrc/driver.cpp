// The CUDA seam: one implementation over the CUDA runtime (the product) and one in-process
// fake for host-only tests of the ownership and poisoning state machine.  The fake never runs
// a kernel and cannot produce results.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>

#include "runtime.hpp"

namespace lb {
namespace {

std::atomic<uint64_t> g_launches{0};

struct DeviceGuard { // binds `device` for the calling thread, restores the previous one
    int previous = -1;
    bool changed = false;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&previous) == cudaSuccess && previous != device) {
            changed = cudaSetDevice(device) == cudaSuccess;
        }
    }
    ~DeviceGuard() {
        if (changed) cudaSetDevice(previous);
    }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct CudaDriver final : Driver {
    EncodeTiledFn encode_tiled = nullptr;

    int device_count(int *count) override { return cudaGetDeviceCount(count); }

    int device_props(int device, int *sm_count, int *cc_major, int *cc_minor, size_t *smem_optin,
                     size_t *l2_bytes) override {
        int value = 0, rc;
        if ((rc = cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device))) return rc;
        *sm_count = value;
        if ((rc = cudaDeviceGetAttribute(&value, cudaDevAttrComputeCapabilityMajor, device))) return rc;
        *cc_major = value;
        if ((rc = cudaDeviceGetAttribute(&value, cudaDevAttrComputeCapabilityMinor, device))) return rc;
        *cc_minor = value;
        if ((rc = cudaDeviceGetAttribute(&value, cudaDevAttrMaxSharedMemoryPerBlockOptin, device))) return rc;
        *smem_optin = (size_t)value;
        if ((rc = cudaDeviceGetAttribute(&value, cudaDevAttrL2CacheSize, device))) return rc;
        *l2_bytes = (size_t)value;
        return 0;
    }

    int stream_device(void *stream, int *device) override {
        // the stream's context decides; resolve it through a capture-safe attribute query
        int rc = cudaStreamGetDevice((cudaStream_t)stream, device);
        if (rc == cudaSuccess) return 0;
        (void)cudaGetLastError();
        return cudaGetDevice(device);
    }

    int pointer_device(const void *ptr, int *device, bool *is_device_memory) override {
        cudaPointerAttributes attributes;
        int rc = cudaPointerGetAttributes(&attributes, ptr);
        if (rc) {
            (void)cudaGetLastError();
            return rc;
        }
        *device = attributes.device;
        *is_device_memory = attributes.type == cudaMemoryTypeDevice ||
                            attributes.type == cudaMemoryTypeManaged;
        return 0;
    }

    int stream_create(int device, void **stream) override {
        DeviceGuard guard(device);
        cudaStream_t created;
        int rc = cudaStreamCreateWithFlags(&created, cudaStreamNonBlocking);
        if (rc == 0) *stream = created;
        return rc;
    }
    int stream_destroy(int device, void *stream) override {
        DeviceGuard guard(device);
        return cudaStreamDestroy((cudaStream_t)stream);
    }
    int stream_sync(void *stream) override { return cudaStreamSynchronize((cudaStream_t)stream); }
    int device_sync(int device) override {
        DeviceGuard guard(device);
        return cudaDeviceSynchronize();
    }
    int event_create(int device, bool timing, void **event) override {
        DeviceGuard guard(device);
        cudaEvent_t created;
        int rc = cudaEventCreateWithFlags(&created, timing ? cudaEventDefault : cudaEventDisableTiming);
        if (rc == 0) *event = created;
        return rc;
    }
    int event_destroy(int device, void *event) override {
        DeviceGuard guard(device);
        return cudaEventDestroy((cudaEvent_t)event);
    }
    int event_record(void *event, void *stream) override {
        return cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream);
    }
    int event_query(void *event, bool *complete) override {
        int rc = cudaEventQuery((cudaEvent_t)event);
        if (rc == cudaErrorNotReady) {
            (void)cudaGetLastError();
            *complete = false;
            return 0;
        }
        *complete = rc == cudaSuccess;
        return rc;
    }
    int event_sync(void *event) override { return cudaEventSynchronize((cudaEvent_t)event); }
    int event_elapsed_ms(void *start, void *end, float *ms) override {
        return cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)end);
    }
    int configure(int device, const std::function<int()> &fn) override {
        DeviceGuard guard(device);
        // Set-up calls (allocation, free, memset) are "potentially unsafe" to a stream capture
        // running in this thread and would invalidate it; a destructor may well run there (a
        // garbage collector finalising an old provider while a Graph is being recorded).  They
        // touch nothing the capture records, so they run in relaxed mode.
        cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
        cudaThreadExchangeStreamCaptureMode(&mode);
        const int rc = fn();
        cudaThreadExchangeStreamCaptureMode(&mode);
        return rc;
    }
    int launch(int device, const std::function<int()> &fn) override {
        DeviceGuard guard(device);
        int rc = fn();
        if (rc == 0) g_launches.fetch_add(1, std::memory_order_relaxed);
        return rc;
    }
    int external(int device, const std::function<int()> &fn) override {
        DeviceGuard guard(device);
        return fn();
    }
    int device_clock_khz(int device, int *khz) override {
        return cudaDeviceGetAttribute(khz, cudaDevAttrClockRate, device);
    }
    int capture_begin(int device, void *stream) override {
        DeviceGuard guard(device);
        return cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal);
    }
    int capture_end(int device, void *stream, void **graph) override {
        DeviceGuard guard(device);
        cudaGraph_t captured = nullptr;
        int rc = cudaStreamEndCapture((cudaStream_t)stream, &captured);
        *graph = captured;
        return rc;
    }
    int capture_status(void *stream, bool *capturing) override {
        cudaStreamCaptureStatus status;
        int rc = cudaStreamIsCapturing((cudaStream_t)stream, &status);
        *capturing = rc == 0 && status != cudaStreamCaptureStatusNone;
        return rc;
    }
    int graph_instantiate(int device, void *graph, void **exec) override {
        DeviceGuard guard(device);
        cudaGraphExec_t instantiated = nullptr;
        int rc = cudaGraphInstantiateWithFlags(&instantiated, (cudaGraph_t)graph, 0);
        *exec = instantiated;
        return rc;
    }
    int graph_launch(int device, void *exec, void *stream) override {
        DeviceGuard guard(device);
        return cudaGraphLaunch((cudaGraphExec_t)exec, (cudaStream_t)stream);
    }
    int graph_destroy(int device, void *graph) override {
        DeviceGuard guard(device);
        return cudaGraphDestroy((cudaGraph_t)graph);
    }
    int graph_exec_destroy(int device, void *exec) override {
        DeviceGuard guard(device);
        return cudaGraphExecDestroy((cudaGraphExec_t)exec);
    }

    int encode_tensor_map_3d(int device, void *map, const void *base, const uint64_t dims[3],
                             const uint64_t strides_bytes[2], const uint32_t box[3]) override {
        DeviceGuard guard(device);
        if (!encode_tiled) {
            void *entry = nullptr;
            cudaDriverEntryPointQueryResult query;
            int rc = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault,
                                             &query);
            if (rc) return rc;
            if (query != cudaDriverEntryPointSuccess || !entry) return cudaErrorNotSupported;
            encode_tiled = (EncodeTiledFn)entry;
        }
        const cuuint64_t global_dims[3] = {dims[0], dims[1], dims[2]};
        const cuuint64_t global_strides[2] = {strides_bytes[0], strides_bytes[1]};
        const cuuint32_t box_dims[3] = {box[0], box[1], box[2]};
        const cuuint32_t element_strides[3] = {1, 1, 1};
        CUresult result = encode_tiled(
            (CUtensorMap *)map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base),
            global_dims, global_strides, box_dims, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return result == CUDA_SUCCESS ? 0 : cudaErrorInvalidValue;
    }

    bool is_fake() const override { return false; }
    uint64_t launch_count() const override { return g_launches.load(); }
};

// ---- fake -------------------------------------------------------------------------------------

struct FakeDriver final : Driver {
    int sm_count = 148;
    std::map<std::string, std::pair<int, int>> armed; // what -> (countdown, error)
    uint64_t launches = 0;
    uintptr_t next_handle = 0x1000;
    std::map<void *, bool> capturing;

    int hit(const char *what) {
        auto it = armed.find(what);
        if (it == armed.end()) return 0;
        if (--it->second.first > 0) return 0;
        const int error = it->second.second;
        armed.erase(it);
        return error;
    }
    void *handle() { return (void *)(next_handle += 0x10); }

    int device_count(int *count) override { *count = 2; return 0; }
    int device_props(int, int *sm, int *major, int *minor, size_t *smem, size_t *l2) override {
        *sm = sm_count; *major = 10; *minor = 0; *smem = 232448; *l2 = 126u << 20;
        return 0;
    }
    // fake streams encode their device in bit 3 of the handle value (0x100 -> 0, 0x108 -> 1)
    int stream_device(void *stream, int *device) override {
        *device = (int)(((uintptr_t)stream >> 3) & 1);
        return 0;
    }
    // fake device pointers: bit 40 set marks "device 1", bit 41 marks "host memory"
    int pointer_device(const void *ptr, int *device, bool *is_device) override {
        const uintptr_t value = (uintptr_t)ptr;
        *device = (int)((value >> 40) & 1);
        *is_device = ((value >> 41) & 1) == 0;
        return 0;
    }
    int stream_create(int device, void **stream) override {
        uintptr_t value = (uintptr_t)handle() & ~(uintptr_t)0xf;
        value |= (uintptr_t)(device & 1) << 3;
        *stream = (void *)value;
        return 0;
    }
    int stream_destroy(int, void *) override { return 0; }
    int stream_sync(void *) override { return hit("stream_sync"); }
    int device_sync(int) override { return hit("device_sync"); }
    int event_create(int, bool, void **event) override { *event = handle(); return hit("event_create"); }
    int event_destroy(int, void *) override { return 0; }
    int event_record(void *, void *) override { return hit("event_record"); }
    int event_query(void *, bool *complete) override { *complete = true; return hit("event_query"); }
    int event_sync(void *) override { return hit("event_sync"); }
    int event_elapsed_ms(void *, void *, float *ms) override { *ms = 0.001f; return 0; }
    int configure(int, const std::function<int()> &) override { return hit("configure"); }
    int launch(int, const std::function<int()> &) override {
        const int error = hit("launch");
        if (error == 0) ++launches;
        return error;
    }
    int external(int, const std::function<int()> &) override { return hit("external"); }
    int device_clock_khz(int, int *khz) override { *khz = 1965000; return 0; }
    int capture_begin(int, void *stream) override {
        const int error = hit("capture_begin");
        if (error == 0) capturing[stream] = true;
        return error;
    }
    int capture_end(int, void *stream, void **graph) override {
        capturing[stream] = false;
        const int error = hit("capture_end");
        *graph = error ? nullptr : handle();
        return error;
    }
    int capture_status(void *stream, bool *is_capturing) override {
        *is_capturing = capturing[stream];
        return 0;
    }
    int graph_instantiate(int, void *, void **exec) override {
        const int error = hit("instantiate");
        *exec = error ? nullptr : handle();
        return error;
    }
    int graph_launch(int, void *, void *) override { return hit("graph_launch"); }
    int graph_destroy(int, void *) override { return 0; }
    int graph_exec_destroy(int, void *) override { return 0; }
    int encode_tensor_map_3d(int, void *map, const void *, const uint64_t *, const uint64_t *,
                             const uint32_t *) override {
        memset(map, 0, 128);
        return hit("encode");
    }
    bool is_fake() const override { return true; }
    uint64_t launch_count() const override { return launches; }
};

CudaDriver g_cuda;
FakeDriver g_fake;
Driver *g_active = &g_cuda;

} // namespace

Driver &driver() { return *g_active; }

void use_fake_driver(bool enable, int sm_count) {
    if (enable) {
        g_fake.armed.clear();
        g_fake.capturing.clear();
        g_fake.launches = 0;
        if (sm_count > 0) g_fake.sm_count = sm_count;
        g_active = &g_fake;
    } else {
        g_active = &g_cuda;
    }
}

void fake_fail(const char *what, int n, int cuda_error) {
    g_fake.armed[what] = std::make_pair(n, cuda_error);
}

int synchronize_stream_or_abort(void *stream, int device) {
    Driver &d = driver();
    const int stream_error = d.stream_sync(stream);
    if (stream_error == 0) return 0;
    const int context_error = d.device_sync(device);
    if (context_error == 0) return stream_error;
    fprintf(stderr,
            "loom_b200 cannot confirm CUDA quiescence after stream and context synchronization "
            "failed; aborting to preserve resource safety: stream=%d; context=%d\n",
            stream_error, context_error);
    abort();
}

} // namespace lb

extern "C" {
void lb_test_use_fake_driver(int enable, int fake_sm_count) {
    lb::use_fake_driver(enable != 0, fake_sm_count);
}
void lb_test_fake_fail(const char *what, int n, int cuda_error) {
    if (what) lb::fake_fail(what, n, cuda_error);
}
uint64_t lb_test_launch_count(void) { return lb::driver().launch_count(); }
}
