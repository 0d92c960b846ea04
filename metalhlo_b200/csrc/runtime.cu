// Device, memory, stream and event entry points of libmhlo_cuda.so plus the thread-local error slot.
// They stand where IntegratedExecutor uses MTLDevice/MTLBuffer/MTLCommandBuffer
// (Sources/MetalHLOCore/Runtime/IntegratedExecutor.swift:106-141,182-190,232-252).
#include <atomic>
#include <cstring>

#include <cstdlib>

#include "common.cuh"

namespace mhlo {

bool dependent_launch_enabled() {
    static const bool on = [] {
        const char* v = getenv("METALHLO_PDL");
        return v != nullptr && v[0] == '1';
    }();
    return on;
}

static thread_local char g_error[1024] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

void clear_error() { g_error[0] = '\0'; }

}  // namespace mhlo

using mhlo::fail;

extern "C" {

const char* mhlo_cuda_version(void) { return "mhlo-cuda 0.1.0 sm_100a"; }

const char* mhlo_cuda_last_error(void) { return mhlo::g_error; }

size_t mhlo_cuda_dtype_size(int dtype) {
    switch (dtype) {
        case MHLO_DT_F16: case MHLO_DT_BF16: case MHLO_DT_I16: case MHLO_DT_UI16: return 2;
        case MHLO_DT_F32: case MHLO_DT_I32: case MHLO_DT_UI32: return 4;
        case MHLO_DT_F64: case MHLO_DT_I64: case MHLO_DT_UI64: return 8;
        case MHLO_DT_I1: case MHLO_DT_I8: case MHLO_DT_UI8: return 1;
        default: return 0;
    }
}

int mhlo_cuda_device_count(int* out_count) {
    if (!out_count) return fail(MHLO_CUDA_INVALID_ARGUMENT, "device_count: null output");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *out_count = 0;
        return fail(MHLO_CUDA_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    }
    *out_count = n;
    return MHLO_CUDA_OK;
}

int mhlo_cuda_device_set(int ordinal) {
    MHLO_CUDA_TRY(cudaSetDevice(ordinal), MHLO_CUDA_NO_DEVICE);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_device_current(int* out_ordinal) {
    if (!out_ordinal) return fail(MHLO_CUDA_INVALID_ARGUMENT, "device_current: null output");
    MHLO_CUDA_TRY(cudaGetDevice(out_ordinal), MHLO_CUDA_NO_DEVICE);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_device_name(int ordinal, char* out_name, size_t cap) {
    if (!out_name || cap == 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "device_name: no output buffer");
    cudaDeviceProp prop;
    MHLO_CUDA_TRY(cudaGetDeviceProperties(&prop, ordinal), MHLO_CUDA_NO_DEVICE);
    snprintf(out_name, cap, "%s", prop.name);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_graph_capture_begin(mhlo_cuda_stream_t stream) {
    if (stream == nullptr) return fail(MHLO_CUDA_INVALID_ARGUMENT, "graph_capture_begin: the default stream cannot be captured");
    // a stream the caller is already recording (its own graph) is left alone: the launches simply join that recording
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    MHLO_CUDA_TRY(cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &status), MHLO_CUDA_UNSUPPORTED);
    if (status != cudaStreamCaptureStatusNone) return fail(MHLO_CUDA_UNSUPPORTED, "graph_capture_begin: the stream is already being captured");
    // thread-local mode: other threads of the process may keep allocating and synchronising while this one records
    MHLO_CUDA_TRY(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal), MHLO_CUDA_UNSUPPORTED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_graph_capture_end(mhlo_cuda_stream_t stream, void** out_graph) {
    if (!out_graph) return fail(MHLO_CUDA_INVALID_ARGUMENT, "graph_capture_end: null output");
    *out_graph = nullptr;
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &graph);
    if (e != cudaSuccess || graph == nullptr) {
        cudaGetLastError();  // the capture was invalidated by something that cannot be recorded
        if (graph) cudaGraphDestroy(graph);
        return fail(MHLO_CUDA_UNSUPPORTED, "graph_capture_end: %s", cudaGetErrorString(e));
    }
    cudaGraphExec_t exec = nullptr;
    const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) {
        cudaGetLastError();
        return fail(MHLO_CUDA_UNSUPPORTED, "graph_capture_end: instantiate: %s", cudaGetErrorString(ie));
    }
    *out_graph = exec;
    return MHLO_CUDA_OK;
}

int mhlo_cuda_graph_launch(void* graph, mhlo_cuda_stream_t stream) {
    if (!graph) return fail(MHLO_CUDA_INVALID_ARGUMENT, "graph_launch: null graph");
    MHLO_CUDA_TRY(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph), static_cast<cudaStream_t>(stream)), MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_graph_destroy(void* graph) {
    if (!graph) return MHLO_CUDA_OK;
    MHLO_CUDA_TRY(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph)), MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_ipc_export(const void* dev_ptr, unsigned char out_handle[64]) {
    if (!dev_ptr || !out_handle) return fail(MHLO_CUDA_INVALID_ARGUMENT, "ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    MHLO_CUDA_TRY(cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr)), MHLO_CUDA_BUFFER_FAILED);
    memcpy(out_handle, &h, sizeof h);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_ipc_open(const unsigned char handle[64], void** out_dev_ptr) {
    if (!handle || !out_dev_ptr) return fail(MHLO_CUDA_INVALID_ARGUMENT, "ipc_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    MHLO_CUDA_TRY(cudaIpcOpenMemHandle(out_dev_ptr, h, cudaIpcMemLazyEnablePeerAccess), MHLO_CUDA_BUFFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_ipc_close(void* dev_ptr) {
    if (!dev_ptr) return MHLO_CUDA_OK;
    MHLO_CUDA_TRY(cudaIpcCloseMemHandle(dev_ptr), MHLO_CUDA_BUFFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_stream_create(mhlo_cuda_stream_t* out_stream) {
    if (!out_stream) return fail(MHLO_CUDA_INVALID_ARGUMENT, "stream_create: null output");
    cudaStream_t s;
    MHLO_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), MHLO_CUDA_NO_DEVICE);
    *out_stream = s;
    return MHLO_CUDA_OK;
}

int mhlo_cuda_stream_destroy(mhlo_cuda_stream_t stream) {
    MHLO_CUDA_TRY(cudaStreamDestroy(static_cast<cudaStream_t>(stream)), MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_stream_sync(mhlo_cuda_stream_t stream) {
    MHLO_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

// Test hook: the next `count` device allocations are refused before they reach the driver.
static std::atomic<int> g_refuse_allocs{0};

int mhlo_cuda_debug_refuse_allocs(int32_t count) {
    g_refuse_allocs.store(count < 0 ? 0 : count);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_alloc(size_t bytes, void** out_dev) {
    if (!out_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "alloc: null output");
    *out_dev = nullptr;
    if (bytes == 0) return MHLO_CUDA_OK;
    int left = g_refuse_allocs.load();
    while (left > 0 && !g_refuse_allocs.compare_exchange_weak(left, left - 1)) {}
    if (left > 0) return fail(MHLO_CUDA_BUFFER_FAILED, "alloc of %zu bytes refused (test hook)", bytes);
    MHLO_CUDA_TRY(cudaMalloc(out_dev, bytes), MHLO_CUDA_BUFFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_free(void* dev) {
    if (!dev) return MHLO_CUDA_OK;
    MHLO_CUDA_TRY(cudaFree(dev), MHLO_CUDA_BUFFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_host_alloc(size_t bytes, void** out_host) {
    if (!out_host) return fail(MHLO_CUDA_INVALID_ARGUMENT, "host_alloc: null output");
    *out_host = nullptr;
    if (bytes == 0) return MHLO_CUDA_OK;
    MHLO_CUDA_TRY(cudaMallocHost(out_host, bytes), MHLO_CUDA_BUFFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_host_free(void* host) {
    if (!host) return MHLO_CUDA_OK;
    MHLO_CUDA_TRY(cudaFreeHost(host), MHLO_CUDA_BUFFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_upload(void* dst_dev, const void* src_host, size_t bytes, mhlo_cuda_stream_t stream) {
    if (bytes == 0) return MHLO_CUDA_OK;
    if (!dst_dev || !src_host) return fail(MHLO_CUDA_INVALID_ARGUMENT, "upload: null pointer");
    MHLO_CUDA_TRY(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice,
                                  static_cast<cudaStream_t>(stream)),
                  MHLO_CUDA_TRANSFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_download(void* dst_host, const void* src_dev, size_t bytes, mhlo_cuda_stream_t stream) {
    if (bytes == 0) return MHLO_CUDA_OK;
    if (!dst_host || !src_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "download: null pointer");
    MHLO_CUDA_TRY(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost,
                                  static_cast<cudaStream_t>(stream)),
                  MHLO_CUDA_TRANSFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_copy(void* dst_dev, const void* src_dev, size_t bytes, mhlo_cuda_stream_t stream) {
    if (bytes == 0) return MHLO_CUDA_OK;
    if (!dst_dev || !src_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "copy: null pointer");
    MHLO_CUDA_TRY(cudaMemcpyAsync(dst_dev, src_dev, bytes, cudaMemcpyDeviceToDevice,
                                  static_cast<cudaStream_t>(stream)),
                  MHLO_CUDA_TRANSFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_memset(void* dst_dev, int byte_value, size_t bytes, mhlo_cuda_stream_t stream) {
    if (bytes == 0) return MHLO_CUDA_OK;
    if (!dst_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "memset: null pointer");
    MHLO_CUDA_TRY(cudaMemsetAsync(dst_dev, byte_value, bytes, static_cast<cudaStream_t>(stream)),
                  MHLO_CUDA_TRANSFER_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_event_create(void** out_event) {
    if (!out_event) return fail(MHLO_CUDA_INVALID_ARGUMENT, "event_create: null output");
    cudaEvent_t e;
    MHLO_CUDA_TRY(cudaEventCreate(&e), MHLO_CUDA_NO_DEVICE);
    *out_event = e;
    return MHLO_CUDA_OK;
}

int mhlo_cuda_event_destroy(void* event) {
    if (!event) return MHLO_CUDA_OK;
    MHLO_CUDA_TRY(cudaEventDestroy(static_cast<cudaEvent_t>(event)), MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_event_record(void* event, mhlo_cuda_stream_t stream) {
    MHLO_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)),
                  MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_event_sync(void* event) {
    if (!event) return fail(MHLO_CUDA_INVALID_ARGUMENT, "event_sync: null event");
    MHLO_CUDA_TRY(cudaEventSynchronize(static_cast<cudaEvent_t>(event)), MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_stream_wait_event(mhlo_cuda_stream_t stream, void* event) {
    if (!event) return fail(MHLO_CUDA_INVALID_ARGUMENT, "stream_wait_event: null event");
    MHLO_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0), MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_stream_host_callback(mhlo_cuda_stream_t stream, void (*fn)(void*), void* user) {
    if (!fn) return fail(MHLO_CUDA_INVALID_ARGUMENT, "stream_host_callback: null function");
    MHLO_CUDA_TRY(cudaLaunchHostFunc(static_cast<cudaStream_t>(stream), fn, user), MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_event_elapsed_ms(void* start, void* stop, float* out_ms) {
    if (!out_ms) return fail(MHLO_CUDA_INVALID_ARGUMENT, "event_elapsed_ms: null output");
    MHLO_CUDA_TRY(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)), MHLO_CUDA_EXECUTION_FAILED);
    MHLO_CUDA_TRY(cudaEventElapsedTime(out_ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)),
                  MHLO_CUDA_EXECUTION_FAILED);
    return MHLO_CUDA_OK;
}

}  // extern "C"
