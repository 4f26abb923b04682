// runtime.cu — error plumbing, device discovery and the thin memory / stream /
// event wrappers of the C ABI (cf. the reference's HIP driver shim,
// engine/hip/hip_driver_cgo.go:7-670).
#include "common.cuh"

#include <cstring>
#include <mutex>
#include <algorithm>
#include <string>
#include <vector>

namespace lthn {

static thread_local std::string g_err;
static thread_local bool g_pdl = false;
bool pdl_enabled() { return g_pdl; }
void pdl_set(bool on) { g_pdl = on; }

int32_t fail(int32_t code, const std::string& msg) { g_err = msg; return code; }
int32_t cuda_fail(cudaError_t e, const char* what) {
    g_err = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    return LTHN_ERR_CUDA;
}
void clear_error() { g_err.clear(); }

static const int kMaxDev = 16;
static std::mutex g_mu;
static uint32_t* g_status[kMaxDev];
static const int kSlots = 5;
static void* g_scratch[kMaxDev][kSlots];
static size_t g_scratch_bytes[kMaxDev][kSlots];

uint32_t* device_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_status[dev]) {
        if (cudaMalloc((void**)&g_status[dev], 256) != cudaSuccess) return nullptr;
        cudaMemset(g_status[dev], 0, 256);
    }
    return g_status[dev];
}

int32_t check_device_status(cudaStream_t s) {
    uint32_t* w = device_status_word();
    if (!w) return fail(LTHN_ERR_CUDA, "no device status word");
    uint32_t v = 0;
    LTHN_CUDA_TRY(cudaMemcpyAsync(&v, w, 4, cudaMemcpyDeviceToHost, s));
    LTHN_CUDA_TRY(cudaStreamSynchronize(s));
    if (v != 0) {
        cudaMemsetAsync(w, 0, 4, s);
        return fail(LTHN_ERR_DEVICE_WAIT, "a device-side bounded wait ran out (status " + std::to_string(v) + ")");
    }
    return LTHN_OK;
}

// Split form for callers that already have a pinned word and a synchronisation point of their
// own: queue the read, synchronise once for everything, then judge the value.
int32_t device_status_read_async(cudaStream_t s, uint32_t* pinned_dst) {
    uint32_t* w = device_status_word();
    if (!w) return fail(LTHN_ERR_CUDA, "no device status word");
    LTHN_CUDA_TRY(cudaMemcpyAsync(pinned_dst, w, 4, cudaMemcpyDeviceToHost, s));
    return LTHN_OK;
}
int32_t device_status_judge(uint32_t v, cudaStream_t s) {
    if (v == 0) return LTHN_OK;
    uint32_t* w = device_status_word();
    if (w) cudaMemsetAsync(w, 0, 4, s);
    return fail(LTHN_ERR_DEVICE_WAIT, "a device-side bounded wait ran out (status " + std::to_string(v) + ")");
}

// Arenas only grow, and a block that was handed out is never freed while the process lives:
// kernels in flight, captured CUDA graphs and other host threads may still hold its address.
// A request beyond the current size allocates a block of at least twice that size (so the
// retired blocks sum to less than the live one) and keeps the old block until exit.
static std::vector<void*> g_retired;

int32_t scratch_get(size_t bytes, void** out, int slot) {
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev || slot < 0 || slot >= kSlots) return fail(LTHN_ERR_INVALID, "scratch: bad device or slot");
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_scratch_bytes[dev][slot] < bytes) {
        size_t want = std::max(bytes, 2 * g_scratch_bytes[dev][slot]);
        if (want < (size_t)(8u << 20)) want = (size_t)(8u << 20);
        void* p = nullptr;
        LTHN_CUDA_TRY(cudaMalloc(&p, want));
        if (g_scratch[dev][slot]) g_retired.push_back(g_scratch[dev][slot]);
        g_scratch[dev][slot] = p;
        g_scratch_bytes[dev][slot] = want;
    }
    *out = g_scratch[dev][slot];
    return LTHN_OK;
}

// Sticky status words outside the arena (a kernel family that must not allocate keeps its own
// word in a __device__ array and registers it here); read and cleared by lthn_device_status.
static uint32_t* g_extra_status[kMaxDev][4];
void device_status_register(uint32_t* word) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return;
    std::lock_guard<std::mutex> lk(g_mu);
    for (auto& w : g_extra_status[dev]) {
        if (w == word) return;
        if (!w) { w = word; return; }
    }
}

}  // namespace lthn

using namespace lthn;

extern "C" {

const char* lthn_last_error(void) { return g_err.c_str(); }

int32_t lthn_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

int32_t lthn_cuda_available(void) {
    int n = lthn_cuda_device_count();
    for (int i = 0; i < n; i++) {
        cudaDeviceProp p;
        if (cudaGetDeviceProperties(&p, i) == cudaSuccess && p.major == 10) return 1;
    }
    return 0;
}

int32_t lthn_cuda_set_device(int32_t device) {
    clear_error();
    LTHN_CUDA_TRY(cudaSetDevice(device));
    return LTHN_OK;
}

int32_t lthn_cuda_device_info(int32_t device, lthn_device_info* out) {
    clear_error();
    LTHN_REQUIRE(out != nullptr, "lthn_cuda_device_info: out is NULL");
    cudaDeviceProp p;
    LTHN_CUDA_TRY(cudaGetDeviceProperties(&p, device));
    memset(out, 0, sizeof(*out));
    strncpy(out->name, p.name, sizeof(out->name) - 1);
    snprintf(out->architecture, sizeof(out->architecture), "sm_%d%d", p.major, p.minor);
    out->memory_size = p.totalGlobalMem;
    out->max_buffer_length = p.totalGlobalMem;
    out->max_recommended_working_set = (uint64_t)((double)p.totalGlobalMem * 0.9);
    out->sm_count = p.multiProcessorCount;
    out->compute_major = p.major;
    out->compute_minor = p.minor;
    return LTHN_OK;
}

int32_t lthn_cuda_mem_info(uint64_t* free_bytes, uint64_t* total_bytes) {
    clear_error();
    size_t f = 0, t = 0;
    LTHN_CUDA_TRY(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return LTHN_OK;
}

// Reads and clears every sticky device status word of the current device after synchronising
// `stream`: the arena word the asynchronous entry points report into (only if one exists) and
// the words of allocation-free entry points. Four-byte copies into host memory: allocates
// nothing on the device.
int32_t lthn_device_status(void* stream, uint32_t* bits) {
    clear_error();
    cudaStream_t s = (cudaStream_t)stream;
    int dev = 0;
    LTHN_CUDA_TRY(cudaGetDevice(&dev));
    LTHN_REQUIRE(dev >= 0 && dev < kMaxDev, "lthn_device_status: device index out of range");
    uint32_t* words[5];
    int n = 0;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (g_status[dev]) words[n++] = g_status[dev];
        for (uint32_t* w : g_extra_status[dev]) if (w) words[n++] = w;
    }
    LTHN_CUDA_TRY(cudaStreamSynchronize(s));
    uint32_t all = 0;
    for (int i = 0; i < n; i++) {
        uint32_t v = 0;
        LTHN_CUDA_TRY(cudaMemcpyAsync(&v, words[i], 4, cudaMemcpyDeviceToHost, s));
        LTHN_CUDA_TRY(cudaStreamSynchronize(s));
        if (v) {
            LTHN_CUDA_TRY(cudaMemsetAsync(words[i], 0, 4, s));
            LTHN_CUDA_TRY(cudaStreamSynchronize(s));
        }
        all |= v;
    }
    if (bits) *bits = all;
    if (all) return fail(LTHN_ERR_DEVICE_WAIT, "a device-side bounded wait ran out (status " + std::to_string(all) + ")");
    return LTHN_OK;
}

int32_t lthn_malloc(void** dptr, size_t bytes) {
    clear_error();
    LTHN_REQUIRE(dptr != nullptr, "lthn_malloc: dptr is NULL");
    *dptr = nullptr;
    if (bytes == 0) return LTHN_OK;
    LTHN_CUDA_TRY(cudaMalloc(dptr, bytes));
    return LTHN_OK;
}
int32_t lthn_free(void* dptr) {
    clear_error();
    if (dptr) LTHN_CUDA_TRY(cudaFree(dptr));
    return LTHN_OK;
}
int32_t lthn_host_alloc(void** hptr, size_t bytes) {
    clear_error();
    LTHN_REQUIRE(hptr != nullptr, "lthn_host_alloc: hptr is NULL");
    *hptr = nullptr;
    if (bytes == 0) return LTHN_OK;
    LTHN_CUDA_TRY(cudaHostAlloc(hptr, bytes, cudaHostAllocDefault));
    return LTHN_OK;
}
int32_t lthn_host_free(void* hptr) {
    clear_error();
    if (hptr) LTHN_CUDA_TRY(cudaFreeHost(hptr));
    return LTHN_OK;
}
int32_t lthn_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
    clear_error();
    if (bytes == 0) return LTHN_OK;
    LTHN_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return LTHN_OK;
}
int32_t lthn_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
    clear_error();
    if (bytes == 0) return LTHN_OK;
    LTHN_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    LTHN_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return LTHN_OK;
}
int32_t lthn_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream) {
    clear_error();
    if (bytes == 0) return LTHN_OK;
    LTHN_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return LTHN_OK;
}
int32_t lthn_memset(void* dst, int32_t value, size_t bytes, void* stream) {
    clear_error();
    if (bytes == 0) return LTHN_OK;
    LTHN_CUDA_TRY(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
    return LTHN_OK;
}
int32_t lthn_stream_create(void** stream) {
    clear_error();
    LTHN_REQUIRE(stream != nullptr, "lthn_stream_create: stream is NULL");
    cudaStream_t s;
    LTHN_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = (void*)s;
    return LTHN_OK;
}
int32_t lthn_stream_destroy(void* stream) {
    clear_error();
    if (stream) LTHN_CUDA_TRY(cudaStreamDestroy((cudaStream_t)stream));
    return LTHN_OK;
}
int32_t lthn_stream_sync(void* stream) {
    clear_error();
    LTHN_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return LTHN_OK;
}
int32_t lthn_device_sync(void) {
    clear_error();
    LTHN_CUDA_TRY(cudaDeviceSynchronize());
    return LTHN_OK;
}
int32_t lthn_event_create(void** event) {
    clear_error();
    LTHN_REQUIRE(event != nullptr, "lthn_event_create: event is NULL");
    cudaEvent_t e;
    LTHN_CUDA_TRY(cudaEventCreate(&e));
    *event = (void*)e;
    return LTHN_OK;
}
int32_t lthn_event_destroy(void* event) {
    clear_error();
    if (event) LTHN_CUDA_TRY(cudaEventDestroy((cudaEvent_t)event));
    return LTHN_OK;
}
int32_t lthn_event_record(void* event, void* stream) {
    clear_error();
    LTHN_CUDA_TRY(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
    return LTHN_OK;
}
int32_t lthn_event_elapsed_ms(void* start, void* stop, float* ms) {
    clear_error();
    LTHN_REQUIRE(ms != nullptr, "lthn_event_elapsed_ms: ms is NULL");
    LTHN_CUDA_TRY(cudaEventSynchronize((cudaEvent_t)stop));
    LTHN_CUDA_TRY(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return LTHN_OK;
}

int32_t lthn_graph_begin(void* stream) {
    clear_error();
    LTHN_REQUIRE(stream != nullptr, "lthn_graph_begin: capture needs a created stream, not the default stream");
    LTHN_CUDA_TRY(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
    return LTHN_OK;
}
int32_t lthn_graph_end(void* stream, void** graph_exec) {
    clear_error();
    LTHN_REQUIRE(graph_exec != nullptr, "lthn_graph_end: graph_exec is NULL");
    cudaGraph_t g = nullptr;
    LTHN_CUDA_TRY(cudaStreamEndCapture((cudaStream_t)stream, &g));
    cudaGraphExec_t ex = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    *graph_exec = (void*)ex;
    return LTHN_OK;
}
int32_t lthn_graph_launch(void* graph_exec, void* stream) {
    clear_error();
    LTHN_CUDA_TRY(cudaGraphLaunch((cudaGraphExec_t)graph_exec, (cudaStream_t)stream));
    return LTHN_OK;
}
int32_t lthn_graph_destroy(void* graph_exec) {
    clear_error();
    if (graph_exec) LTHN_CUDA_TRY(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
    return LTHN_OK;
}

}  // extern "C"
