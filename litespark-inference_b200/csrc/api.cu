// Library state: device selection, stream, sticky error record, memory and timing helpers.
#include <stdarg.h>
#include <string.h>
#include <stdlib.h>
#include <mutex>

#include "common.cuh"

namespace lspk {

static std::mutex g_mu;
static char g_err[1024] = "";
static int g_err_count = 0;
static int g_device = -1;
static int g_sm_count = 0;
static cudaStream_t g_stream = nullptr;
static bool g_pdl = true;
static cudaEvent_t g_ev0 = nullptr, g_ev1 = nullptr;
static void* g_flush_buf = nullptr;
static const size_t kFlushBytes = 256u << 20;   // twice the 126 MB L2

void set_error(const char* fmt, ...) {
    std::lock_guard<std::mutex> lk(g_mu);
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    ++g_err_count;
}

int fail(int code, const char* fmt, ...) {
    std::lock_guard<std::mutex> lk(g_mu);
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    ++g_err_count;
    return code;
}

static unsigned long long* g_trace = nullptr;
static int g_trace_cap = 0;
unsigned long long* trace_buffer() { return g_trace; }
int trace_capacity() { return g_trace_cap; }

static unsigned g_scratch_gen = 1;
unsigned scratch_generation() { return g_scratch_gen; }
void scratch_moved() { ++g_scratch_gen; }

static cudaStream_t g_stream_override = nullptr;    // measurement aid: launches go here while set
cudaStream_t stream() { return g_stream_override ? g_stream_override : g_stream; }
cudaStream_t main_stream() { return g_stream; }
void set_stream_override(cudaStream_t s) { g_stream_override = s; }
bool pdl_enabled() { return g_pdl; }
int sm_count() { return g_sm_count; }

// Word that kernels with bounded waits set when a wait runs out.  It is part of the library image (zero when
// the module is loaded), so binding to a device allocates nothing; its device address is looked up once.
static __device__ int g_wait_flag_word[4];
static int* g_wait_flag = nullptr;
int* device_wait_flag() { return g_wait_flag; }
int bound_device() { return g_device; }

// Lazily bind to a device the first time any entry point needs one.

int ensure_init() {
    if (g_device >= 0) return LSPK_OK;
    const char* env = getenv("LITESPARK_DEVICE");
    return lspk_init(env ? atoi(env) : 0);
}

}  // namespace lspk

using namespace lspk;

extern "C" {

int lspk_init(int device) {
    if (g_device == device && g_stream) return LSPK_OK;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return fail(LSPK_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    if (device < 0 || device >= n) return fail(LSPK_ERR_ARG, "device %d out of range (have %d)", device, n);
    cudaDeviceProp prop;
    LSPK_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(LSPK_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                    device, prop.major, prop.minor);
    if (g_device >= 0 && g_device != device)
        return fail(LSPK_ERR_STATE, "library already bound to device %d", g_device);
    LSPK_CUDA(cudaSetDevice(device));
    // Nothing below allocates device memory.  Either every object exists and the library is bound, or none
    // is kept and a later call starts again from a clean state.
    cudaStream_t st = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    void* flag = nullptr;
    e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&flag, g_wait_flag_word);
    if (e != cudaSuccess) {
        if (e1) cudaEventDestroy(e1);
        if (e0) cudaEventDestroy(e0);
        if (st) cudaStreamDestroy(st);
        return fail(LSPK_ERR_CUDA, "lspk_init: binding to device %d failed: %s", device, cudaGetErrorString(e));
    }
    g_stream = st;
    g_ev0 = e0;
    g_ev1 = e1;
    g_wait_flag = static_cast<int*>(flag);
    g_sm_count = prop.multiProcessorCount;
    g_device = device;
    const char* p = getenv("LITESPARK_PDL");
    if (p) g_pdl = atoi(p) != 0;
    return LSPK_OK;
}

int lspk_mem_info(size_t* free_bytes, size_t* total_bytes) {
    if (int rc = ensure_init()) return rc;
    size_t f = 0, t = 0;
    LSPK_CUDA(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return LSPK_OK;
}

int lspk_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
    return n;
}

int lspk_sm_count(void) { return ensure_init() == LSPK_OK ? g_sm_count : 0; }

const char* lspk_last_error(void) { return g_err; }
int lspk_error_count(void) { return g_err_count; }
void lspk_clear_error(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_err[0] = 0;
    g_err_count = 0;
}

int lspk_set_pdl(int enabled) {
    g_pdl = enabled != 0;
    return LSPK_OK;
}

int lspk_sync(void) {
    if (int rc = ensure_init()) return rc;
    LSPK_CUDA(cudaStreamSynchronize(g_stream));
    return LSPK_OK;
}

void* lspk_malloc(size_t bytes) {
    if (ensure_init()) return nullptr;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
    if (e != cudaSuccess) {
        fail(LSPK_ERR_CUDA, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
        return nullptr;
    }
    return p;
}

int lspk_free(void* dev) {
    if (!dev) return LSPK_OK;
    LSPK_CUDA(cudaFree(dev));
    return LSPK_OK;
}

void* lspk_host_alloc(size_t bytes) {
    if (ensure_init()) return nullptr;
    void* p = nullptr;
    cudaError_t e = cudaMallocHost(&p, bytes ? bytes : 16);
    if (e != cudaSuccess) {
        fail(LSPK_ERR_CUDA, "cudaMallocHost(%zu) failed: %s", bytes, cudaGetErrorString(e));
        return nullptr;
    }
    return p;
}

int lspk_host_free(void* host) {
    if (!host) return LSPK_OK;
    LSPK_CUDA(cudaFreeHost(host));
    return LSPK_OK;
}

int lspk_h2d_async(void* dev, const void* host, size_t bytes) {
    if (int rc = ensure_init()) return rc;
    LSPK_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, g_stream));
    return LSPK_OK;
}
int lspk_d2h_async(void* host, const void* dev, size_t bytes) {
    if (int rc = ensure_init()) return rc;
    LSPK_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, g_stream));
    return LSPK_OK;
}
int lspk_h2d(void* dev, const void* host, size_t bytes) {
    if (int rc = lspk_h2d_async(dev, host, bytes)) return rc;
    LSPK_CUDA(cudaStreamSynchronize(g_stream));
    return LSPK_OK;
}
int lspk_d2h(void* host, const void* dev, size_t bytes) {
    if (int rc = lspk_d2h_async(host, dev, bytes)) return rc;
    LSPK_CUDA(cudaStreamSynchronize(g_stream));
    return LSPK_OK;
}
int lspk_memset(void* dev, int value, size_t bytes) {
    if (int rc = ensure_init()) return rc;
    LSPK_CUDA(cudaMemsetAsync(dev, value, bytes, g_stream));
    return LSPK_OK;
}

int lspk_flush_l2(void) {
    if (int rc = ensure_init()) return rc;
    if (!g_flush_buf) LSPK_CUDA(cudaMalloc(&g_flush_buf, kFlushBytes));
    static int v = 0;
    LSPK_CUDA(cudaMemsetAsync(g_flush_buf, ++v & 0xff, kFlushBytes, g_stream));
    return LSPK_OK;
}

// Install a device buffer for in-kernel phase traces.  Kernels launched (or captured into a graph)
// afterwards record into it; lspk_trace_read copies the records out and resets the counter.
int lspk_trace_begin(int max_records) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(max_records >= 1, "lspk_trace_begin: max_records must be positive");
    // A buffer that is large enough is kept (only its counter is cleared): graphs captured while it was
    // installed hold its address.  A larger one replaces it; such graphs must then be rebuilt by their owner.
    if (g_trace && max_records <= g_trace_cap) {
        LSPK_CUDA(cudaDeviceSynchronize());
        LSPK_CUDA(cudaMemset(g_trace, 0, 8));
        LSPK_CUDA(cudaDeviceSynchronize());
        return LSPK_OK;
    }
    if (g_trace) {
        LSPK_CUDA(cudaDeviceSynchronize());
        cudaFree(g_trace);
    }
    g_trace = nullptr;
    g_trace_cap = 0;
    const size_t bytes = (1 + (size_t)max_records * kTraceWords) * 8;
    LSPK_CUDA(cudaMalloc((void**)&g_trace, bytes));
    LSPK_CUDA(cudaMemset(g_trace, 0, bytes));
    LSPK_CUDA(cudaDeviceSynchronize());
    g_trace_cap = max_records;
    return LSPK_OK;
}

int lspk_trace_read(unsigned long long* host_out, int max_records, int* n_out) {
    LSPK_REQUIRE(g_trace && host_out && n_out, "lspk_trace_read: no trace buffer installed");
    LSPK_CUDA(cudaStreamSynchronize(g_stream));
    unsigned long long n = 0;
    LSPK_CUDA(cudaMemcpy(&n, g_trace, 8, cudaMemcpyDeviceToHost));
    if (n > (unsigned long long)g_trace_cap) n = g_trace_cap;
    if (n > (unsigned long long)max_records) n = max_records;
    LSPK_CUDA(cudaMemcpy(host_out, g_trace + 1, (size_t)n * kTraceWords * 8, cudaMemcpyDeviceToHost));
    LSPK_CUDA(cudaMemset(g_trace, 0, 8));
    *n_out = (int)n;
    return LSPK_OK;
}

int lspk_timer_start(void) {
    if (int rc = ensure_init()) return rc;
    LSPK_CUDA(cudaEventRecord(g_ev0, g_stream));
    return LSPK_OK;
}
int lspk_timer_stop(float* ms_out) {
    if (int rc = ensure_init()) return rc;
    LSPK_CUDA(cudaEventRecord(g_ev1, g_stream));
    LSPK_CUDA(cudaEventSynchronize(g_ev1));
    LSPK_CUDA(cudaEventElapsedTime(ms_out, g_ev0, g_ev1));
    return LSPK_OK;
}

}  // extern "C"
