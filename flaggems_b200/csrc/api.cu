// Library-wide state of the C ABI: error text, device status word, launch counter.
#include <stdarg.h>
#include <atomic>
#include <string.h>

#include "common.cuh"

static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

__device__ unsigned int g_fg_status = 0;

void fg_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

void fg_count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

unsigned int* fg_status_word_device_ptr() {
    // One symbol address per device; looked up lazily for the current device.
    static unsigned int* ptrs[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_fg_status) != cudaSuccess) return nullptr;
        ptrs[dev] = (unsigned int*)p;
    }
    return ptrs[dev];
}

int fg_device_index() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
    return dev > 63 ? 63 : dev;
}

int fg_num_sms() {
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        sms[dev] = v;
    }
    return sms[dev];
}

extern "C" {

int fg_version(void) { return 100; }

const char* fg_last_error(void) { return g_err; }

uint64_t fg_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int fg_device_status(unsigned int* status) {
    FG_REQUIRE(status != nullptr, FG_ERR_INVALID_ARGUMENT, "status must not be NULL");
    unsigned int v = 0, zero = 0;
    FG_CUDA(cudaDeviceSynchronize());
    FG_CUDA(cudaMemcpyFromSymbol(&v, g_fg_status, sizeof(v)));
    if (v != 0) FG_CUDA(cudaMemcpyToSymbol(g_fg_status, &zero, sizeof(zero)));
    *status = v;
    if (v != 0) {
        fg_set_error("device status 0x%08x: %s (code %u, site %u)", v,
                     (v >> 16) == 2u ? "a row of the expert-parallel exchange was addressed outside its buffer and dropped"
                                     : "a bounded wait inside a kernel ran out",
                     v >> 16, v & 0xffffu);
        return FG_ERR_DEVICE_STATUS;
    }
    return FG_OK;
}

// ---- buffers shared between the ranks of one node (CUDA IPC) -------------------------------
int fg_symm_alloc(int64_t bytes, void** ptr, unsigned char* handle64) {
    FG_REQUIRE(bytes > 0 && ptr && handle64, FG_ERR_INVALID_ARGUMENT, "bad arguments");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    FG_CUDA(cudaMalloc(&p, (size_t)bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        fg_set_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
        return FG_ERR_CUDA;
    }
    memcpy(handle64, &h, 64);
    *ptr = p;
    return FG_OK;
}

int fg_symm_open(const unsigned char* handle64, void** ptr) {
    FG_REQUIRE(handle64 && ptr, FG_ERR_INVALID_ARGUMENT, "bad arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    FG_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return FG_OK;
}

int fg_symm_close(void* ptr) {
    FG_CUDA(cudaIpcCloseMemHandle(ptr));
    return FG_OK;
}

int fg_symm_free(void* ptr) {
    FG_CUDA(cudaFree(ptr));
    return FG_OK;
}

}  // extern "C"
